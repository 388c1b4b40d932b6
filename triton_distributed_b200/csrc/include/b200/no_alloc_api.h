// Decode GEMM for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library whose
// calling context forbids cudaMalloc: code running inside a memory pool that owns the whole device,
// plugins called from a serving runtime after its memory plan is frozen, or hosts that pre-size every
// buffer and treat any later allocation as an error.
//
// b200_gemm_skinny_static computes exactly what b200_gemm_skinny computes (same kernel), but the fp32
// split accumulation area and the per-tile tickets live in arrays compiled into the library image
// instead of buffers handed in by the caller. The caller passes only its inputs and its output.
//
// Limits and rules:
//   * capacity: ceil(N / 128) * (dual ? 2 : 1) * roundup(M, 16) * 128 <= 1,048,576 floats (4 MiB) and
//     ceil(N / 128) <= 4096 tiles. Larger problems are rejected with an error; nothing is launched.
//     Every GPU that loads the library holds these 4 MiB + 16 KiB until the process exits.
//   * the first call on each device resolves the device address of the arrays (cudaGetSymbolAddress, with
//     that device current) under a lock, so host threads may race to make it. Make that first call outside of
//     any stream capture.
//   * no call allocates or frees: no cudaMalloc / cudaFree, no allocating library routine.
//   * all calls on a device share the one area. The kernel leaves it zeroed when it finishes, which is what
//     the next call relies on, so two calls that overlap on the GPU (different streams without an ordering
//     between them) race on it and give wrong sums. Serialise them.
//   * if a call was cut short (a device error), call b200_gemm_skinny_static_reset before the next one.
#pragma once
#include <cstdint>

extern "C" {

// X [M, K] (row pitch ldx), W [rows, K] (row pitch ldw), C [M, N] (row pitch ldc); element type `dtype`
// (0 = bf16, 1 = f16). dual == 0: rows = N, C = X W^T. dual == 1: W = [gate (N rows); up (N rows)] and
// C = silu(X gate^T) * (X up^T). 1 <= M <= 256 (<= 128 when dual), K % 8 == 0.
// Returns 0, or an error code whose text b200_last_error() gives.
int b200_gemm_skinny_static(const void* X, const void* W, void* C, int M, int N, int K, int ldx, int ldw, int ldc,
                            int dual, int dtype, void* stream);

// Zero the built-in area of the current device on `stream` (a memset, no allocation).
int b200_gemm_skinny_static_reset(void* stream);

// Capacity of the built-in area in floats (for callers that want to check before calling).
long long b200_gemm_skinny_static_capacity_floats();
}
