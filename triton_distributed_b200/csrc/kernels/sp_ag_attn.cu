// All-gather of sequence-sharded K/V straight into global token order, for context-parallel prefill attention.
//
// Every rank holds, for every sequence of the batch, its 1 / world share of the tokens: with zig-zag sharding the
// chunks r and 2 * world - 1 - r of the 2 * world chunks the sequence is cut into (which balances causal work), else
// the r-th of world chunks. One kernel writes every local K row and V row into the row of its GLOBAL position in the
// gathered buffers of all ranks (its own included), so the attention kernel that follows reads each sequence's keys
// as one contiguous, ordered run and needs no index table: the permutation is folded into the gather.
//
// Role in the reference: the copy-engine / NVSHMEM KV all-gather of
// python/triton_dist/kernels/nvidia/sp_ag_attention_intra_node.py:105-183 (which gathers rank-major and leaves the
// zig-zag arithmetic to the attention kernel, :360-371).
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

namespace b200 {

struct SpKvParams {
  const uint4* k_shard;  // [n_local, row_vec]
  const uint4* v_shard;
  uint4* k_full;         // symmetric [>= total_k, row_vec]
  uint4* v_full;
  const int* cu_k;       // [B + 1] first GLOBAL key row of every sequence
  int B, zigzag, row_vec, n_local;
};

// Global row of local token t (the tokens of a rank are concatenated over the sequences in batch order).
__device__ __forceinline__ long long sp_global_row(const SpKvParams& p, int t, int rank, int world) {
  int lo = 0, hi = p.B;  // largest b with cu_k[b] / world <= t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.cu_k[mid] / world <= t) lo = mid; else hi = mid;
  }
  const int start = p.cu_k[lo], len = p.cu_k[lo + 1] - start;
  const int j = t - start / world;
  if (p.zigzag) {
    const int c = len / (2 * world);
    return j < c ? static_cast<long long>(start) + rank * c + j
                 : static_cast<long long>(start) + (2 * world - 1 - rank) * c + (j - c);
  }
  return static_cast<long long>(start) + rank * (len / world) + j;
}

__global__ void __launch_bounds__(256) sp_kv_scatter_kernel(const SpKvParams p, const SymmCtx ctx) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < p.n_local; t += nwarps) {
    const long long g = sp_global_row(p, t, ctx.rank, ctx.world);
    for (int i = lane; i < p.row_vec; i += 32) {
      const uint4 kv = ld_v4_nc(p.k_shard + static_cast<size_t>(t) * p.row_vec + i);
      const uint4 vv = ld_v4_nc(p.v_shard + static_cast<size_t>(t) * p.row_vec + i);
      uint4* kd = p.k_full + g * p.row_vec + i;
      uint4* vd = p.v_full + g * p.row_vec + i;
      for (int k = 0; k < ctx.world; ++k) {
        int peer = ctx.rank + k;
        if (peer >= ctx.world) peer -= ctx.world;
        st_v4(symm_at(ctx, kd, peer), kv);
        st_v4(symm_at(ctx, vd, peer), vv);
      }
    }
  }
  __threadfence_system();
}

}  // namespace b200

using namespace b200;

// k_shard / v_shard: [n_local, row_bytes] contiguous rows of this rank's tokens (row_bytes = kv heads x head dim x
// element size, a multiple of 16); k_full / v_full: symmetric buffers of at least cu_k[B] rows; cu_k int32 [B + 1] on
// the device with every sequence length divisible by 2 * world (zig-zag) or world. The caller brackets the call with
// cross-rank barriers: one after it (the rows of all ranks have landed) and one after the consumer has read them.
B200_API int b200_sp_kv_scatter(const void* symm_ctx, const void* k_shard, const void* v_shard, void* k_full, void* v_full,
                                const int* cu_k, int B, int n_local, int row_bytes, int zigzag, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "row bytes (%d) must be a positive multiple of 16", row_bytes);
  B200_REQUIRE(B >= 1 && n_local >= 0, "bad batch / token count");
  if (n_local == 0) return kOk;
  SpKvParams p;
  memset(&p, 0, sizeof(p));
  p.k_shard = static_cast<const uint4*>(k_shard);
  p.v_shard = static_cast<const uint4*>(v_shard);
  p.k_full = static_cast<uint4*>(k_full);
  p.v_full = static_cast<uint4*>(v_full);
  p.cu_k = cu_k;
  p.B = B; p.zigzag = zigzag; p.row_vec = row_bytes / 16; p.n_local = n_local;
  const int warps_per_cta = 8;
  int grid = (n_local + warps_per_cta - 1) / warps_per_cta;
  if (grid > 4 * sm_count()) grid = 4 * sm_count();
  sp_kv_scatter_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
