// Tutorial 06 - a reduce-scatter written twice: pull from the peers, and let the NVSwitch do the sum.
//
// Every rank holds `partial` [world, n] fp32 in the symmetric heap (row r is its contribution to rank r's result).
// Rank r wants out[i] = sum over ranks s of partial_s[r][i].
//
//   pull      after a barrier (every rank's partials are complete and visible), each thread loads its 16-byte vector
//             of row [rank] from every peer through symm_at (all loads issued before the first add) and sums them in
//             rank order, so the result is the same on every run
//   multimem  one multimem.ld_reduce on the multicast address of row [rank] returns the sum over all ranks: the switch
//             reads the peers and adds; the GPU receives one vector instead of `world`
//
// The reference builds its reduce-scatter from a scatter and a ring reduce on copy engines
// (tutorials/05-intra-node-reduce-scatter.py); inside an NVSwitch node a direct pull needs no ring.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

using namespace b200;

__global__ void __launch_bounds__(512) reduce_scatter_kernel(const SymmCtx ctx, float* partial, float* out, int n, uint32_t* flags, uint32_t epoch,
                                      int use_multimem, uint32_t* ok_out) {
  const bool ok = barrier_all_block(ctx, flags, epoch);
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
  if (!ok) return;
  float* mine = partial + static_cast<size_t>(ctx.rank) * n;  // LOCAL address of row [rank]
  for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (use_multimem) {
      acc = multimem_ld_reduce_f32x4(mc_ptr(ctx, mine + i));
    } else {
      uint4 v[kMaxRanks];
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)
        if (s < ctx.world) v[s] = ld_v4_relaxed_sys(symm_at(ctx, mine + i, s));
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)
        if (s < ctx.world) {
          acc.x += __uint_as_float(v[s].x);
          acc.y += __uint_as_float(v[s].y);
          acc.z += __uint_as_float(v[s].z);
          acc.w += __uint_as_float(v[s].w);
        }
    }
    *reinterpret_cast<float4*>(out + i) = acc;
  }
}

extern "C" __attribute__((visibility("default"))) int tutorial_reduce_scatter(const void* symm_ctx, void* partial, void* out,
                                                                              int n, void* flags, unsigned epoch,
                                                                              int use_multimem, void* ok_out, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  if (n % 4 != 0) return -1;
  if (use_multimem && ctx.mc_base == 0) return -2;  // no NVLS mapping on this heap
  reduce_scatter_kernel<<<1, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      ctx, static_cast<float*>(partial), static_cast<float*>(out), n, static_cast<uint32_t*>(flags), epoch, use_multimem,
      static_cast<uint32_t*>(ok_out));
  return static_cast<int>(cudaGetLastError());
}
