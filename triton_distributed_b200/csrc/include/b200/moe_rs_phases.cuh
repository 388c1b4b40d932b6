// Top-k reduction + reduce-scatter that follows the down-projection of a tensor-parallel MoE layer, shared by the
// bf16 and the fp8 grouped GEMM kernels (their RS modes end with it).
//
// On entry every CTA of the grid has written its tiles of gemm_out [Tr * world * topk, N] (row = token * topk + k,
// routing weight already applied). The function
//   1. crosses a grid barrier (the k copies of a token come from tiles of different CTAs),
//   2. for every owner rank, starting with the rank after this one, sums the k copies of each of the owner's tokens
//      and stores the row into slot [this rank] of the owner's symmetric buffer, then adds the delivered rows to the
//      owner's counter for this source with a release,
//   3. waits until every source has delivered this rank's Tr rows and sums the `world` slots into rs_out [Tr, N]
//      (with `nvls` the rows stay at their producers and the owner sums them with multimem.ld_reduce through the switch).
// It is called by all threads of all CTAs of a cooperative launch and returns false if a wait ran out (the status
// block then holds the record). Role in the reference: the scatter / top-k reduce / reduce-scatter consumers of
// python/triton_dist/kernels/nvidia/moe_reduce_rs.py:379-601, 816-926.
#pragma once
#include "b200/primitives.cuh"

namespace b200 {

struct MoeRsArgs {
  const void* gemm_out;   // [n_pairs, ldo] 16-bit
  int ldo, N, topk, Tr, Tr_cap, bf16;
  void* slots;            // symmetric [world][Tr_cap][N], the parity buffer of this call
  uint32_t* rs_cnt;       // symmetric u32[world]: rows received per source
  const uint32_t* rs_base;  // local u32[world]: counter values before this call
  void* rs_out;           // [Tr, N]
  uint32_t* barrier_ctr;  // local u32 used by the grid barrier
  int nvls;               // 1: the summed rows stay in this rank's own slots [owner][row]; the owner adds the `world`
                          // copies with multimem.ld_reduce (the switch does the additions, fp32 accumulation)
};

__device__ __forceinline__ uint4 moe_rs_pack8(const float (&acc)[8], bool bf16) {
  return bf16 ? make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]))
              : make_uint4(pack_f16x2(acc[0], acc[1]), pack_f16x2(acc[2], acc[3]), pack_f16x2(acc[4], acc[5]), pack_f16x2(acc[6], acc[7]));
}
__device__ __forceinline__ void moe_rs_add8(float (&acc)[8], const uint4& x, bool bf16) {
  const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = bf16 ? unpack_bf16x2(xs[q]) : unpack_f16x2(xs[q]);
    acc[2 * q] += f.x;
    acc[2 * q + 1] += f.y;
  }
}

__device__ __forceinline__ bool moe_rs_phases(const SymmCtx& ctx, const MoeRsArgs& a, uint32_t epoch) {
  if (!grid_barrier(ctx, a.barrier_ctr, epoch, gridDim.x)) return false;
  const bool bf16 = a.bf16 != 0;
  const int vec_per_row = a.N / 8;
  const uint8_t* out = static_cast<const uint8_t*>(a.gemm_out);
  // phase 2: for every owner (starting after this rank), sum the k copies of each of its tokens and push the row
  for (int s = 1; s <= ctx.world; ++s) {
    int owner = ctx.rank + s;
    if (owner >= ctx.world) owner -= ctx.world;
    int my_rows = 0;
    for (int lrow = blockIdx.x; lrow < a.Tr; lrow += gridDim.x) {
      ++my_rows;
      const int t = owner * a.Tr + lrow;
      uint8_t* rdst;
      if (a.nvls) {  // keep the row here, at the offset of the owner's segment: the owner reads it through the switch
        rdst = static_cast<uint8_t*>(a.slots) + (static_cast<size_t>(owner) * a.Tr_cap + lrow) * a.N * 2;
      } else {
        uint8_t* dst = static_cast<uint8_t*>(a.slots) + (static_cast<size_t>(ctx.rank) * a.Tr_cap + lrow) * a.N * 2;
        rdst = symm_at(ctx, dst, owner);
      }
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const uint8_t* src = out + (static_cast<size_t>(t) * a.topk * a.ldo + v * 8) * 2;
        for (int k0 = 0; k0 < a.topk; k0 += 4) {  // four copies in flight before the first add
          uint4 x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            x[u] = k0 + u < a.topk ? ld_v4_relaxed_sys(src + static_cast<size_t>(k0 + u) * a.ldo * 2) : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int u = 0; u < 4; ++u) moe_rs_add8(acc, x[u], bf16);
        }
        st_v4(rdst + static_cast<size_t>(v) * 16, moe_rs_pack8(acc, bf16));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && my_rows > 0) {
      fence_acq_rel_sys();
      red_add_release_sys(symm_at(ctx, a.rs_cnt + ctx.rank, owner), static_cast<uint32_t>(my_rows));
    }
  }
  // phase 3: this rank's rows have arrived from everyone -> sum the slots
  bool ok = true;
  if (threadIdx.x < ctx.world)
    ok = wait_flag<WaitCmp::GE, true>(ctx, a.rs_cnt + threadIdx.x, a.rs_base[threadIdx.x] + static_cast<uint32_t>(a.Tr),
                                      threadIdx.x, __LINE__);
  if (!__syncthreads_and(ok)) return false;
  const uint8_t* slots = static_cast<const uint8_t*>(a.slots);
  for (int lrow = blockIdx.x; lrow < a.Tr; lrow += gridDim.x) {
    if (a.nvls) {
      const uint8_t* mine = slots + (static_cast<size_t>(ctx.rank) * a.Tr_cap + lrow) * a.N * 2;
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        const uint4 x = bf16 ? multimem_ld_reduce_bf16x8(mc_ptr(ctx, mine + v * 16)) : multimem_ld_reduce_f16x8(mc_ptr(ctx, mine + v * 16));
        st_v4(static_cast<uint8_t*>(a.rs_out) + (static_cast<size_t>(lrow) * a.N + v * 8) * 2, x);
      }
      continue;
    }
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      uint4 x[kMaxRanks];
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)
        x[s] = s < ctx.world ? ld_v4_relaxed_sys(slots + ((static_cast<size_t>(s) * a.Tr_cap + lrow) * a.N + v * 8) * 2)
                             : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) moe_rs_add8(acc, x[s], bf16);
      st_v4(static_cast<uint8_t*>(a.rs_out) + (static_cast<size_t>(lrow) * a.N + v * 8) * 2, moe_rs_pack8(acc, bf16));
    }
  }
  return true;
}

}  // namespace b200
