// Sequence-parallel decode: merge of the split-KV partials of this rank, exchange of the per-rank (O, LSE)
// partials with the low-latency packet protocol, and the cross-rank LSE combine, in ONE kernel.
//
// Each rank has attended to its own shard of the KV cache (decode_attn.cu). CTA (b, h) then
//   1. merges this rank's split partials of head (b, h) in registers,
//   2. sends the 128 output words and the LSE as {value, epoch} packets to every peer (plain P2P stores, or a
//      single multimem.st per packet when the heap is bound to an NVLS multicast object),
//   3. polls the packets of the other ranks for the same head (the data is its own arrival flag, so there is no
//      barrier and no separate signal), and
//   4. writes softmax-consistent output sum_r exp(lse_r - max) O_r / sum_r exp(lse_r - max); ranks whose shard was
//      empty carry lse = -inf and drop out.
// Packet areas are double-buffered by epoch parity; the epoch lives in device memory (CUDA-graph replayable).
//
// Role in the reference: SpGQAFlashDecodeAttention.forward = intra-rank combine kernel + staged copy into a
// symmetric buffer + LL all-gather kernel + inter-rank combine kernel
// (python/triton_dist/layers/nvidia/sp_flash_decode_layer.py:83-185, kernels/nvidia/flash_decode.py:393-532,
// low_latency_allgather.py:530-566, 762-777).
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/attn_merge.cuh"

#include <cstring>

namespace b200 {

constexpr int kSpD = 128;

struct SpParams {
  const float* o_part;    // [BH, S, 128] split partials of this rank (normalised per split)
  const float* lse_part;  // [BH, S]
  int S, BH;
  uint64_t* ll[2];        // symmetric packet areas [world][BH][129] per parity
  uint32_t* sync;         // local u32[2]
  void* out;              // [BH, 128] bf16 / f16
  float* out_lse;         // [BH] or null
  int bf16, use_mc;
};

__global__ void __launch_bounds__(kSpD) sp_decode_combine_kernel(const SpParams p, const SymmCtx ctx) {
  __shared__ float lse_of[kMaxRanks];
  const uint32_t epoch = epoch_begin(p.sync);
  uint64_t* ll = p.ll[epoch & 1];
  const int bh = blockIdx.x, d = threadIdx.x;
  const int me = ctx.rank, world = ctx.world;
  // 1. local merge over splits
  float o_mine, lse_mine;
  merge_splits(p.lse_part + static_cast<size_t>(bh) * p.S, 1, p.o_part + static_cast<size_t>(bh) * p.S * kSpD + d, kSpD, p.S,
               o_mine, lse_mine);
  // 2. send packets: word d, and the LSE as word 128 (thread 0)
  const size_t base = (static_cast<size_t>(me) * p.BH + bh) * (kSpD + 1);
  if (world > 1) {
    if (p.use_mc) {
      const uint64_t v = (static_cast<uint64_t>(epoch) << 32) | __float_as_uint(o_mine);
      asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_ptr(ctx, ll + base + d)), "l"(v) : "memory");
      if (d == 0) {
        const uint64_t w = (static_cast<uint64_t>(epoch) << 32) | __float_as_uint(lse_mine);
        asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_ptr(ctx, ll + base + kSpD)), "l"(w) : "memory");
      }
    } else {
      for (int k = 1; k < world; ++k) {
        const int peer = (me + k) % world;
        ll_store(symm_at(ctx, ll + base + d, peer), __float_as_uint(o_mine), epoch);
        if (d == 0) ll_store(symm_at(ctx, ll + base + kSpD, peer), __float_as_uint(lse_mine), epoch);
      }
    }
  }
  // 3. receive the other ranks' partials of this head
  float o_r[kMaxRanks];
  bool ok = true;
  if (d < world) {
    if (d == me) {
      lse_of[d] = lse_mine;
    } else {
      uint32_t w = 0;
      ok = ll_load(ctx, ll + (static_cast<size_t>(d) * p.BH + bh) * (kSpD + 1) + kSpD, epoch, &w);
      lse_of[d] = ok ? __uint_as_float(w) : -INFINITY;
    }
  }
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) {
    o_r[r] = 0.f;
    if (r < world) {
      if (r == me) {
        o_r[r] = o_mine;
      } else {
        uint32_t w = 0;
        ok = ll_load(ctx, ll + (static_cast<size_t>(r) * p.BH + bh) * (kSpD + 1) + d, epoch, &w) && ok;
        o_r[r] = __uint_as_float(w);
      }
    }
  }
  ok = __syncthreads_and(ok);
  // 4. combine
  if (ok) {
    float m = -INFINITY;
    for (int r = 0; r < world; ++r) m = fmaxf(m, lse_of[r]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < world && lse_of[r] != -INFINITY) {
        const float w = __expf(lse_of[r] - m);
        den += w;
        num += w * o_r[r];
      }
    }
    const float o = den > 0.f ? num / den : 0.f;
    if (p.bf16) static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(bh) * kSpD + d] = __float2bfloat16(o);
    else static_cast<__half*>(p.out)[static_cast<size_t>(bh) * kSpD + d] = __float2half(o);
    if (d == 0 && p.out_lse) p.out_lse[bh] = den > 0.f ? m + logf(den) : -INFINITY;
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

// ------------------------------------------------------------------------------------------------
// Bulk variant for many rows (large batches). The packet protocol above sends one 8-byte packet per output word and
// polls each of them; beyond about a thousand rows per rank the packet rate through the switch, not the bytes, sets the
// time (2048 rows: 264 K packets per rank and call). Here the merged rows travel as plain coalesced 4-byte stores
// (128 bytes per warp and peer, half the bytes of the packets), one release flag per rank follows them, and the
// cross-rank combine runs after every rank's flag has arrived. Rows are 132 floats apart (128 outputs, the LSE, pad).
// The grid is launched cooperatively (every CTA waits for the flags, so all of them must be resident) and walks the rows.
constexpr int kSpRow = 132;

struct SpBulkParams {
  const float* o_part;
  const float* lse_part;
  int S, BH;
  float* buf[2];     // symmetric, per parity: [world][BH][132] floats
  uint32_t* flags;   // symmetric u32[2][kMaxRanks]: flags[parity][source] = epoch
  uint32_t* sync;    // local u32[4]: epoch, done counter, arrival counter
  void* out;
  float* out_lse;
  int bf16;
};

__global__ void __launch_bounds__(kSpD) sp_decode_combine_bulk_kernel(const SpBulkParams p, const SymmCtx ctx) {
  __shared__ float lse_of[kMaxRanks];
  const uint32_t epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  float* buf = p.buf[par];
  uint32_t* flags = p.flags + par * kMaxRanks;
  const int d = threadIdx.x;
  const int me = ctx.rank, world = ctx.world;
  // 1. merge this rank's splits of every row and store the result into slot [me] on every rank
  for (int bh = blockIdx.x; bh < p.BH; bh += gridDim.x) {
    float o_mine, lse_mine;
    merge_splits(p.lse_part + static_cast<size_t>(bh) * p.S, 1, p.o_part + static_cast<size_t>(bh) * p.S * kSpD + d, kSpD, p.S,
                 o_mine, lse_mine);
    float* row = buf + (static_cast<size_t>(me) * p.BH + bh) * kSpRow;
    for (int k = 0; k < world; ++k) {
      const int peer = (me + k) % world;
      float* dst = symm_at(ctx, row, peer);
      dst[d] = o_mine;
      if (d == 0) dst[kSpD] = lse_mine;
    }
  }
  // 2. the last CTA to arrive releases flag[me] = epoch on every rank; every CTA then waits for all sources
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    if (atom_add_acqrel_gpu(p.sync + 2, 1u) == gridDim.x - 1) {
      p.sync[2] = 0;
      fence_acq_rel_sys();
      for (int r = 0; r < world; ++r) st_release_sys(symm_at(ctx, flags + me, r), epoch);
    }
  }
  bool ok = true;
  if (threadIdx.x < world) ok = wait_flag<WaitCmp::GE, true>(ctx, flags + threadIdx.x, epoch, threadIdx.x, __LINE__);
  ok = __syncthreads_and(ok);
  // 3. cross-rank combine from this rank's own memory (past L1: the rows were written by other GPUs)
  if (ok) {
    for (int bh = blockIdx.x; bh < p.BH; bh += gridDim.x) {
      if (d < world) lse_of[d] = __ldcg(buf + (static_cast<size_t>(d) * p.BH + bh) * kSpRow + kSpD);
      float o_r[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        o_r[r] = r < world ? __ldcg(buf + (static_cast<size_t>(r) * p.BH + bh) * kSpRow + d) : 0.f;
      __syncthreads();
      float m = -INFINITY;
      for (int r = 0; r < world; ++r) m = fmaxf(m, lse_of[r]);
      float den = 0.f, num = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < world && lse_of[r] != -INFINITY) {
          const float w = __expf(lse_of[r] - m);
          den += w;
          num += w * o_r[r];
        }
      }
      const float o = den > 0.f ? num / den : 0.f;
      if (p.bf16) static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(bh) * kSpD + d] = __float2bfloat16(o);
      else static_cast<__half*>(p.out)[static_cast<size_t>(bh) * kSpD + d] = __float2half(o);
      if (d == 0 && p.out_lse) p.out_lse[bh] = den > 0.f ? m + logf(den) : -INFINITY;
      __syncthreads();  // lse_of is reused by the next row
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

}  // namespace b200

using namespace b200;

// Bulk exchange (see the kernel): buf0 / buf1 are the symmetric parity areas of at least world * BH * 132 floats each
// (the packet areas of b200_sp_decode_combine are large enough), flags symmetric u32[2 * 8] zero-initialised once and
// used by bulk calls only, sync local u32[4] zero-initialised once and used by bulk calls only.
B200_API int b200_sp_decode_combine_bulk(const void* symm_ctx, const float* o_part, const float* lse_part, int BH, int S,
                                         void* buf0, void* buf1, uint32_t* flags, uint32_t* sync, void* out, float* out_lse,
                                         int dtype, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "sp decode combine writes bf16/f16");
  if (BH == 0) return kOk;
  SpBulkParams p;
  memset(&p, 0, sizeof(p));
  p.o_part = o_part; p.lse_part = lse_part; p.S = S; p.BH = BH;
  p.buf[0] = static_cast<float*>(buf0); p.buf[1] = static_cast<float*>(buf1);
  p.flags = flags; p.sync = sync; p.out = out; p.out_lse = out_lse; p.bf16 = dtype == kBF16;
  int per_sm = 0;
  B200_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sp_decode_combine_bulk_kernel, kSpD, 0));
  per_sm = per_sm > 2 ? 2 : per_sm;  // every CTA waits on the same flags: a few hundred CTAs keep the polling off that L2 line's back
  B200_REQUIRE(per_sm >= 1, "sp decode bulk kernel does not fit an SM");
  const int cap = per_sm * sm_count();
  const int grid = BH < cap ? BH : cap;
  B200_CHECK_CUDA(launch_cooperative(sp_decode_combine_bulk_kernel, dim3(grid), dim3(kSpD), 0,
                                     static_cast<cudaStream_t>(stream), p, ctx));
  return kOk;
}

// o_part fp32 [BH, S, 128], lse_part fp32 [BH, S]: this rank's split partials. ll0 / ll1: symmetric u64 areas of
// world * BH_cap * 129 packets (the kernel indexes them with this call's BH, which every rank must share).
B200_API int b200_sp_decode_combine(const void* symm_ctx, const float* o_part, const float* lse_part, int BH, int S,
                                    void* ll0, void* ll1, uint32_t* sync, void* out, float* out_lse, int dtype, int use_mc,
                                    void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "sp decode combine writes bf16/f16");
  B200_REQUIRE(!use_mc || ctx.mc_base != 0, "multimem packets need an NVLS multicast mapping");
  if (BH == 0) return kOk;
  SpParams p;
  memset(&p, 0, sizeof(p));
  p.o_part = o_part; p.lse_part = lse_part; p.S = S; p.BH = BH;
  p.ll[0] = static_cast<uint64_t*>(ll0); p.ll[1] = static_cast<uint64_t*>(ll1);
  p.sync = sync; p.out = out; p.out_lse = out_lse; p.bf16 = dtype == kBF16; p.use_mc = use_mc;
  sp_decode_combine_kernel<<<BH, kSpD, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
