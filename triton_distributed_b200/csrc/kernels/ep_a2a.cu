// Expert-parallel all-to-all: dispatch (tokens -> the ranks that own their experts) and combine (expert outputs
// -> back to the token's rank, summed over its k experts), plus the generic sorted-rows all-to-all of the
// reference's low-latency API.
//
//   ep_row_a2a    rows already sorted by global expert; rank d receives the rows of its experts from source s at
//                 rows s * max_m ... of its receive buffer, with the per-expert counts and optional per-row scales
//                 (fast_all_to_all, python/triton_dist/kernels/nvidia/low_latency_all_to_all.py:35-118, 198-257)
//   ep_dispatch   fused permute + optional online fp8 quantisation + send: one warp per token reads the bf16 row
//                 once, quantises every 128 channels to e4m3 with an fp32 scale (amax / 448, as in
//                 tutorials/04-deepseek-infer-all2all.py:189-193) and stores the row (+ scales) straight into the
//                 slot of each of its k experts' ranks, in the sender's expert order (grouped-GEMM ready)
//   ep_combine    sends the expert outputs back and, once all peers' rows have landed, sums the k returned rows of
//                 every token with its routing weights (the reference leaves the weighted sum to torch index_add,
//                 test_all_to_all.py:366-367, and kernel_combine_token ignores the weights, ep_a2a.py:192-206)
//   ep_recv_plan  turns the received [source, local expert] counts into the sorted-row / tile metadata of the
//                 grouped GEMM (rows grouped by local expert, then source), without a host round trip
//                 (kernel_get_ag_splits_and_recv_offset + CPU polling in the reference, ep_a2a.py:243-306,
//                 layers/nvidia/ep_a2a_layer.py:173-193)
//
// Many CTAs per kernel (the reference uses one CTA per peer), 16-byte P2P stores, receive buffers double-buffered
// by epoch parity, one release flag per (source, destination) written by the last CTA to finish, bounded waits.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>
#include <cuda_fp8.h>

namespace b200 {

constexpr int kEpThreads = 256;
constexpr int kEpMaxExperts = 1024;

struct EpParams {
  int world_unused;
  int T, H, topk, E, E_local, max_m;
  int row_bytes;            // payload bytes per row as sent (H * 2 for bf16, H for fp8)
  int scale_floats;         // fp32 scales per row (0 = none)
  int quant;                // dispatch: 1 = bf16 -> e4m3 online
  const void* x;            // dispatch: [T, H] bf16; row_a2a: rows [n, row_bytes]
  const float* x_scale;     // row_a2a: [n, scale_floats] or null
  const int32_t* topk_ids;  // [T, topk]
  const int32_t* pair_pos;  // [T * topk] position of every pair in the expert-sorted order (unpadded sort)
  const int32_t* counts;    // [E] pairs per global expert (dispatch / combine); row_a2a: null
  const int32_t* cum_in;    // row_a2a: [E + 1] cumulative splits
  uint8_t* recv[2];         // symmetric [world * max_m, row_bytes]
  float* recv_scale[2];     // symmetric [world * max_m, scale_floats]
  int32_t* recv_splits[2];  // symmetric [world, E_local]
  uint32_t* flags;          // symmetric u32[2][kMaxRanks]
  uint32_t* sync;           // local u32[4]: epoch, done counter, CTA arrival counter
  // combine
  const void* expert_out;   // [world * max_m, H] bf16 rows in the receive layout of the matching dispatch
  const uint32_t* dispatch_sync;  // epoch word of the dispatch whose layout is being reversed
  const int32_t* dispatch_splits[2];
  uint8_t* comb[2];         // symmetric [world * max_m, H] bf16
  const float* topk_weight; // [T, topk] or null (plain sum)
  void* out;                // [T, H] bf16
  // dispatch, optional: grouped-GEMM metadata of the received rows, built by CTA 0 once every source has delivered
  int32_t* plan_sorted_ids;       // null = no plan
  int32_t* plan_tile_expert;
  int32_t* plan_totals;
  int32_t* plan_rows_per_expert;
  int plan_cap_rows, plan_block_m;
};

// cum[e] = pairs of experts < e; every CTA computes it for itself (E <= 1024): coalesced load, then warp 0 scans
// 32 experts per step.
__device__ __forceinline__ void build_cum(const int32_t* counts, const int32_t* cum_in, int E, int* cum) {
  if (cum_in) {
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cum[e] = cum_in[e];
  } else {
    for (int e = threadIdx.x; e < E; e += blockDim.x) cum[e + 1] = counts[e];
    __syncthreads();
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      int carry = 0;
      for (int base = 0; base < E; base += 32) {
        const int v = base + lane < E ? cum[base + lane + 1] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += u;
        }
        if (base + lane < E) cum[base + lane + 1] = carry + incl;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) cum[0] = 0;
    }
  }
  __syncthreads();
}

// Last CTA to arrive releases flag[me] = epoch on every rank; then CTA 0 (or every CTA) waits for all sources.
__device__ __forceinline__ bool signal_and_wait(const SymmCtx& ctx, uint32_t* flags_par, uint32_t* arrive_ctr, uint32_t epoch,
                                                bool every_cta_waits) {
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    if (atom_add_acqrel_gpu(arrive_ctr, 1u) == gridDim.x - 1) {
      *arrive_ctr = 0;
      fence_acq_rel_sys();
      for (int d = 0; d < ctx.world; ++d) st_release_sys(symm_at(ctx, flags_par + ctx.rank, d), epoch);
    }
  }
  bool ok = true;
  if ((every_cta_waits || blockIdx.x == 0) && threadIdx.x < ctx.world)
    ok = wait_flag<WaitCmp::EQ, true>(ctx, flags_par + threadIdx.x, epoch, threadIdx.x, __LINE__);
  return __syncthreads_and(ok);
}

// Chunks per token row in the dispatch kernel: eight 128-channel blocks when quantising, 2 KB of bf16 otherwise.
__host__ __device__ __forceinline__ int ep_dispatch_chunks(int H, int quant) {
  return quant ? (H / 128 + 7) / 8 : (H * 2 + 2047) / 2048;
}

// One warp copies one row; eight (then four) independent 16-byte loads in flight per lane.
__device__ __forceinline__ void copy_row_warp(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
  int i = lane * 16;
  for (; i + 7 * 512 < bytes; i += 8 * 512) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ld_v4_relaxed_sys(src + i + u * 512);
#pragma unroll
    for (int u = 0; u < 8; ++u) st_v4(dst + i + u * 512, v[u]);
  }
  for (; i + 3 * 512 < bytes; i += 4 * 512) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = ld_v4_relaxed_sys(src + i + u * 512);
#pragma unroll
    for (int u = 0; u < 4; ++u) st_v4(dst + i + u * 512, v[u]);
  }
  for (; i < bytes; i += 512) st_v4(dst + i, ld_v4_relaxed_sys(src + i));
}

__device__ __forceinline__ void ep_recv_plan_body(const int32_t* splits, int world, int E_local, int max_m, int block_m,
                                                  int32_t* sorted_ids, int32_t* tile_expert, int32_t* totals,
                                                  int32_t* rows_per_expert, int cap_rows, int* estart,
                                                  int (*src_off)[kEpMaxExperts + 1]);

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kEpThreads) ep_row_a2a_kernel(const EpParams p, const SymmCtx ctx) {
  __shared__ int cum[kEpMaxExperts + 1];
  const uint32_t epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  build_cum(nullptr, p.cum_in, p.E, cum);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kEpThreads / 32;
  const int n = cum[p.E];
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
      const int d = e / p.E_local;
      *symm_at(ctx, p.recv_splits[par] + ctx.rank * p.E_local + (e - d * p.E_local), d) = cum[e + 1] - cum[e];
    }
  for (int r = blockIdx.x * warps + warp; r < n; r += gridDim.x * warps) {
    int d = 0;
    while (d + 1 < ctx.world && r >= cum[(d + 1) * p.E_local]) ++d;
    const int idx = r - cum[d * p.E_local];
    if (idx >= p.max_m) {  // more rows for this peer than its receive area holds: drop the row, tell the host
      if (lane == 0) report_status(ctx, kStatusBadArgument, d, p.max_m, idx, __LINE__);
      continue;
    }
    const size_t slot = static_cast<size_t>(ctx.rank) * p.max_m + idx;
    copy_row_warp(symm_at(ctx, p.recv[par] + slot * p.row_bytes, d), static_cast<const uint8_t*>(p.x) + static_cast<size_t>(r) * p.row_bytes,
                  p.row_bytes, lane);
    if (p.scale_floats && lane < p.scale_floats)
      for (int j = lane; j < p.scale_floats; j += 32)
        symm_at(ctx, p.recv_scale[par] + slot * p.scale_floats, d)[j] = p.x_scale[static_cast<size_t>(r) * p.scale_floats + j];
  }
  signal_and_wait(ctx, p.flags + par * kMaxRanks, p.sync + 2, epoch, false);
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kEpThreads) ep_dispatch_kernel(const EpParams p, const SymmCtx ctx) {
  __shared__ int cum[kEpMaxExperts + 1];
  const uint32_t epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  build_cum(p.counts, nullptr, p.E, cum);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kEpThreads / 32;
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
      const int d = e / p.E_local;
      *symm_at(ctx, p.recv_splits[par] + ctx.rank * p.E_local + (e - d * p.E_local), d) = p.counts[e];
    }
  const uint8_t* x = static_cast<const uint8_t*>(p.x);
  // A work item is one chunk of one token's row (1024 channels when quantising, 2 KB otherwise), so that a small batch
  // still spreads over the whole grid and no warp walks a row in a chain of dependent round trips.
  const int nchunk = ep_dispatch_chunks(p.H, p.quant);
  const int items = p.T * nchunk;
  for (int it = blockIdx.x * warps + warp; it < items; it += gridDim.x * warps) {
    const int t = it / nchunk, chunk = it - t * nchunk;
    // destination of each of the k copies (lane k holds copy k)
    uint8_t* my_dst = nullptr;
    float* my_sdst = nullptr;
    if (lane < p.topk) {  // a copy whose expert id or slot is out of range is dropped and reported (null destination)
      const int e = p.topk_ids[t * p.topk + lane];
      if (e >= 0 && e < p.E) {
        const int d = e / p.E_local;
        const int idx = p.pair_pos[t * p.topk + lane] - cum[d * p.E_local];
        if (idx >= 0 && idx < p.max_m) {
          const size_t slot = static_cast<size_t>(ctx.rank) * p.max_m + idx;
          my_dst = symm_at(ctx, p.recv[par] + slot * p.row_bytes, d);
          if (p.scale_floats) my_sdst = symm_at(ctx, p.recv_scale[par] + slot * p.scale_floats, d);
        } else {
          report_status(ctx, kStatusBadArgument, d, p.max_m, idx, __LINE__);
        }
      } else {
        report_status(ctx, kStatusBadArgument, lane, p.E, static_cast<uint32_t>(e), __LINE__);
      }
    }
    const uint8_t* row = x + static_cast<size_t>(t) * p.H * 2;
    if (!p.quant) {
      {  // four loads in flight, then k stores each
        const int i0 = chunk * (4 * 512) + lane * 16;
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[u] = i0 + u * 512 < p.H * 2 ? *reinterpret_cast<const uint4*>(row + i0 + u * 512) : make_uint4(0, 0, 0, 0);
        for (int k = 0; k < p.topk; ++k) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_dst), k));
          if (dst == nullptr) continue;
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i0 + u * 512 < p.H * 2) st_v4(dst + i0 + u * 512, v[u]);
        }
      }
    } else {
      // each half-warp owns one 128-channel block per step (a lane holds 8 channels); four steps are loaded at once
      const int half = lane >> 4, hl = lane & 15;
      const int nblk = p.H / 128;
      {
        const int b0 = chunk * 8;
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int blk = b0 + 2 * u + half;
          raw[u] = blk < nblk ? *reinterpret_cast<const uint4*>(row + (static_cast<size_t>(blk) * 128 + hl * 8) * 2)
                              : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int blk = b0 + 2 * u + half;
          const bool in = blk < nblk;
          float f[8];
          const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 x2 = unpack_bf16x2(w[q]);
            f[2 * q] = x2.x;
            f[2 * q + 1] = x2.y;
          }
          float amax = 0.f;
#pragma unroll
          for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float scale = amax / 448.f;
          const float den = scale > 0.f ? scale : 1.f;  // exact division, so that rounding ties fall as in x / scale
          uint32_t lo = 0, hi = 0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t a = __nv_cvt_float_to_fp8(__fdiv_rn(f[q], den), __NV_SATFINITE, __NV_E4M3);
            const uint32_t c = __nv_cvt_float_to_fp8(__fdiv_rn(f[4 + q], den), __NV_SATFINITE, __NV_E4M3);
            lo |= a << (8 * q);
            hi |= c << (8 * q);
          }
          for (int k = 0; k < p.topk; ++k) {
            uint8_t* dst = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_dst), k));
            float* sdst = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_sdst), k));
            if (in && dst != nullptr) {
              *reinterpret_cast<uint2*>(dst + blk * 128 + hl * 8) = make_uint2(lo, hi);
              if (hl == 0) sdst[blk] = scale;
            }
          }
        }
      }
    }
  }
  const bool all_in = signal_and_wait(ctx, p.flags + par * kMaxRanks, p.sync + 2, epoch, false);
  if (blockIdx.x == 0 && p.plan_sorted_ids != nullptr && all_in) {
    // every source's splits have landed (the wait above acquired them): CTA 0 lays out the grouped-GEMM plan of the
    // received rows here, which saves the separate one-CTA launch that used to follow every dispatch
    __shared__ int estart[kEpMaxExperts + 1];
    __shared__ int src_off[kMaxRanks][kEpMaxExperts + 1];
    ep_recv_plan_body(p.recv_splits[par], ctx.world, p.E_local, p.max_m, p.plan_block_m, p.plan_sorted_ids, p.plan_tile_expert,
                      p.plan_totals, p.plan_rows_per_expert, p.plan_cap_rows, estart, src_off);
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(const EpParams p, const SymmCtx ctx) {
  __shared__ int cum[kEpMaxExperts + 1];
  __shared__ int src_rows[kMaxRanks];
  const uint32_t epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  const int dpar = ld_relaxed_gpu(p.dispatch_sync) & 1;  // layout of the last completed dispatch
  build_cum(p.counts, nullptr, p.E, cum);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kEpThreads / 32;
  if (threadIdx.x < ctx.world) {
    int n = 0;
    for (int e = 0; e < p.E_local; ++e) n += p.dispatch_splits[dpar][threadIdx.x * p.E_local + e];
    src_rows[threadIdx.x] = n < p.max_m ? n : p.max_m;  // a sender that overflowed its area dropped the excess rows
  }
  __syncthreads();
  // phase 1: return every received row's output to the rank it came from, same slot numbering. The rows of all
  // sources form one index space, so that every warp of the grid has a row (a loop over the sources with a warp
  // stride inside would keep only rows-per-source warps busy at a time)
  const uint8_t* eo = static_cast<const uint8_t*>(p.expert_out);
  const int row_bytes = p.H * 2;
  int total_rows = 0;
  for (int s = 0; s < ctx.world; ++s) total_rows += src_rows[s];
  for (int f = blockIdx.x * warps + warp; f < total_rows; f += gridDim.x * warps) {
    int s = 0, i = f;
    while (i >= src_rows[s]) i -= src_rows[s++];
    const size_t from = (static_cast<size_t>(s) * p.max_m + i) * row_bytes;
    const size_t to = (static_cast<size_t>(ctx.rank) * p.max_m + i) * row_bytes;
    copy_row_warp(symm_at(ctx, p.comb[par] + to, s), eo + from, row_bytes, lane);
  }
  const bool ok = signal_and_wait(ctx, p.flags + par * kMaxRanks, p.sync + 2, epoch, true);
  // phase 2: weighted sum of the k returned rows of every token. A work item is one 1 KB column chunk of one token
  // (two 512-byte steps, the 2 x topk loads of a lane issued together): a whole row per warp would be row_bytes / 512
  // dependent memory round trips on only T warps.
  if (ok) {
    constexpr int kChunk = 1024;
    const int nchunk = (row_bytes + kChunk - 1) / kChunk;
    const int items = p.T * nchunk;
    for (int it = blockIdx.x * warps + warp; it < items; it += gridDim.x * warps) {
      const int t = it / nchunk, c0 = (it - t * nchunk) * kChunk;
      const uint8_t* my_src = nullptr;
      float my_w = 1.f;
      if (lane < p.topk) {  // copies that the dispatch dropped (bad expert id, full receive area) contribute nothing
        const int e = p.topk_ids[t * p.topk + lane];
        if (e >= 0 && e < p.E) {
          const int d = e / p.E_local;
          const int idx = p.pair_pos[t * p.topk + lane] - cum[d * p.E_local];
          if (idx >= 0 && idx < p.max_m) {
            my_src = p.comb[par] + (static_cast<size_t>(d) * p.max_m + idx) * row_bytes;
            if (p.topk_weight) my_w = p.topk_weight[t * p.topk + lane];
          }
        }
      }
      float acc[2][8];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[h][q] = 0.f;
      for (int k0 = 0; k0 < p.topk; k0 += 8) {  // same trip count for every lane (shuffles inside)
        uint4 v[2][8];
        float wk[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int k = k0 + u < p.topk ? k0 + u : k0;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_src), k));
          const float w = __shfl_sync(0xffffffffu, my_w, k);
          const bool use = k0 + u < p.topk && src != nullptr;
          wk[u] = use ? w : 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int i = c0 + h * 512 + lane * 16;
            v[h][u] = (use && i < row_bytes) ? ld_v4_relaxed_sys(src + i) : make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t w4[4] = {v[h][u].x, v[h][u].y, v[h][u].z, v[h][u].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = unpack_bf16x2(w4[q]);
              acc[h][2 * q] += wk[u] * f.x;
              acc[h][2 * q + 1] += wk[u] * f.y;
            }
          }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = c0 + h * 512 + lane * 16;
        if (i < row_bytes)
          st_v4(static_cast<uint8_t*>(p.out) + static_cast<size_t>(t) * row_bytes + i,
                make_uint4(pack_bf16x2(acc[h][0], acc[h][1]), pack_bf16x2(acc[h][2], acc[h][3]),
                           pack_bf16x2(acc[h][4], acc[h][5]), pack_bf16x2(acc[h][6], acc[h][7])));
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

// Build grouped-GEMM metadata from recv_splits [world, E_local]: rows grouped by local expert, then source.
// sorted_ids[i] = row index in the receive buffer (s * max_m + offset), pad = world * max_m. Executed by ONE CTA of any
// size (a multiple of 32 threads); `estart` and `src_off` are shared memory.
__device__ __forceinline__ void ep_recv_plan_body(const int32_t* splits, int world, int E_local, int max_m, int block_m,
                                                  int32_t* sorted_ids, int32_t* tile_expert, int32_t* totals,
                                                  int32_t* rows_per_expert, int cap_rows, int* estart,
                                                  int (*src_off)[kEpMaxExperts + 1]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  // role 0: padded expert starts; roles 1..world: offsets inside each source's area (32 experts per step)
  for (int role = warp; role <= world; role += nwarps) {
    int carry = 0;
    for (int base = 0; base < E_local; base += 32) {
      const int e = base + lane;
      int v = 0;
      if (e < E_local) {
        if (role == 0) {
          int c = 0;
          for (int s = 0; s < world; ++s) c += splits[s * E_local + e];
          rows_per_expert[e] = c;
          v = (c + block_m - 1) / block_m * block_m;
        } else {
          v = splits[(role - 1) * E_local + e];
        }
      }
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (e < E_local) {
        if (role == 0) estart[e] = carry + incl - v;
        else src_off[role - 1][e] = carry + incl - v;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      if (role == 0) {
        estart[E_local] = carry;
        totals[0] = carry;
        totals[1] = carry / block_m;
      } else {
        src_off[role - 1][E_local] = carry;
      }
    }
  }
  __syncthreads();
  const int pad = world * max_m;
  for (int i = threadIdx.x; i < min(estart[E_local], cap_rows); i += blockDim.x) sorted_ids[i] = pad;
  __syncthreads();
  for (int e = warp; e < E_local; e += nwarps) {  // one warp per local expert: the experts are independent
    int dst = estart[e];
    for (int s = 0; s < world; ++s) {
      const int n = src_off[s][e + 1] - src_off[s][e];
      for (int i = lane; i < n; i += 32)
        if (dst + i < cap_rows) sorted_ids[dst + i] = s * max_m + src_off[s][e] + i;
      dst += n;
    }
    for (int t = estart[e] / block_m + lane; t < estart[e + 1] / block_m; t += 32) tile_expert[t] = e;
  }
}

__global__ void __launch_bounds__(1024) ep_recv_plan_kernel(const int32_t* splits, int world, int E_local, int max_m, int block_m,
                                                            int32_t* sorted_ids, int32_t* tile_expert, int32_t* totals,
                                                            int32_t* rows_per_expert, int cap_rows) {
  __shared__ int estart[kEpMaxExperts + 1];              // padded start row of every local expert
  __shared__ int src_off[kMaxRanks][kEpMaxExperts + 1];  // offset of (s, e) inside source s's area; [E_local] = total
  ep_recv_plan_body(splits, world, E_local, max_m, block_m, sorted_ids, tile_expert, totals, rows_per_expert, cap_rows, estart,
                    src_off);
}

static int ep_grid(int rows) {
  int g = (rows + 7) / 8;
  const int cap = sm_count();
  return g < 1 ? 1 : (g > cap ? cap : g);
}

}  // namespace b200

using namespace b200;

#define EP_CTX()      \
  SymmCtx ctx;        \
  memcpy(&ctx, symm_ctx, sizeof(ctx))

// rows [n, row_bytes] sorted by global expert; cum int32 [E + 1]; scales fp32 [n, scale_floats] or null.
B200_API int b200_ep_row_a2a(const void* symm_ctx, const void* rows, int row_bytes, const int32_t* cum, int n_upper, int E,
                             int E_local, int max_m, const float* scales, int scale_floats, void* recv0, void* recv1,
                             void* recv_scale0, void* recv_scale1, int32_t* splits0, int32_t* splits1, uint32_t* flags,
                             uint32_t* sync, void* stream) {
  EP_CTX();
  B200_REQUIRE(row_bytes % 16 == 0, "row bytes (%d) must be a multiple of 16", row_bytes);
  B200_REQUIRE(E <= kEpMaxExperts && E == E_local * ctx.world, "experts (%d) must equal E_local * world and be <= %d", E, kEpMaxExperts);
  EpParams p;
  memset(&p, 0, sizeof(p));
  p.E = E; p.E_local = E_local; p.max_m = max_m; p.row_bytes = row_bytes; p.scale_floats = scales ? scale_floats : 0;
  p.x = rows; p.x_scale = scales; p.cum_in = cum;
  p.recv[0] = static_cast<uint8_t*>(recv0); p.recv[1] = static_cast<uint8_t*>(recv1);
  p.recv_scale[0] = static_cast<float*>(recv_scale0); p.recv_scale[1] = static_cast<float*>(recv_scale1);
  p.recv_splits[0] = splits0; p.recv_splits[1] = splits1; p.flags = flags; p.sync = sync;
  ep_row_a2a_kernel<<<ep_grid(n_upper), kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

// x bf16 [T, H]; topk_ids int32 [T, topk]; pair_pos / counts from an unpadded (block 1) expert sort of the pairs.
// quant != 0: rows travel as e4m3 [H] with H / 128 fp32 scales; else as bf16.
B200_API int b200_ep_dispatch(const void* symm_ctx, const void* x, int T, int H, int topk, const int32_t* topk_ids,
                              const int32_t* pair_pos, const int32_t* counts, int E, int E_local, int max_m, int quant,
                              void* recv0, void* recv1, void* recv_scale0, void* recv_scale1, int32_t* splits0,
                              int32_t* splits1, uint32_t* flags, uint32_t* sync, void* stream) {
  EP_CTX();
  B200_REQUIRE(H % 128 == 0, "hidden (%d) must be a multiple of 128", H);
  B200_REQUIRE(topk >= 1 && topk <= 32, "top-k (%d) must be in [1, 32]", topk);
  B200_REQUIRE(E <= kEpMaxExperts && E == E_local * ctx.world, "experts (%d) must equal E_local * world and be <= %d", E, kEpMaxExperts);
  EpParams p;
  memset(&p, 0, sizeof(p));
  p.T = T; p.H = H; p.topk = topk; p.E = E; p.E_local = E_local; p.max_m = max_m; p.quant = quant;
  p.row_bytes = quant ? H : 2 * H; p.scale_floats = quant ? H / 128 : 0;
  p.x = x; p.topk_ids = topk_ids; p.pair_pos = pair_pos; p.counts = counts;
  p.recv[0] = static_cast<uint8_t*>(recv0); p.recv[1] = static_cast<uint8_t*>(recv1);
  p.recv_scale[0] = static_cast<float*>(recv_scale0); p.recv_scale[1] = static_cast<float*>(recv_scale1);
  p.recv_splits[0] = splits0; p.recv_splits[1] = splits1; p.flags = flags; p.sync = sync;
  ep_dispatch_kernel<<<ep_grid(T * ep_dispatch_chunks(H, quant)), kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

// b200_ep_dispatch that also builds the grouped-GEMM plan of the received rows (see b200_ep_recv_plan) in the same launch.
B200_API int b200_ep_dispatch_planned(const void* symm_ctx, const void* x, int T, int H, int topk, const int32_t* topk_ids,
                                      const int32_t* pair_pos, const int32_t* counts, int E, int E_local, int max_m, int quant,
                                      void* recv0, void* recv1, void* recv_scale0, void* recv_scale1, int32_t* splits0,
                                      int32_t* splits1, uint32_t* flags, uint32_t* sync, int block_m, int32_t* sorted_ids,
                                      int32_t* tile_expert, int32_t* totals, int32_t* rows_per_expert, int cap_rows,
                                      void* stream) {
  EP_CTX();
  B200_REQUIRE(H % 128 == 0, "hidden (%d) must be a multiple of 128", H);
  B200_REQUIRE(topk >= 1 && topk <= 32, "top-k (%d) must be in [1, 32]", topk);
  B200_REQUIRE(E <= kEpMaxExperts && E == E_local * ctx.world, "experts (%d) must equal E_local * world and be <= %d", E, kEpMaxExperts);
  B200_REQUIRE(sorted_ids && tile_expert && totals && rows_per_expert && block_m >= 1, "missing plan buffers");
  EpParams p;
  memset(&p, 0, sizeof(p));
  p.T = T; p.H = H; p.topk = topk; p.E = E; p.E_local = E_local; p.max_m = max_m; p.quant = quant;
  p.row_bytes = quant ? H : 2 * H; p.scale_floats = quant ? H / 128 : 0;
  p.x = x; p.topk_ids = topk_ids; p.pair_pos = pair_pos; p.counts = counts;
  p.recv[0] = static_cast<uint8_t*>(recv0); p.recv[1] = static_cast<uint8_t*>(recv1);
  p.recv_scale[0] = static_cast<float*>(recv_scale0); p.recv_scale[1] = static_cast<float*>(recv_scale1);
  p.recv_splits[0] = splits0; p.recv_splits[1] = splits1; p.flags = flags; p.sync = sync;
  p.plan_sorted_ids = sorted_ids; p.plan_tile_expert = tile_expert; p.plan_totals = totals;
  p.plan_rows_per_expert = rows_per_expert; p.plan_cap_rows = cap_rows; p.plan_block_m = block_m;
  ep_dispatch_kernel<<<ep_grid(T * ep_dispatch_chunks(H, quant)), kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

// expert_out bf16 [world * max_m, H] in the receive layout of the last dispatch; out bf16 [T, H].
B200_API int b200_ep_combine(const void* symm_ctx, const void* expert_out, int T, int H, int topk, const int32_t* topk_ids,
                             const int32_t* pair_pos, const int32_t* counts, const float* topk_weight, int E, int E_local,
                             int max_m, const uint32_t* dispatch_sync, const int32_t* dsplits0, const int32_t* dsplits1,
                             void* comb0, void* comb1, uint32_t* flags, uint32_t* sync, void* out, void* stream) {
  EP_CTX();
  B200_REQUIRE(H % 8 == 0 && topk >= 1 && topk <= 32, "bad hidden / top-k");
  EpParams p;
  memset(&p, 0, sizeof(p));
  p.T = T; p.H = H; p.topk = topk; p.E = E; p.E_local = E_local; p.max_m = max_m;
  p.topk_ids = topk_ids; p.pair_pos = pair_pos; p.counts = counts; p.topk_weight = topk_weight;
  p.expert_out = expert_out; p.dispatch_sync = dispatch_sync; p.dispatch_splits[0] = dsplits0; p.dispatch_splits[1] = dsplits1;
  p.comb[0] = static_cast<uint8_t*>(comb0); p.comb[1] = static_cast<uint8_t*>(comb1); p.flags = flags; p.sync = sync; p.out = out;
  int grid = ep_grid(T > max_m ? T : max_m);
  ep_combine_kernel<<<grid, kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

B200_API int b200_ep_recv_plan(const int32_t* splits, int world, int E_local, int max_m, int block_m, int32_t* sorted_ids,
                               int32_t* tile_expert, int32_t* totals, int32_t* rows_per_expert, int cap_rows, void* stream) {
  B200_REQUIRE(E_local <= kEpMaxExperts && world <= kMaxRanks, "too many local experts / ranks");
  ep_recv_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(splits, world, E_local, max_m, block_m, sorted_ids,
                                                                        tile_expert, totals, rows_per_expert, cap_rows);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
