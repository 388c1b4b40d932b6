// MoE routing metadata in one launch (plus one tiny launch for the tile order), with no host sync, no
// allocation and no device-wide synchronise, so it can sit inside a CUDA graph.
//
//   moe_sort     stable sort of the (token, k) pairs by (segment, expert), every run padded to BLOCK_M rows:
//                  segments == 1      pairs sorted by expert over all tokens (AG + grouped GEMM, EP dispatch);
//                                     each tile also records the first / last source rank of its rows
//                  segments == ranks  every source-rank block of tokens sorted on its own (grouped GEMM + RS)
//                One warp owns one (segment, expert) group: it counts its matches with ballots, publishes the
//                padded count, obtains its offset by looking back at the groups before it (bounded spin on
//                epoch-tagged counts), then compacts its matches in order. Stable, deterministic, E <= 1024.
//   moe_tile_order  counting sort of the tiles by arrival stage ((seg_end - rank - shift) mod world), stable.
//
// Role in the reference: csrc/lib/moe_utils.cu:60-353 (moe_ag_scatter_align_block_size, grid 1 or ranks CTAs,
// cudaMalloc + cudaDeviceSynchronize per call), kernels/nvidia/moe_utils.py:142-248 (single-CTA index kernel),
// kernels/nvidia/threadblock_swizzle_ag_moe.cu:247-417 (<<<1,1024>>> tile scheduler) and the host loop
// moe_reduce_rs.py:79-169.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

namespace b200 {

struct MoeSortParams {
  const int32_t* ids;      // [n_pairs] expert of pair p = t * topk + k
  int n_pairs, topk, num_experts, block_m;
  int segments;            // 1 or number of ranks
  int pairs_per_segment;   // n_pairs / segments
  int tokens_per_rank;     // for the source rank of a row (segments == 1 mode)
  int32_t* sorted_ids;     // [cap] pair index per sorted row, pad = n_pairs
  int32_t* tile_expert;    // [tile cap]
  int32_t* tile_seg_start; // [tile cap]
  int32_t* tile_seg_end;   // [tile cap]
  int32_t* pair_pos;       // nullable [n_pairs]: sorted position of every pair (inverse of sorted_ids)
  int32_t* group_count;    // [segments * experts] matches per group (unpadded)
  int32_t* totals;         // [2 + segments]: m_pad, num_tiles, tiles per segment
  uint64_t* lookback;      // [segments * experts]: (epoch << 32) | padded count
  uint32_t* sync;          // [2] epoch, done counter
  uint64_t timeout_ns;
  uint32_t* status;
};

constexpr int kSortWarps = 16;

__global__ void __launch_bounds__(kSortWarps * 32) moe_sort_kernel(const MoeSortParams p) {
  const uint32_t epoch = epoch_begin(p.sync);
  const int lane = threadIdx.x & 31;
  const int g = blockIdx.x * kSortWarps + (threadIdx.x >> 5);
  const int G = p.segments * p.num_experts;
  SymmCtx c;
  c.status = p.status;
  c.timeout_ns = p.timeout_ns;
  if (g < G) {
    const int seg = g / p.num_experts, e = g - seg * p.num_experts;
    const int p0 = seg * p.pairs_per_segment, p1 = p0 + p.pairs_per_segment;
    // ---- count ----
    // 16-byte loads, two chunks of 128 ids in flight per warp: the scan is latency-bound otherwise
    const bool vec_ok = (p0 % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.ids) & 15u) == 0);
    int count = 0;
    int b0 = p0;
    if (vec_ok) {
      for (; b0 + 256 <= p1; b0 += 256) {
        const int4 a = *reinterpret_cast<const int4*>(p.ids + b0 + lane * 4);
        const int4 c = *reinterpret_cast<const int4*>(p.ids + b0 + 128 + lane * 4);
        count += (a.x == e) + (a.y == e) + (a.z == e) + (a.w == e) + (c.x == e) + (c.y == e) + (c.z == e) + (c.w == e);
      }
    }
    for (; b0 < p1; b0 += 32) {
      const int i = b0 + lane;
      count += (i < p1 && p.ids[i] == e) ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
    const int padded = (count + p.block_m - 1) / p.block_m * p.block_m;
    if (lane == 0) {
      p.group_count[g] = count;
      const uint64_t v = (static_cast<uint64_t>(epoch) << 32) | static_cast<uint32_t>(padded);
      asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p.lookback + g), "l"(v) : "memory");
    }
    // ---- offset = sum of padded counts of the groups before this one ----
    long long offset = 0;
    bool ok = true;
    for (int j = lane; j < g; j += 32) {
      uint64_t v;
      uint64_t t0 = 0;
      uint32_t spins = 0;
      while (true) {
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.lookback + j) : "memory");
        if (static_cast<uint32_t>(v >> 32) == epoch) break;
        if ((++spins & 63u) == 0u) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > p.timeout_ns) {
            report_status(c, kStatusWaitTimeout, j, epoch, static_cast<uint32_t>(v >> 32), __LINE__);
            ok = false;
            break;
          }
        }
      }
      offset += static_cast<uint32_t>(v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) offset += __shfl_xor_sync(0xffffffffu, offset, o);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      // ---- compact in order ----
      int written = 0;
      const int first_tile = static_cast<int>(offset / p.block_m);
      auto emit = [&](int i, int pos) {
        p.sorted_ids[offset + pos] = i;
        if (p.pair_pos) p.pair_pos[i] = static_cast<int32_t>(offset + pos);
        // segment bounds of the tile this row falls into (only needed when sorting over all tokens)
        if (p.segments == 1) {
          const int src = (i / p.topk) / p.tokens_per_rank;
          const int tile = first_tile + pos / p.block_m;
          atomicMin(p.tile_seg_start + tile, src);
          atomicMax(p.tile_seg_end + tile, src);
        }
      };
      int b1 = p0;
      if (vec_ok) {
        // lane l holds ids [b1 + 4l, b1 + 4l + 4): order inside the chunk is (lane, j)
        for (; b1 + 128 <= p1; b1 += 128) {
          const int4 a = *reinterpret_cast<const int4*>(p.ids + b1 + lane * 4);
          const int h0 = a.x == e, h1 = a.y == e, h2 = a.z == e, h3 = a.w == e;
          const int mine_n = h0 + h1 + h2 + h3;
          int incl = mine_n;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
          }
          int pos = written + incl - mine_n;
          const int i0 = b1 + lane * 4;
          if (h0) emit(i0, pos++);
          if (h1) emit(i0 + 1, pos++);
          if (h2) emit(i0 + 2, pos++);
          if (h3) emit(i0 + 3, pos++);
          written += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
      for (; b1 < p1; b1 += 32) {
        const int i = b1 + lane;
        const bool hit = i < p1 && p.ids[i] == e;
        const uint32_t m = __ballot_sync(0xffffffffu, hit);
        if (hit) emit(i, written + __popc(m & ((1u << lane) - 1u)));
        written += __popc(m);
      }
      for (int i = count + lane; i < padded; i += 32) p.sorted_ids[offset + i] = p.n_pairs;
      for (int t = lane; t < padded / p.block_m; t += 32) {
        p.tile_expert[first_tile + t] = e;
        if (p.segments > 1) {
          p.tile_seg_start[first_tile + t] = seg;
          p.tile_seg_end[first_tile + t] = seg;
        }
      }
      if (lane == 0) {
        if (p.segments > 1 && e == p.num_experts - 1) {
          // cumulative: tiles of segments 0..seg
          p.totals[2 + seg] = static_cast<int>((offset + padded) / p.block_m);
        }
        if (g == G - 1) {
          p.totals[0] = static_cast<int>(offset + padded);
          p.totals[1] = static_cast<int>((offset + padded) / p.block_m);
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

// tile_seg_start / tile_seg_end must hold +inf / -1 before the sort in segments == 1 mode.
__global__ void moe_sort_init_kernel(int32_t* seg_start, int32_t* seg_end, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    seg_start[i] = 0x7fffffff;
    seg_end[i] = -1;
  }
}

// Stable counting sort of the tiles by stage; one CTA. order[j] = tile issued j-th.
__global__ void __launch_bounds__(1024) moe_tile_order_kernel(const int32_t* tile_seg_end, const int32_t* totals, int rank,
                                                              int world, int shift, int32_t* order) {
  __shared__ int warp_sums[32];
  __shared__ int base;
  const int n = totals[1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) base = 0;
  __syncthreads();
  for (int s = 0; s < world; ++s) {
    for (int start = 0; start < n; start += 1024) {
      const int t = start + tid;
      bool hit = false;
      if (t < n) {
        int st = (tile_seg_end[t] - rank - shift) % world;
        if (st < 0) st += world;
        hit = st == s;
      }
      const uint32_t m = __ballot_sync(0xffffffffu, hit);
      if (lane == 0) warp_sums[warp] = __popc(m);
      __syncthreads();
      int before = 0, total = 0;
      for (int w = 0; w < 32; ++w) {
        const int v = warp_sums[w];
        if (w < warp) before += v;
        total += v;
      }
      if (hit) order[base + before + __popc(m & ((1u << lane) - 1u))] = t;
      __syncthreads();
      if (tid == 0) base += total;
      __syncthreads();
    }
  }
}

}  // namespace b200

using namespace b200;

// Capacity helpers: rows and tiles needed in the worst case.
B200_API long long b200_moe_sorted_capacity(int n_pairs, int num_experts, int block_m, int segments) {
  const long long groups = static_cast<long long>(num_experts) * segments;
  return (static_cast<long long>(n_pairs) + groups * (block_m - 1) + block_m - 1) / block_m * block_m;
}

// ids int32 [n_pairs]; outputs sized by b200_moe_sorted_capacity (rows) and capacity / block_m (tiles).
// group_count int32 [segments * E]; totals int32 [2 + segments]; lookback u64 [segments * E] and sync u32 [2] are
// zero-initialised once and owned by the caller (one pair per concurrent user). pair_pos (nullable) int32 [n_pairs].
B200_API int b200_moe_sort(const int32_t* ids, int n_pairs, int topk, int num_experts, int block_m, int segments,
                           int tokens_per_rank, int32_t* sorted_ids, int32_t* tile_expert, int32_t* tile_seg_start,
                           int32_t* tile_seg_end, int32_t* group_count, int32_t* totals, uint64_t* lookback,
                           uint32_t* sync, uint32_t* status, int32_t* pair_pos, void* stream) {
  B200_REQUIRE(num_experts >= 1 && num_experts <= 1024, "number of experts (%d) must be in [1, 1024]", num_experts);
  B200_REQUIRE(segments >= 1 && n_pairs % segments == 0, "pairs (%d) must divide into %d segments", n_pairs, segments);
  B200_REQUIRE(block_m >= 1 && topk >= 1 && tokens_per_rank >= 1, "bad block_m / topk / tokens_per_rank");
  const int G = num_experts * segments;
  const int ctas = (G + kSortWarps - 1) / kSortWarps;
  B200_REQUIRE(ctas <= 2 * sm_count(), "too many (segment, expert) groups (%d) for a co-resident grid", G);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tile_cap = static_cast<int>(b200_moe_sorted_capacity(n_pairs, num_experts, block_m, segments) / block_m);
  if (segments == 1) moe_sort_init_kernel<<<(tile_cap + 255) / 256, 256, 0, s>>>(tile_seg_start, tile_seg_end, tile_cap);
  MoeSortParams p;
  memset(&p, 0, sizeof(p));
  p.ids = ids; p.n_pairs = n_pairs; p.topk = topk; p.num_experts = num_experts; p.block_m = block_m;
  p.segments = segments; p.pairs_per_segment = n_pairs / segments; p.tokens_per_rank = tokens_per_rank;
  p.sorted_ids = sorted_ids; p.tile_expert = tile_expert; p.tile_seg_start = tile_seg_start; p.tile_seg_end = tile_seg_end;
  p.pair_pos = pair_pos;
  p.group_count = group_count; p.totals = totals; p.lookback = lookback; p.sync = sync;
  p.timeout_ns = 2000000000ull; p.status = status;
  moe_sort_kernel<<<ctas, kSortWarps * 32, 0, s>>>(p);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

B200_API int b200_moe_tile_order(const int32_t* tile_seg_end, const int32_t* totals, int rank, int world, int shift,
                                 int32_t* order, void* stream) {
  B200_REQUIRE(world >= 1 && world <= kMaxRanks, "world (%d) out of range", world);
  moe_tile_order_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(tile_seg_end, totals, rank, world, shift, order);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
