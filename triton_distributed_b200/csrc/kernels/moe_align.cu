// MoE routing metadata without a host sync, an allocation or a device-wide synchronise, so it can sit inside a
// CUDA graph. Four short launches (no kernel waits on another CTA, so nothing has to be co-resident):
//
//   moe_sort     stable sort of the (token, k) pairs by (segment, expert), every run padded to BLOCK_M rows:
//                  segments == 1      pairs sorted by expert over all tokens (AG + grouped GEMM, EP dispatch);
//                                     each tile also records the first / last source rank of its rows
//                  segments == ranks  every source-rank block of tokens sorted on its own (grouped GEMM + RS)
//                1. count    one CTA per chunk of 512 pairs: shared-memory histogram -> counts[chunk][expert]
//                2. prefix   per (segment, expert): exclusive prefix of the counts over the chunks, group totals
//                3. offsets  one CTA: padded group sizes scanned into group offsets; tile table and pad rows
//                4. scatter  one CTA per chunk: position = group offset + chunk prefix + rank inside the chunk
//                Stable, deterministic, E <= 1024.
//   moe_tile_order  counting sort of the tiles by arrival stage (ring step after which every source shard of the tile
//                   has landed), stable.
//
// Role in the reference: csrc/lib/moe_utils.cu:60-353 (moe_ag_scatter_align_block_size, grid 1 or ranks CTAs,
// cudaMalloc + cudaDeviceSynchronize per call), kernels/nvidia/moe_utils.py:142-248 (single-CTA index kernel),
// kernels/nvidia/threadblock_swizzle_ag_moe.cu:247-417 (<<<1,1024>>> tile scheduler) and the host loop
// moe_reduce_rs.py:79-169.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstdlib>
#include <cstring>

namespace b200 {

constexpr int kChunk = 512;  // pairs per CTA in the count and scatter kernels

struct MoeSortParams {
  const int32_t* ids;      // [n_pairs] expert of pair p = t * topk + k
  int n_pairs, topk, num_experts, block_m;
  int segments;            // 1 or number of ranks
  int pairs_per_segment;   // n_pairs / segments
  int chunks_per_segment;  // ceil(pairs_per_segment / kChunk)
  int tokens_per_rank;     // for the source rank of a row (segments == 1 mode)
  int32_t* sorted_ids;     // [cap] pair index per sorted row, pad = n_pairs
  int32_t* tile_expert;    // [tile cap]
  int32_t* tile_seg_start; // [tile cap]
  int32_t* tile_seg_end;   // [tile cap]
  int32_t* pair_pos;       // nullable [n_pairs]: sorted position of every pair (inverse of sorted_ids)
  int32_t* group_count;    // [segments * experts] matches per group (unpadded)
  int32_t* totals;         // [2 + segments]: m_pad, num_tiles, cumulative tiles per segment
  int32_t* chunk_cnt;      // scratch [segments * chunks_per_segment][experts]: counts, then exclusive prefixes
  int32_t* group_off;      // scratch [segments * experts]: first sorted row of every group
};

// ---- 1. per-chunk histogram
__global__ void __launch_bounds__(kChunk) moe_count_kernel(const MoeSortParams p) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < p.num_experts; e += kChunk) hist[e] = 0;
  __syncthreads();
  const int seg = blockIdx.x / p.chunks_per_segment, c = blockIdx.x - seg * p.chunks_per_segment;
  const int i = c * kChunk + threadIdx.x;
  if (i < p.pairs_per_segment) {
    const int e = p.ids[seg * p.pairs_per_segment + i];
    if (e >= 0 && e < p.num_experts) atomicAdd(hist + e, 1);
  }
  __syncthreads();
  int32_t* out = p.chunk_cnt + static_cast<size_t>(blockIdx.x) * p.num_experts;
  for (int e = threadIdx.x; e < p.num_experts; e += kChunk) out[e] = hist[e];
}

// ---- 2. exclusive prefix over the chunks of a segment, 32 experts per CTA; thread (tx, ty) owns expert tx and the
//         ty-th contiguous slice of the chunks
__global__ void __launch_bounds__(1024) moe_chunk_prefix_kernel(const MoeSortParams p) {
  __shared__ int32_t part[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int e = blockIdx.x * 32 + tx, seg = blockIdx.y;
  const int per = (p.chunks_per_segment + 31) / 32;
  const int c0 = min(p.chunks_per_segment, ty * per), c1 = min(p.chunks_per_segment, c0 + per);
  int32_t* col = p.chunk_cnt + static_cast<size_t>(seg) * p.chunks_per_segment * p.num_experts + e;
  int sum = 0;
  if (e < p.num_experts)
    for (int c = c0; c < c1; ++c) sum += col[static_cast<size_t>(c) * p.num_experts];
  part[ty][tx] = sum;
  __syncthreads();
  int before = 0, total = 0;
  for (int k = 0; k < 32; ++k) {
    const int v = part[k][tx];
    if (k < ty) before += v;
    total += v;
  }
  if (e < p.num_experts) {
    int run = before;
    for (int c = c0; c < c1; ++c) {
      const int v = col[static_cast<size_t>(c) * p.num_experts];
      col[static_cast<size_t>(c) * p.num_experts] = run;
      run += v;
    }
    if (ty == 0) p.group_count[seg * p.num_experts + e] = total;
  }
}

// ---- 3. group offsets (scan of the padded group sizes), tile table, pad rows, totals; one CTA
__global__ void __launch_bounds__(1024) moe_offsets_kernel(const MoeSortParams p) {
  __shared__ int32_t warp_tot[32];
  __shared__ int32_t carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.segments * p.num_experts;
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int g0 = 0; g0 < G; g0 += 1024) {
    const int g = g0 + tid;
    const int count = g < G ? p.group_count[g] : 0;
    const int padded = (count + p.block_m - 1) / p.block_m * p.block_m;
    int incl = padded;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int off = before + incl - padded;
    if (g < G) p.group_off[g] = off;
    __syncthreads();
    if (tid == 1023) carry = off + padded;
    __syncthreads();
  }
  // tiles and pad rows, one warp per group
  for (int g = warp; g < G; g += 32) {
    const int seg = g / p.num_experts, e = g - seg * p.num_experts;
    const int count = p.group_count[g], off = p.group_off[g];
    const int padded = (count + p.block_m - 1) / p.block_m * p.block_m;
    for (int i = count + lane; i < padded; i += 32) p.sorted_ids[off + i] = p.n_pairs;
    const int first_tile = off / p.block_m;
    for (int t = lane; t < padded / p.block_m; t += 32) {
      p.tile_expert[first_tile + t] = e;
      p.tile_seg_start[first_tile + t] = p.segments > 1 ? seg : 0x7fffffff;  // min / max of the source ranks follow
      p.tile_seg_end[first_tile + t] = p.segments > 1 ? seg : -1;            // in the scatter kernel
    }
    if (lane == 0 && e == p.num_experts - 1) p.totals[2 + seg] = (off + padded) / p.block_m;  // cumulative
  }
  if (tid == 0) {
    p.totals[0] = carry;
    p.totals[1] = carry / p.block_m;
  }
}

// ---- 4. scatter: stable rank of every pair among the pairs of its expert in the chunk
__global__ void __launch_bounds__(kChunk) moe_scatter_kernel(const MoeSortParams p) {
  __shared__ int32_t sid[kChunk];
  const int seg = blockIdx.x / p.chunks_per_segment, c = blockIdx.x - seg * p.chunks_per_segment;
  const int i = c * kChunk + threadIdx.x;
  const int pair = seg * p.pairs_per_segment + i;
  int e = -1;
  if (i < p.pairs_per_segment) {
    e = p.ids[pair];
    if (e < 0 || e >= p.num_experts) e = -1;
  }
  sid[threadIdx.x] = e;
  __syncthreads();
  int rank = 0;
  const int tid = threadIdx.x;
  const int warp_first = tid & ~31;
  for (int j = 0; j < warp_first; ++j) rank += sid[j] == e ? 1 : 0;   // uniform over the warp: broadcast reads
  const uint32_t same = __match_any_sync(0xffffffffu, e);              // skipped lanes (e == -1) only match each other
  rank += __popc(same & ((1u << (tid & 31)) - 1u));
  if (e < 0) return;
  const int pos = p.group_off[seg * p.num_experts + e] + p.chunk_cnt[static_cast<size_t>(blockIdx.x) * p.num_experts + e] + rank;
  p.sorted_ids[pos] = pair;
  if (p.pair_pos) p.pair_pos[pair] = pos;
  if (p.segments == 1) {
    const int src = (pair / p.topk) / p.tokens_per_rank;
    const int tile = pos / p.block_m;
    atomicMin(p.tile_seg_start + tile, src);
    atomicMax(p.tile_seg_end + tile, src);
  }
}

// ---- small problems in ONE launch (B200DIST_MOE_SORT_SMALL=0 turns it off): at most 8192 pairs and 1024 (segment, expert)
// groups. One CTA of 32 warps; warp w owns a contiguous block of pairs and counts them per group in its own row of a
// shared [32][G] table (one leader lane per distinct group and 32-pair chunk, so no atomics), which also gives every
// pair its rank among the warp's pairs of the same group. A scan over the warps per group, a scan over the groups,
// and every pair knows its position. Same outputs as the four-kernel path.
constexpr int kSmallMaxPerLane = 8;

__global__ void __launch_bounds__(1024) moe_sort_small_kernel(const MoeSortParams p) {
  extern __shared__ int32_t wcnt[];          // [32][G] per-warp counts, then exclusive offsets over the warps
  __shared__ int32_t warp_tot[32];
  __shared__ int32_t carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.segments * p.num_experts;
  for (int i = tid; i < 32 * G; i += 1024) wcnt[i] = 0;
  if (tid == 0) carry = 0;
  __syncthreads();
  // warp w owns pairs [w * per_warp, (w + 1) * per_warp), per_warp a multiple of 32
  const int per_warp = ((p.n_pairs + 31) / 32 + 31) / 32 * 32;
  const int w0 = warp * per_warp;
  int my_group[kSmallMaxPerLane], my_rank[kSmallMaxPerLane];
  int32_t* mine = wcnt + warp * G;
#pragma unroll
  for (int k = 0; k < kSmallMaxPerLane; ++k) {
    my_group[k] = -1;
    my_rank[k] = 0;
    if (k * 32 < per_warp) {   // uniform over the warp
      const int pair = w0 + k * 32 + lane;
      int g = -1;
      if (pair < p.n_pairs) {
        const int e = p.ids[pair];
        if (e >= 0 && e < p.num_experts) g = (pair / p.pairs_per_segment) * p.num_experts + e;
      }
      const uint32_t same = __match_any_sync(0xffffffffu, g);
      const int leader = __ffs(same) - 1;
      int old = 0;
      if (g >= 0 && lane == leader) {
        old = mine[g];
        mine[g] = old + __popc(same);
      }
      old = __shfl_sync(0xffffffffu, old, leader);
      my_group[k] = g;
      my_rank[k] = old + __popc(same & ((1u << lane) - 1u));
      __syncwarp();
    }
  }
  __syncthreads();
  // per group: exclusive scan of the counts over the warps, total, padded size
  for (int g0 = 0; g0 < G; g0 += 1024) {
    const int g = g0 + tid;
    int total = 0;
    if (g < G) {
      for (int w = 0; w < 32; ++w) {
        const int v = wcnt[w * G + g];
        wcnt[w * G + g] = total;
        total += v;
      }
      p.group_count[g] = total;
    }
    const int padded = (total + p.block_m - 1) / p.block_m * p.block_m;
    int incl = padded;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int off = before + incl - padded;
    if (g < G) {
      p.group_off[g] = off;
      const int seg = g / p.num_experts, e = g - seg * p.num_experts;
      for (int i = total; i < padded; ++i) p.sorted_ids[off + i] = p.n_pairs;
      for (int t = 0; t < padded / p.block_m; ++t) {
        p.tile_expert[off / p.block_m + t] = e;
        p.tile_seg_start[off / p.block_m + t] = p.segments > 1 ? seg : 0x7fffffff;
        p.tile_seg_end[off / p.block_m + t] = p.segments > 1 ? seg : -1;
      }
      if (e == p.num_experts - 1) p.totals[2 + seg] = (off + padded) / p.block_m;
    }
    __syncthreads();
    if (tid == 1023) carry = off + padded;
    __syncthreads();
  }
  if (tid == 0) {
    p.totals[0] = carry;
    p.totals[1] = carry / p.block_m;
  }
  __threadfence_block();
  __syncthreads();   // group_off and the tile table (global memory, this CTA) are visible to every thread
#pragma unroll
  for (int k = 0; k < kSmallMaxPerLane; ++k) {
    const int g = my_group[k];
    if (g >= 0) {
      const int pair = w0 + k * 32 + lane;
      const int pos = p.group_off[g] + wcnt[warp * G + g] + my_rank[k];
      p.sorted_ids[pos] = pair;
      if (p.pair_pos) p.pair_pos[pair] = pos;
      if (p.segments == 1) {
        const int src = (pair / p.topk) / p.tokens_per_rank;
        const int tile = pos / p.block_m;
        atomicMin(p.tile_seg_start + tile, src);
        atomicMax(p.tile_seg_end + tile, src);
      }
    }
  }
}

// Stable counting sort of the tiles by stage; one CTA. order[j] = tile issued j-th.
// The stage of a tile is the ring step (starting at `rank`) after which ALL of its source shards have arrived: a tile
// whose sources seg_start..seg_end run past rank - 1 holds a row of the last shard to arrive.
__global__ void __launch_bounds__(1024) moe_tile_order_kernel(const int32_t* tile_seg_start, const int32_t* tile_seg_end,
                                                              const int32_t* totals, int rank, int world, int shift,
                                                              int32_t* order) {
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
        if (tile_seg_start != nullptr) {
          int first = (tile_seg_start[t] - rank - shift) % world;
          if (first < 0) first += world;
          if (first > st) st = world - 1;  // the range wraps around this rank
        }
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

static bool small_sort_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200DIST_MOE_SORT_SMALL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

// Scratch (int32 elements) that b200_moe_sort needs for a problem of this size.
B200_API long long b200_moe_sort_scratch_ints(int n_pairs, int num_experts, int segments) {
  const long long pps = n_pairs / (segments > 0 ? segments : 1);
  const long long chunks = (pps + kChunk - 1) / kChunk;
  return (chunks * segments + 1) * num_experts + static_cast<long long>(segments) * num_experts;
}

// ids int32 [n_pairs]; outputs sized by b200_moe_sorted_capacity (rows) and capacity / block_m (tiles).
// group_count int32 [segments * E]; totals int32 [2 + segments]; scratch int32 [b200_moe_sort_scratch_ints(...)]
// (no initialisation needed); pair_pos (nullable) int32 [n_pairs]. Ids outside [0, E) are skipped.
B200_API int b200_moe_sort(const int32_t* ids, int n_pairs, int topk, int num_experts, int block_m, int segments,
                           int tokens_per_rank, int32_t* sorted_ids, int32_t* tile_expert, int32_t* tile_seg_start,
                           int32_t* tile_seg_end, int32_t* group_count, int32_t* totals, int32_t* scratch,
                           int32_t* pair_pos, void* stream) {
  B200_REQUIRE(num_experts >= 1 && num_experts <= 1024, "number of experts (%d) must be in [1, 1024]", num_experts);
  B200_REQUIRE(segments >= 1 && n_pairs % segments == 0, "pairs (%d) must divide into %d segments", n_pairs, segments);
  B200_REQUIRE(block_m >= 1 && topk >= 1 && tokens_per_rank >= 1, "bad block_m / topk / tokens_per_rank");
  B200_REQUIRE(n_pairs >= 1, "no pairs to sort");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MoeSortParams p;
  memset(&p, 0, sizeof(p));
  p.ids = ids; p.n_pairs = n_pairs; p.topk = topk; p.num_experts = num_experts; p.block_m = block_m;
  p.segments = segments; p.pairs_per_segment = n_pairs / segments; p.tokens_per_rank = tokens_per_rank;
  p.chunks_per_segment = (p.pairs_per_segment + kChunk - 1) / kChunk;
  p.sorted_ids = sorted_ids; p.tile_expert = tile_expert; p.tile_seg_start = tile_seg_start; p.tile_seg_end = tile_seg_end;
  p.pair_pos = pair_pos;
  p.group_count = group_count; p.totals = totals;
  p.chunk_cnt = scratch;
  p.group_off = scratch + static_cast<size_t>(p.chunks_per_segment) * segments * num_experts;
  const int chunks = p.chunks_per_segment * segments;
  if (small_sort_enabled() && n_pairs <= 32 * 32 * kSmallMaxPerLane && segments * num_experts <= 1024) {
    const size_t smem = static_cast<size_t>(32) * segments * num_experts * sizeof(int32_t);
    static bool configured[64] = {false};
    int dev = 0;
    B200_CHECK_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
      B200_CHECK_CUDA(cudaFuncSetAttribute(moe_sort_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
      configured[dev & 63] = true;
    }
    moe_sort_small_kernel<<<1, 1024, smem, s>>>(p);
    B200_CHECK_CUDA(cudaGetLastError());
    return kOk;
  }
  moe_count_kernel<<<chunks, kChunk, num_experts * sizeof(int32_t), s>>>(p);
  moe_chunk_prefix_kernel<<<dim3((num_experts + 31) / 32, segments), 1024, 0, s>>>(p);
  moe_offsets_kernel<<<1, 1024, 0, s>>>(p);
  moe_scatter_kernel<<<chunks, kChunk, 0, s>>>(p);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

B200_API int b200_moe_tile_order(const int32_t* tile_seg_start, const int32_t* tile_seg_end, const int32_t* totals, int rank, int world, int shift,
                                 int32_t* order, void* stream) {
  B200_REQUIRE(world >= 1 && world <= kMaxRanks, "world (%d) out of range", world);
  moe_tile_order_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(tile_seg_start, tile_seg_end, totals, rank, world, shift, order);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
