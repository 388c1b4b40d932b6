// Top-p (nucleus) sampling in one kernel, one cluster of eight CTAs per row, without sorting.
//
// The nucleus of a row is {i : p_i >= t*} where t* is the largest threshold whose kept mass still reaches
// top_p; that is the same set a descending sort + cumulative sum selects (up to ties), but it can be found
// from two shared-memory histograms of probability mass, so the 152K-entry vocabulary is never sorted or
// scanned in global memory. The token is then drawn from the kept entries in index order with one uniform
// random number per row supplied by the caller.
//
// Role in the reference: flashinfer.sampling.top_p_sampling_from_probs behind sample_token
// (python/triton_dist/models/utils.py:77-96).
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cooperative_groups.h>

namespace b200 {

constexpr int kSampleThreads = 1024;
constexpr int kSampleCtas = 8;  // CTAs (one cluster) per row

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) {
    t = warp_max(t);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Strided pass over the slice [lo, hi) of a row (lo a multiple of 4) with four independent 16-byte loads in flight
// per thread. f(index, value) is called for every element.
template <typename F>
__device__ __forceinline__ void for_range(const float* __restrict__ row, int lo, int hi, F f) {
  const int tid = threadIdx.x;
  int done = lo;
  if ((reinterpret_cast<uintptr_t>(row + lo) & 15u) == 0) {
    const int nvec = (hi - lo) / 4;
    const float4* r4 = reinterpret_cast<const float4*>(row + lo);
    int i = tid;
    for (; i + 3 * kSampleThreads < nvec; i += 4 * kSampleThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = r4[i + u * kSampleThreads];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int b = lo + (i + u * kSampleThreads) * 4;
        f(b, v[u].x); f(b + 1, v[u].y); f(b + 2, v[u].z); f(b + 3, v[u].w);
      }
    }
    for (; i < nvec; i += kSampleThreads) {
      const float4 v = r4[i];
      const int b = lo + i * 4;
      f(b, v.x); f(b + 1, v.y); f(b + 2, v.z); f(b + 3, v.w);
    }
    done = lo + nvec * 4;
  }
  for (int i = done + tid; i < hi; i += kSampleThreads) f(i, row[i]);
}

// Histogram cells are 64-bit fixed point (2^-40): integer shared-memory atomics are native and exact, float ones
// are compare-and-swap loops that serialise when neighbouring logits fall into the same bin.
typedef unsigned long long u64;
__device__ __forceinline__ u64 to_fixed(float e) { return static_cast<u64>(e * 1099511627776.f); }

// Inclusive scan of 1024 cells in shared memory (one per thread), Hillis-Steele.
__device__ __forceinline__ void scan1024(u64* a) {
  const int tid = threadIdx.x;
  for (int off = 1; off < kSampleThreads; off <<= 1) {
    const u64 add = tid >= off ? a[tid - off] : 0ull;
    __syncthreads();
    a[tid] += add;
    __syncthreads();
  }
}
// First index whose inclusive prefix reaches `target` (kSampleThreads - 1 when none does).
__device__ __forceinline__ int first_reaching(const u64* incl, u64 target, int* slot) {
  const int tid = threadIdx.x;
  if (tid == 0) *slot = kSampleThreads - 1;
  __syncthreads();
  if (incl[tid] >= target && (tid == 0 || incl[tid - 1] < target)) *slot = tid;
  __syncthreads();
  return *slot;
}

// The nucleus threshold is found with two histograms over z = (max - logit) / T instead of a sort or a
// bisection: 1024 bins of width 1/32 locate the bin in which the kept mass crosses top_p, 1024 sub-bins of that
// bin pin the threshold to a relative probability error of e^(1/32768).
//
// A row is spread over a cluster of eight CTAs (a decode batch has few rows, and one SM cannot stream a 600 KB row
// fast enough): every CTA works on an eighth of the vocabulary and the CTAs exchange their maxima, histograms and
// kept masses through distributed shared memory. Four passes over the slice in total.
__global__ void __cluster_dims__(kSampleCtas, 1, 1) __launch_bounds__(kSampleThreads)
top_p_sample_kernel(const float* __restrict__ logits, int ld, int V, float inv_temperature, float top_p,
                    const float* __restrict__ uniform, long long* __restrict__ out) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[33];
  __shared__ u64 cells_a[kSampleThreads], cells_b[kSampleThreads], merged[kSampleThreads];
  __shared__ float hist[32];
  __shared__ int chosen, slot;
  __shared__ float x_max, x_mass;          // read by the other CTAs of the cluster
  __shared__ int x_arg;
  __shared__ float all_max[kSampleCtas], all_mass[kSampleCtas];
  __shared__ int all_arg[kSampleCtas];
  const int crank = static_cast<int>(cluster.block_rank());
  const int row_id = blockIdx.x / kSampleCtas;
  const float* row = logits + static_cast<size_t>(row_id) * ld;
  const int tid = threadIdx.x;
  const int per = ((V + kSampleCtas - 1) / kSampleCtas + 3) & ~3;
  const int lo = min(V, crank * per), hi = min(V, lo + per);
  griddep_launch_dependents();
  griddep_wait();

  // ---- pass 1: maximum and the lowest index attaining it
  float mx = -INFINITY;
  int arg = 0x7fffffff;
  for_range(row, lo, hi, [&](int i, float v) {
    if (v > mx || (v == mx && i < arg)) { mx = v; arg = i; }
  });
  const float lmax = block_reduce_max(mx, red);
  if (tid == 0) chosen = 0x7fffffff;
  cells_a[tid] = 0ull;
  cells_b[tid] = 0ull;
  __syncthreads();
  if (mx == lmax && arg != 0x7fffffff) atomicMin(&chosen, arg);
  __syncthreads();
  if (tid == 0) { x_max = lmax; x_arg = chosen; }
  cluster.sync();
  if (tid < kSampleCtas) {
    all_max[tid] = *cluster.map_shared_rank(&x_max, tid);
    all_arg[tid] = *cluster.map_shared_rank(&x_arg, tid);
  }
  __syncthreads();
  float gmax = -INFINITY;
  int garg = 0x7fffffff;
#pragma unroll
  for (int c = 0; c < kSampleCtas; ++c) {
    if (all_max[c] > gmax || (all_max[c] == gmax && all_arg[c] < garg)) { gmax = all_max[c]; garg = all_arg[c]; }
  }
  __syncthreads();
  if (tid == 0) chosen = garg;  // the fallback choice

  float thr_z = INFINITY;  // keep entries with z < thr_z
  if (top_p < 1.f) {
    // ---- pass 2: coarse histogram of probability mass over z
    for_range(row, lo, hi, [&](int, float v) {
      const float z = (gmax - v) * inv_temperature;  // >= 0
      atomicAdd(cells_a + min(kSampleThreads - 1, static_cast<int>(z * 32.f)), to_fixed(__expf(-z)));
    });
    cluster.sync();
    u64 sum = 0ull;
#pragma unroll
    for (int c = 0; c < kSampleCtas; ++c) sum += cluster.map_shared_rank(cells_a, c)[tid];
    merged[tid] = sum;
    __syncthreads();
    scan1024(merged);
    const u64 target = static_cast<u64>(static_cast<double>(top_p) * static_cast<double>(merged[kSampleThreads - 1]));
    const int b = first_reaching(merged, target, &slot);
    const u64 before = b > 0 ? merged[b - 1] : 0ull;
    __syncthreads();
    // ---- pass 3: refine inside bin b
    for_range(row, lo, hi, [&](int, float v) {
      const float z = (gmax - v) * inv_temperature;
      const float zb = z * 32.f;
      if (min(kSampleThreads - 1, static_cast<int>(zb)) == b)
        atomicAdd(cells_b + min(kSampleThreads - 1, max(0, static_cast<int>((zb - b) * 1024.f))), to_fixed(__expf(-z)));
    });
    cluster.sync();
    sum = 0ull;
#pragma unroll
    for (int c = 0; c < kSampleCtas; ++c) sum += cluster.map_shared_rank(cells_b, c)[tid];
    merged[tid] = sum;
    __syncthreads();
    scan1024(merged);
    const int sb = first_reaching(merged, target > before ? target - before : 0ull, &slot);
    thr_z = b == kSampleThreads - 1 ? INFINITY : (b + (sb + 1) * (1.f / 1024.f)) * (1.f / 32.f);
    __syncthreads();
  }
  // ---- pass 4: draw in index order among the kept entries. Inside the CTA's slice, warp w owns the contiguous
  // range [lo + w * R, lo + (w + 1) * R), cut into 32 sub-blocks of S entries; lane j ends up with the kept mass of
  // sub-block j (coalesced reads). The target is located by CTA, by warp, by sub-block, then by a walk of S / 32 steps.
  const int lane = tid & 31, warp = tid >> 5;
  const int S = ((per + 1023) / 1024 + 31) / 32 * 32;  // multiple of 32, 32 * 32 * S >= per
  const int R = 32 * S;
  const int r0 = min(hi, lo + warp * R), r1 = min(hi, r0 + R);
  auto kept_mass = [&](int i) -> float {
    if (i >= r1) return 0.f;
    const float z = (gmax - row[i]) * inv_temperature;
    return z < thr_z ? __expf(-z) : 0.f;
  };
  float sub = 0.f;  // lane j: mass of sub-block j
  for (int j = 0; j < 32; j += 2) {
    float m0 = 0.f, m1 = 0.f;
    const int b0 = r0 + j * S, b1 = b0 + S;
    if (b0 < r1) {
      for (int k = lane; k < S; k += 32) {
        m0 += kept_mass(b0 + k);
        m1 += kept_mass(b1 + k);
      }
    }
    m0 = warp_sum(m0);
    m1 = warp_sum(m1);
    if (lane == j) sub = m0;
    if (lane == j + 1) sub = m1;
  }
  float sub_incl = sub;  // inclusive scan of the sub-block masses over the lanes
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, sub_incl, o);
    if (lane >= o) sub_incl += v;
  }
  const float mine = __shfl_sync(0xffffffffu, sub_incl, 31);
  __syncthreads();
  if (lane == 0) hist[warp] = mine;
  __syncthreads();
  float incl = hist[lane];  // every warp scans the 32 warp totals
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  const float cta_mass = __shfl_sync(0xffffffffu, incl, 31);
  if (tid == 0) x_mass = cta_mass;
  cluster.sync();
  if (tid < kSampleCtas) all_mass[tid] = *cluster.map_shared_rank(&x_mass, tid);
  __syncthreads();
  float cta_before = 0.f, total = 0.f;
#pragma unroll
  for (int c = 0; c < kSampleCtas; ++c) {
    if (c < crank) cta_before += all_mass[c];
    total += all_mass[c];
  }
  const float target = uniform[row_id] * total;
  // the CTA whose interval holds the target; rounding at the upper end goes to the last CTA that kept anything
  int sel = -1, last_nonempty = 0;
  {
    float run = 0.f;
#pragma unroll
    for (int c = 0; c < kSampleCtas; ++c) {
      if (all_mass[c] > 0.f) {
        last_nonempty = c;
        if (sel < 0 && target < run + all_mass[c]) sel = c;
      }
      run += all_mass[c];
    }
    if (sel < 0) sel = last_nonempty;
  }
  if (crank == sel) {
    const float my_incl = cta_before + __shfl_sync(0xffffffffu, incl, warp);
    const float my_before = my_incl - mine;
    // warp whose interval holds the target (rounding: the last warp that kept anything)
    const float w_incl = cta_before + incl;  // lane l: inclusive mass up to warp l
    const uint32_t wpass = __ballot_sync(0xffffffffu, hist[lane] > 0.f && target < w_incl);
    const uint32_t wnonempty = __ballot_sync(0xffffffffu, hist[lane] > 0.f);
    const int wsel = wpass ? __ffs(wpass) - 1 : 31 - __clz(wnonempty | 1u);
    if (warp == wsel && mine > 0.f) {
      const uint32_t pass = __ballot_sync(0xffffffffu, sub > 0.f && my_before + sub_incl > target);
      const uint32_t nonempty = __ballot_sync(0xffffffffu, sub > 0.f);
      const int jsel = pass ? __ffs(pass) - 1 : 31 - __clz(nonempty);
      float acc = my_before + __shfl_sync(0xffffffffu, sub_incl - sub, jsel);
      int pick = -1, last_kept = -1;
      const int s0 = r0 + jsel * S, s1 = min(r1, s0 + S);
      for (int b0 = s0; b0 < s1 && pick < 0; b0 += 32) {
        const float m = kept_mass(b0 + lane);
        float sc = m;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float v = __shfl_up_sync(0xffffffffu, sc, o);
          if (lane >= o) sc += v;
        }
        const uint32_t hit = __ballot_sync(0xffffffffu, m > 0.f && acc + sc > target);
        const uint32_t kept = __ballot_sync(0xffffffffu, m > 0.f);
        if (hit) pick = b0 + __ffs(hit) - 1;
        else if (kept) last_kept = b0 + 31 - __clz(kept);
        acc += __shfl_sync(0xffffffffu, sc, 31);
      }
      if (pick < 0) pick = last_kept;  // rounding: the last kept entry of the sub-block
      if (pick >= 0 && lane == 0) chosen = pick;
    }
    __syncthreads();
    if (tid == 0) out[row_id] = chosen;
  }
  cluster.sync();  // no CTA's shared memory goes away while a peer may still read it
}

}  // namespace b200

using namespace b200;

// logits fp32 [B, V] with row pitch ld; uniform fp32 [B] in [0, 1); out int64 [B].
B200_API int b200_top_p_sample(const float* logits, int ld, int B, int V, float temperature, float top_p,
                               const float* uniform, long long* out, void* stream) {
  B200_REQUIRE(temperature > 0.f, "temperature must be positive (use argmax for greedy decoding)");
  B200_REQUIRE(top_p > 0.f, "top_p must be positive");
  if (B == 0) return kOk;
  top_p_sample_kernel<<<B * kSampleCtas, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(logits, ld, V, 1.f / temperature,
                                                                                   top_p, uniform, out);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
