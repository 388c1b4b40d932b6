// Top-p (nucleus) sampling in one kernel, one CTA per row, without sorting.
//
// The nucleus of a row is {i : p_i >= t*} where t* is the largest threshold whose kept mass still reaches
// top_p; that is the same set a descending sort + cumulative sum selects (up to ties), but it can be found
// by bisection on t with one block reduction per step, so the 152K-entry vocabulary is never sorted or
// scanned in global memory. The token is then drawn from the kept entries in index order with one uniform
// random number per row supplied by the caller.
//
// Role in the reference: flashinfer.sampling.top_p_sampling_from_probs behind sample_token
// (python/triton_dist/models/utils.py:77-96).
#include "b200/host.h"
#include "b200/primitives.cuh"

namespace b200 {

constexpr int kSampleThreads = 1024;

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

__global__ void __launch_bounds__(kSampleThreads) top_p_sample_kernel(const float* __restrict__ logits, int ld, int V,
                                                                      float inv_temperature, float top_p,
                                                                      const float* __restrict__ uniform,
                                                                      long long* __restrict__ out) {
  __shared__ float red[33];
  __shared__ float prefix[kSampleThreads];
  __shared__ int chosen;
  const float* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  const int tid = threadIdx.x;

  float mx = -INFINITY;
  int arg = 0;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float v = row[i];
    if (v > mx) { mx = v; arg = i; }
  }
  const float gmax = block_reduce_max(mx, red);
  // lowest index attaining the maximum: the fallback choice
  if (tid == 0) chosen = 0x7fffffff;
  __syncthreads();
  if (mx == gmax) atomicMin(&chosen, arg);
  float z = 0.f;
  for (int i = tid; i < V; i += kSampleThreads) z += __expf((row[i] - gmax) * inv_temperature);
  const float Z = block_reduce_sum(z, red);
  const float inv_z = 1.f / Z;

  // bisection on the probability threshold: mass(lo) >= top_p > mass(hi)
  float lo = 0.f, hi = inv_z * 1.0001f;
  if (top_p < 1.f) {
    for (int it = 0; it < 18; ++it) {
      const float mid = 0.5f * (lo + hi);
      float m = 0.f;
      for (int i = tid; i < V; i += kSampleThreads) {
        const float p = __expf((row[i] - gmax) * inv_temperature) * inv_z;
        m += p >= mid ? p : 0.f;
      }
      const float mass = block_reduce_sum(m, red);
      if (mass >= top_p) lo = mid; else hi = mid;
    }
  }
  // draw in index order among the kept entries: thread t owns the contiguous chunk [c0, c1)
  const int per = (V + kSampleThreads - 1) / kSampleThreads;
  const int c0 = min(V, tid * per), c1 = min(V, c0 + per);
  float mine = 0.f;
  for (int i = c0; i < c1; ++i) {
    const float p = __expf((row[i] - gmax) * inv_temperature) * inv_z;
    mine += p >= lo ? p : 0.f;
  }
  prefix[tid] = mine;
  __syncthreads();
  // inclusive scan over 1024 chunk sums (Hillis-Steele in shared memory)
  for (int off = 1; off < kSampleThreads; off <<= 1) {
    const float add = tid >= off ? prefix[tid - off] : 0.f;
    __syncthreads();
    prefix[tid] += add;
    __syncthreads();
  }
  const float total = prefix[kSampleThreads - 1];
  const float target = uniform[blockIdx.x] * total;
  const float before = prefix[tid] - mine;
  if (mine > 0.f && target >= before && target < prefix[tid]) {
    float acc = before;
    int pick = -1;
    for (int i = c0; i < c1; ++i) {
      const float p = __expf((row[i] - gmax) * inv_temperature) * inv_z;
      if (p >= lo) {
        acc += p;
        pick = i;
        if (acc > target) break;
      }
    }
    if (pick >= 0) chosen = pick;
  }
  __syncthreads();
  if (tid == 0) out[blockIdx.x] = chosen;
}

}  // namespace b200

using namespace b200;

// logits fp32 [B, V] with row pitch ld; uniform fp32 [B] in [0, 1); out int64 [B].
B200_API int b200_top_p_sample(const float* logits, int ld, int B, int V, float temperature, float top_p,
                               const float* uniform, long long* out, void* stream) {
  B200_REQUIRE(temperature > 0.f, "temperature must be positive (use argmax for greedy decoding)");
  B200_REQUIRE(top_p > 0.f, "top_p must be positive");
  if (B == 0) return kOk;
  top_p_sample_kernel<<<B, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(logits, ld, V, 1.f / temperature,
                                                                                   top_p, uniform, out);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
