// Merge of the split-KV partial results of decode attention (one output element per thread).
//
// Every split s of a (sequence, head) row leaves a normalised partial output o_s[128] and the log-sum-exp lse_s of
// its scores; an empty split leaves lse_s = -inf and an undefined o_s. The merged row is
//   o = sum_s exp(lse_s - m) o_s / sum_s exp(lse_s - m),   lse = m + log(sum_s exp(lse_s - m)),   m = max_s lse_s.
// The loop takes eight splits per pass and issues their sixteen loads before it uses any of them, carrying a running
// maximum, so the merge costs one memory round trip per eight splits instead of one per split (a loop that tests
// lse_s before it loads o_s cannot overlap its loads). Loads bypass L1 because in the single-launch decode the
// partials were written by other CTAs of the same kernel.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>

namespace b200 {

__device__ __forceinline__ void merge_splits(const float* lse, long long lse_stride, const float* o, long long o_stride,
                                             int S, float& o_out, float& lse_out) {
  float m = -CUDART_INF_F, den = 0.f, acc = 0.f;
  for (int s0 = 0; s0 < S; s0 += 8) {
    float l[8], v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = s0 + j < S;
      l[j] = in ? __ldcg(lse + (s0 + j) * lse_stride) : -CUDART_INF_F;
      v[j] = in ? __ldcg(o + (s0 + j) * o_stride) : 0.f;
    }
    float bm = m;
#pragma unroll
    for (int j = 0; j < 8; ++j) bm = fmaxf(bm, l[j]);
    if (bm == -CUDART_INF_F) continue;  // nothing but empty splits so far
    const float rescale = __expf(m - bm);  // exp(-inf) = 0 on the first non-empty pass
    den *= rescale;
    acc *= rescale;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (l[j] != -CUDART_INF_F) {
        const float w = __expf(l[j] - bm);
        den += w;
        acc += w * v[j];
      }
    }
    m = bm;
  }
  o_out = den > 0.f ? acc / den : 0.f;
  lse_out = den > 0.f ? m + logf(den) : -CUDART_INF_F;
}

}  // namespace b200
