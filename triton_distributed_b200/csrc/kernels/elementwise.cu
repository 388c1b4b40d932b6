// Memory-bound model ops, one pass over HBM each:
//   rmsnorm          y = (x [+ residual]) * rsqrt(mean(x^2) + eps) * gamma, optionally emitting the new residual
//   qk_norm_rope     per-head RMSNorm of q and k, neox-style rotary embedding from a cos|sin cache, and the
//                    write of k / v into the paged KV cache, all in one kernel over the fused qkv projection
//   silu_mul         SwiGLU gate: silu(gate) * up over a fused [gate | up] projection
//   topk_softmax     router: softmax over experts + top-k (ids, weights)
//   embedding        out[t] = table[ids[t]] (token embedding lookup, 16-byte vectors)
//
// Role in the reference: flashinfer.norm.rmsnorm, flashinfer.apply_rope_with_cos_sin_cache_inplace and
// the unfused torch act_fn(gate) * up (python/triton_dist/layers/nvidia/tp_attn.py:60-75,159-195,
// tp_mlp.py:159-160), and the softmax/topk of select_experts (kernels/nvidia/moe_reduce_rs.py:172-189).
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>
#include <cuda_fp8.h>

namespace b200 {

template <bool BF16>
__device__ __forceinline__ void unpack8(uint4 v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = BF16 ? unpack_bf16x2(w[i]) : unpack_f16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float* f) {
  return BF16 ? make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]))
              : make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
}

// One CTA per row (grid-strided). hidden % 8 == 0 and hidden <= 8 * 4 * blockDim.x.
template <bool BF16>
__global__ void __launch_bounds__(512) rmsnorm_kernel(const uint4* __restrict__ x, const uint4* residual_in,
                                                      uint4* residual_out, const uint4* __restrict__ gamma,
                                                      uint4* __restrict__ y, int rows, int hidden, float eps) {
  __shared__ float red[32];
  const int nv = hidden / 8;
  griddep_launch_dependents();
  // the gain is a weight (not an output of the kernel launched just before this one): it is fetched before the
  // dependency wait, past L1, and stays in registers for every row
  uint4 gv[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = threadIdx.x + u * blockDim.x;
    gv[u] = i < nv ? __ldcg(gamma + i) : make_uint4(0, 0, 0, 0);
  }
  griddep_wait();
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    // every load of the row is issued before the first store: residual_in may alias residual_out, so a load placed
    // after a store has to wait for it, which would make this one memory round trip per chunk
    uint4 xv[4], rv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      xv[u] = rv[u] = make_uint4(0, 0, 0, 0);
      if (i < nv) {
        xv[u] = x[static_cast<size_t>(r) * nv + i];
        if (residual_in) rv[u] = residual_in[static_cast<size_t>(r) * nv + i];
      }
    }
    float v[4][8];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      if (i < nv) {
        unpack8<BF16>(xv[u], v[u]);
        if (residual_in) {
          float q[8];
          unpack8<BF16>(rv[u], q);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[u][e] += q[e];
          const uint4 packed = pack8<BF16>(v[u]);
          if (residual_out) residual_out[static_cast<size_t>(r) * nv + i] = packed;
          unpack8<BF16>(packed, v[u]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[u][e] * v[u][e];
      }
    }
    ss = warp_sum(ss);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    if (threadIdx.x < 32) {
      tot = warp_sum(tot);
      if (threadIdx.x == 0) red[0] = tot;
    }
    __syncthreads();
    const float inv = rsqrtf(red[0] / hidden + eps);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      if (i < nv) {
        float g[8], o[8];
        unpack8<BF16>(gv[u], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[u][e] * inv * g[e];
        y[static_cast<size_t>(r) * nv + i] = pack8<BF16>(o);
      }
    }
  }
}

// One warp per (token, head) of the fused projection qkv[T, (Hq + 2 Hkv) * 128]. Lane l owns elements
// 4l..4l+3 of the head; the rotary partner (i +- 64) sits in lane l ^ 16.
//   q heads  -> RMSNorm(q_gamma) -> RoPE -> q_out[T, Hq, 128]
//   k heads  -> RMSNorm(k_gamma) -> RoPE -> k_cache[slot[t], h, :]
//   v heads  -> v_cache[slot[t], h, :]
// cos_sin is [max_pos, 128] = cos(64) | sin(64) in fp32. gamma pointers may be null (no head norm).
template <bool BF16>
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const uint2* __restrict__ qkv, const int* __restrict__ positions,
                                                           const int64_t* __restrict__ slots, const uint2* q_gamma,
                                                           const uint2* k_gamma, const float* __restrict__ cos_sin,
                                                           uint2* __restrict__ q_out, uint2* k_cache, uint2* v_cache,
                                                           int T, int Hq, int Hkv, float eps) {
  const int heads = Hq + 2 * Hkv;
  griddep_launch_dependents();
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int t = warp_global / heads;
  const int h = warp_global - t * heads;
  const uint2* gamma = h < Hq ? q_gamma : k_gamma;
  // the gains are weights (not outputs of the kernel launched just before this one): fetched before the wait, past L1
  const uint2 g = (gamma != nullptr && warp_global < T * heads && h < Hq + Hkv) ? __ldcg(gamma + lane) : make_uint2(0, 0);
  griddep_wait();
  if (warp_global >= T * heads) return;
  const uint2 raw = qkv[(static_cast<size_t>(t) * heads + h) * 32 + lane];
  const int64_t slot = slots ? slots[t] : t;
  const int pos = positions[t];
  if (h >= Hq + Hkv) {  // v: straight copy into the cache
    if (slot >= 0) v_cache[(static_cast<size_t>(slot) * Hkv + (h - Hq - Hkv)) * 32 + lane] = raw;
    return;
  }
  float x[4];
  {
    const float2 a = BF16 ? unpack_bf16x2(raw.x) : unpack_f16x2(raw.x);
    const float2 b = BF16 ? unpack_bf16x2(raw.y) : unpack_f16x2(raw.y);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  }
  if (gamma) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / 128.f + eps);
    const float2 ga = BF16 ? unpack_bf16x2(g.x) : unpack_f16x2(g.x);
    const float2 gb = BF16 ? unpack_bf16x2(g.y) : unpack_f16x2(g.y);
    // round to the storage dtype after the norm, as a separate norm kernel would
    float n0 = x[0] * inv * ga.x, n1 = x[1] * inv * ga.y, n2 = x[2] * inv * gb.x, n3 = x[3] * inv * gb.y;
    const float2 r0 = BF16 ? unpack_bf16x2(pack_bf16x2(n0, n1)) : unpack_f16x2(pack_f16x2(n0, n1));
    const float2 r1 = BF16 ? unpack_bf16x2(pack_bf16x2(n2, n3)) : unpack_f16x2(pack_f16x2(n2, n3));
    x[0] = r0.x; x[1] = r0.y; x[2] = r1.x; x[3] = r1.y;
  }
  // neox rotation: out[i] = x[i] cos[i] - x[i+64] sin[i] (i < 64); out[i+64] = x[i+64] cos[i] + x[i] sin[i]
  const int fi = (lane & 15) * 4;  // frequency index of this lane's first element
  const float4 c = *reinterpret_cast<const float4*>(cos_sin + static_cast<size_t>(pos) * 128 + fi);
  const float4 s = *reinterpret_cast<const float4*>(cos_sin + static_cast<size_t>(pos) * 128 + 64 + fi);
  const float cs[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
  float o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float partner = __shfl_xor_sync(0xffffffffu, x[e], 16);
    o[e] = lane < 16 ? x[e] * cs[e] - partner * sn[e] : x[e] * cs[e] + partner * sn[e];
  }
  uint2 outv;
  outv.x = BF16 ? pack_bf16x2(o[0], o[1]) : pack_f16x2(o[0], o[1]);
  outv.y = BF16 ? pack_bf16x2(o[2], o[3]) : pack_f16x2(o[2], o[3]);
  if (h < Hq) {
    q_out[(static_cast<size_t>(t) * Hq + h) * 32 + lane] = outv;
  } else if (slot >= 0) {
    k_cache[(static_cast<size_t>(slot) * Hkv + (h - Hq)) * 32 + lane] = outv;
  }
}

// out[t, i] = silu(x[t, i]) * x[t, inter + i]; x is [T, 2 * inter] with row pitch ldx.
template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, int T,
                                                       int inter, int ldx) {
  const int nv = inter / 8;
  griddep_launch_dependents();
  griddep_wait();
  const size_t total = static_cast<size_t>(T) * nv;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = idx / nv, i = idx - static_cast<size_t>(t) * nv;
    float g[8], u[8], o[8];
    unpack8<BF16>(x[static_cast<size_t>(t) * (ldx / 8) + i], g);
    unpack8<BF16>(x[static_cast<size_t>(t) * (ldx / 8) + nv + i], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    out[idx] = pack8<BF16>(o);
  }
}

// SwiGLU gate fused with the block quantisation of its result: out8[t, i] = e4m3(silu(x[t, i]) * x[t, inter + i] / s) with
// one fp32 scale s = amax / 448 per 128 channels (the activation format of the block-scaled fp8 grouped GEMM), so the
// down-projection of an fp8 expert reads a quarter of the bytes a bf16 intermediate would cost. One half-warp owns a
// 128-channel block (a lane holds 8 channels), as in the dispatch kernel of ep_a2a.cu.
template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_fp8_kernel(const uint4* __restrict__ x, uint2* __restrict__ out8,
                                                           float* __restrict__ out_scale, int T, int inter, int ldx) {
  griddep_launch_dependents();
  griddep_wait();
  const int nblk = inter / 128;
  const int lane = threadIdx.x & 31, hl = lane & 15;
  const long long half_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const long long n_half = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  const long long total = static_cast<long long>(T) * nblk;
  // every lane runs the same number of iterations (the shuffles below need the whole warp): round the bound up to
  // whole warps of work and predicate the memory accesses instead
  const long long rounds = (total + n_half - 1) / n_half;
  for (long long r = 0; r < rounds; ++r) {
    const long long w = half_id + r * n_half;
    const bool in = w < total;
    const int t = in ? static_cast<int>(w / nblk) : 0, blk = in ? static_cast<int>(w - static_cast<long long>(t) * nblk) : 0;
    float g[8], u[8], o[8];
    const size_t base = static_cast<size_t>(t) * (ldx / 8) + static_cast<size_t>(blk) * 16 + hl;
    unpack8<BF16>(in ? x[base] : make_uint4(0, 0, 0, 0), g);
    unpack8<BF16>(in ? x[base + inter / 8] : make_uint4(0, 0, 0, 0), u);
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
      amax = fmaxf(amax, fabsf(o[e]));
    }
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    const float scale = amax / 448.f;
    const float den = scale > 0.f ? scale : 1.f;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      lo |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fdiv_rn(o[q], den), __NV_SATFINITE, __NV_E4M3)) << (8 * q);
      hi |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fdiv_rn(o[4 + q], den), __NV_SATFINITE, __NV_E4M3)) << (8 * q);
    }
    if (in) {
      out8[(static_cast<size_t>(t) * inter + static_cast<size_t>(blk) * 128) / 8 + hl] = make_uint2(lo, hi);
      if (hl == 0) out_scale[static_cast<size_t>(t) * nblk + blk] = scale;
    }
  }
}

// Router: one warp per token. logits [T, E] (fp32 or 16-bit), E <= 512. Writes top-k ids (int32) and
// softmax probabilities (fp32, optionally renormalised over the k winners).
template <typename LoadF>
__device__ __forceinline__ void topk_softmax_warp(LoadF load, int E, int k, int* ids, float* weights, bool renorm) {
  const int lane = threadIdx.x & 31;
  float v[16];
  float mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const int e = lane + 32 * u;
    v[u] = e < E ? load(e) : -INFINITY;
    mx = fmaxf(mx, v[u]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    v[u] = lane + 32 * u < E ? __expf(v[u] - mx) : 0.f;
    sum += v[u];
  }
  sum = warp_sum(sum);
  float picked = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int u = 0; u < 16; ++u)
      if (v[u] > best) { best = v[u]; best_e = lane + 32 * u; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (lane == 0) { ids[j] = best_e; weights[j] = best / sum; }
    picked += best / sum;
#pragma unroll
    for (int u = 0; u < 16; ++u)
      if (lane + 32 * u == best_e) v[u] = -1.f;
  }
  if (renorm) {
    __syncwarp();
    if (lane < k) weights[lane] /= picked;
  }
}
__global__ void topk_softmax_kernel(const void* logits, int dtype, int T, int E, int k, int* ids, float* weights,
                                    int renorm) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  if (dtype == kF32) {
    const float* p = static_cast<const float*>(logits) + static_cast<size_t>(t) * E;
    topk_softmax_warp([&](int e) { return p[e]; }, E, k, ids + static_cast<size_t>(t) * k, weights + static_cast<size_t>(t) * k, renorm != 0);
  } else if (dtype == kBF16) {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(logits) + static_cast<size_t>(t) * E;
    topk_softmax_warp([&](int e) { return __bfloat162float(p[e]); }, E, k, ids + static_cast<size_t>(t) * k, weights + static_cast<size_t>(t) * k, renorm != 0);
  } else {
    const __half* p = static_cast<const __half*>(logits) + static_cast<size_t>(t) * E;
    topk_softmax_warp([&](int e) { return __half2float(p[e]); }, E, k, ids + static_cast<size_t>(t) * k, weights + static_cast<size_t>(t) * k, renorm != 0);
  }
}

}  // namespace b200

using namespace b200;

// ids int64 [T]; table [V, H]; out [T, H]. Ids outside [0, V) read as zero rows. Optionally also emits, for the
// RMSNorm that follows, the row's sum of squares (sumsq_out fp32 [T], stored) and the row times the norm's gain
// (scaled_out [T, H] with gamma [H]), so that the consumer GEMM can apply 1 / rms in its epilogue.
// (torch's F.embedding in python/triton_dist/models/qwen.py:213.)
namespace b200 {
template <bool BF16>
__global__ void __launch_bounds__(256) embedding_kernel(const long long* __restrict__ ids, const uint4* __restrict__ table,
                                                        uint4* __restrict__ out, int T, long long V, int row_vec,
                                                        const uint4* __restrict__ gamma, uint4* __restrict__ scaled_out,
                                                        float* __restrict__ sumsq_out) {
  __shared__ float red[8];
  griddep_launch_dependents();
  griddep_wait();
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = ids[t];
    const bool ok = id >= 0 && id < V;
    float ss = 0.f;
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) {
      const uint4 v = ok ? ld_v4_nc(table + id * row_vec + i) : make_uint4(0, 0, 0, 0);
      out[static_cast<size_t>(t) * row_vec + i] = v;
      if (sumsq_out != nullptr || scaled_out != nullptr) {
        float f[8];
        unpack8<BF16>(v, f);
#pragma unroll
        for (int q = 0; q < 8; ++q) ss += f[q] * f[q];
        if (scaled_out != nullptr) {
          float g[8];
          unpack8<BF16>(gamma[i], g);
#pragma unroll
          for (int q = 0; q < 8; ++q) f[q] *= g[q];
          scaled_out[static_cast<size_t>(t) * row_vec + i] = pack8<BF16>(f);
        }
      }
    }
    if (sumsq_out != nullptr) {
      ss = warp_sum(ss);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int w = 0; w < 8; ++w) tot += red[w];
        sumsq_out[t] = tot;
      }
    }
  }
}
}  // namespace b200
B200_API int b200_embedding(const long long* ids, const void* table, void* out, int T, long long V, int H, int dtype,
                            const void* gamma, void* scaled_out, float* sumsq_out, void* stream) {
  B200_REQUIRE(dtype == b200::kBF16 || dtype == b200::kF16, "embedding handles bf16 / f16 tables");
  B200_REQUIRE(H > 0 && H % 8 == 0, "embedding width (%d) must be a multiple of 8", H);
  B200_REQUIRE(scaled_out == nullptr || gamma != nullptr, "scaled_out needs gamma");
  if (T <= 0) return b200::kOk;
  const int grid = T < 4 * b200::sm_count() ? T : 4 * b200::sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == b200::kBF16)
    B200_CHECK_CUDA(b200::launch_pdl(b200::embedding_kernel<true>, dim3(grid), dim3(256), 0, s, ids, static_cast<const uint4*>(table),
                                     static_cast<uint4*>(out), T, V, H / 8, static_cast<const uint4*>(gamma),
                                     static_cast<uint4*>(scaled_out), sumsq_out));
  else
    B200_CHECK_CUDA(b200::launch_pdl(b200::embedding_kernel<false>, dim3(grid), dim3(256), 0, s, ids, static_cast<const uint4*>(table),
                                     static_cast<uint4*>(out), T, V, H / 8, static_cast<const uint4*>(gamma),
                                     static_cast<uint4*>(scaled_out), sumsq_out));
  return b200::kOk;
}

B200_API int b200_rmsnorm(const void* x, const void* residual_in, void* residual_out, const void* gamma, void* y,
                          int rows, int hidden, float eps, int dtype, void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "rmsnorm supports bf16/f16");
  B200_REQUIRE(hidden % 8 == 0 && hidden <= 8 * 4 * 512, "hidden (%d) must be a multiple of 8 and <= 16384", hidden);
  if (rows == 0) return kOk;
  int threads = ((hidden / 8 + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  if (threads > 512) threads = 512;
  const int grid = rows < 4 * sm_count() ? rows : 4 * sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    B200_CHECK_CUDA(launch_pdl(rmsnorm_kernel<true>, grid, threads, 0, s, static_cast<const uint4*>(x),
                               static_cast<const uint4*>(residual_in), static_cast<uint4*>(residual_out),
                               static_cast<const uint4*>(gamma), static_cast<uint4*>(y), rows, hidden, eps));
  else
    B200_CHECK_CUDA(launch_pdl(rmsnorm_kernel<false>, grid, threads, 0, s, static_cast<const uint4*>(x),
                               static_cast<const uint4*>(residual_in), static_cast<uint4*>(residual_out),
                               static_cast<const uint4*>(gamma), static_cast<uint4*>(y), rows, hidden, eps));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

B200_API int b200_qk_norm_rope(const void* qkv, const int* positions, const int64_t* slots, const void* q_gamma,
                               const void* k_gamma, const float* cos_sin, void* q_out, void* k_cache, void* v_cache,
                               int T, int Hq, int Hkv, int head_dim, float eps, int dtype, void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "qk_norm_rope supports bf16/f16");
  B200_REQUIRE(head_dim == 128, "qk_norm_rope is specialised for head_dim 128, got %d", head_dim);
  if (T == 0) return kOk;
  const long long warps = static_cast<long long>(T) * (Hq + 2 * Hkv);
  const int grid = static_cast<int>((warps + 7) / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    B200_CHECK_CUDA(launch_pdl(qk_norm_rope_kernel<true>, grid, 256, 0, s, static_cast<const uint2*>(qkv), positions, slots,
                               static_cast<const uint2*>(q_gamma), static_cast<const uint2*>(k_gamma), cos_sin,
                               static_cast<uint2*>(q_out), static_cast<uint2*>(k_cache), static_cast<uint2*>(v_cache), T, Hq,
                               Hkv, eps));
  else
    B200_CHECK_CUDA(launch_pdl(qk_norm_rope_kernel<false>, grid, 256, 0, s, static_cast<const uint2*>(qkv), positions, slots,
                               static_cast<const uint2*>(q_gamma), static_cast<const uint2*>(k_gamma), cos_sin,
                               static_cast<uint2*>(q_out), static_cast<uint2*>(k_cache), static_cast<uint2*>(v_cache), T, Hq,
                               Hkv, eps));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

B200_API int b200_silu_mul(const void* x, void* out, int T, int inter, int ldx, int dtype, void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "silu_mul supports bf16/f16");
  B200_REQUIRE(inter % 8 == 0 && ldx % 8 == 0, "inter (%d) and ldx (%d) must be multiples of 8", inter, ldx);
  if (T == 0) return kOk;
  const long long total = static_cast<long long>(T) * (inter / 8);
  long long blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < 8LL * sm_count() ? blocks : 8LL * sm_count());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    B200_CHECK_CUDA(launch_pdl(silu_mul_kernel<true>, grid, 256, 0, s, static_cast<const uint4*>(x), static_cast<uint4*>(out), T, inter, ldx));
  else
    B200_CHECK_CUDA(launch_pdl(silu_mul_kernel<false>, grid, 256, 0, s, static_cast<const uint4*>(x), static_cast<uint4*>(out), T, inter, ldx));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

// x [T, 2 * inter] (row pitch ldx elements, gate | up); out8 e4m3 [T, inter]; out_scale fp32 [T, inter / 128].
B200_API int b200_silu_mul_fp8(const void* x, void* out8, float* out_scale, int T, int inter, int ldx, int dtype, void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "silu_mul_fp8 reads bf16 / f16");
  B200_REQUIRE(inter % 128 == 0 && ldx % 8 == 0, "the intermediate size (%d) must be a multiple of 128", inter);
  if (T == 0) return kOk;
  const long long halves = static_cast<long long>(T) * (inter / 128);
  const long long blocks = (halves * 16 + 255) / 256;
  const int grid = static_cast<int>(blocks < 8LL * sm_count() ? blocks : 8LL * sm_count());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    B200_CHECK_CUDA(launch_pdl(silu_mul_fp8_kernel<true>, grid, 256, 0, s, static_cast<const uint4*>(x), static_cast<uint2*>(out8), out_scale, T, inter, ldx));
  else
    B200_CHECK_CUDA(launch_pdl(silu_mul_fp8_kernel<false>, grid, 256, 0, s, static_cast<const uint4*>(x), static_cast<uint2*>(out8), out_scale, T, inter, ldx));
  return kOk;
}

B200_API int b200_topk_softmax(const void* logits, int dtype, int T, int E, int k, int* ids, float* weights, int renorm,
                               void* stream) {
  B200_REQUIRE(E >= 1 && E <= 512, "number of experts (%d) must be in [1, 512]", E);
  B200_REQUIRE(k >= 1 && k <= E && k <= 32, "top-k (%d) must be in [1, min(E, 32)]", k);
  B200_REQUIRE(dtype == kF32 || dtype == kBF16 || dtype == kF16, "router logits must be f32/bf16/f16");
  if (T == 0) return kOk;
  topk_softmax_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, dtype, T, E, k, ids, weights,
                                                                                  renorm);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
