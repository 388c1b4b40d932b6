// AllReduce over the symmetric heap, optionally fused with residual-add + RMSNorm, plus the on-stream
// cross-rank barrier.
//
// Methods (python/triton_dist/kernels/allreduce.py:28-61, kernels/nvidia/allreduce.py:223-692):
//   ONE_SHOT            every rank pushes its chunk into slot[rank] of every peer, then sums the slots
//   TWO_SHOT            rank r pulls slice r from every peer, sums it, pushes the result to every peer
//   ONE_SHOT_MULTIMEM   multimem.ld_reduce over the whole buffer (the switch does the sum)
//   TWO_SHOT_MULTIMEM   multimem.ld_reduce of slice r, multimem.st of the result to all ranks
//
// Structure shared by all methods: CTA b of every rank works on the same part of the data, so it only
// synchronises with CTA b of the peers (flags[phase][b][rank], monotone epochs) and no grid-wide
// barrier is needed. The workspace is double-buffered by epoch parity, which is what makes it safe for
// a fast rank to start call n+1 while a slow one still reads the buffers of call n (a rank cannot
// finish call n+1 before every peer has entered it). The epoch lives in device memory so a captured
// CUDA graph replays correctly.
//
// Fused form: the reduced vector is a matrix [rows, hidden]; CTAs own whole rows, add the residual,
// emit the new residual and the RMS-normalised row (row ownership follows the two-shot slices, so the
// owner normalises once and broadcasts both results).
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

namespace b200 {

constexpr int kArMaxCtas = 128;
constexpr int kArThreads = 512;

enum ArMethod : int { kOneShot = 0, kTwoShot = 1, kOneShotMc = 2, kTwoShotMc = 3 };

struct ArParams {
  const void* in;
  void* out;
  void* ws[2];        // symmetric; ONE_SHOT: [world][n]; others: [n] (staging, reduced in place for two-shot)
  uint32_t* flags;    // symmetric u32[2][kArMaxCtas][kMaxRanks]
  uint32_t* sync;     // local u32[4]: [0] epoch, [1] done counter
  uint64_t n;         // elements, multiple of (16 / elem size) * world for the two-shot / multimem methods
  int method;
  int dtype;
  // fused residual + RMSNorm (hidden > 0 enables it)
  int hidden;
  const void* residual_in;  // [rows, hidden] or null
  void* residual_out;       // [rows, hidden] (may alias residual_in) or null
  const void* gamma;        // [hidden]
  void* normed_out;         // [rows, hidden]
  float eps;
};

template <int DT> struct Vec;  // 16-byte vector of DT viewed as floats
template <> struct Vec<kBF16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
  }
  static __device__ __forceinline__ uint4 mc_reduce(const void* p) { return multimem_ld_reduce_bf16x8(p); }
};
template <> struct Vec<kF16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    float2 a = unpack_f16x2(v.x), b = unpack_f16x2(v.y), c = unpack_f16x2(v.z), d = unpack_f16x2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
  }
  static __device__ __forceinline__ uint4 mc_reduce(const void* p) { return multimem_ld_reduce_f16x8(p); }
};
template <> struct Vec<kF32> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ uint4 mc_reduce(const void* p) {
    float4 r = multimem_ld_reduce_f32x4(p);
    return make_uint4(__float_as_uint(r.x), __float_as_uint(r.y), __float_as_uint(r.z), __float_as_uint(r.w));
  }
};

// CTA-level cross-rank barrier: CTA b of this rank meets CTA b of every peer.
__device__ __forceinline__ bool cta_peer_barrier(const SymmCtx& c, uint32_t* flags, int phase, uint32_t epoch) {
  uint32_t* mine = flags + (static_cast<size_t>(phase) * kArMaxCtas + blockIdx.x) * kMaxRanks;
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < c.world) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(c, mine + c.rank, threadIdx.x), epoch);
    ok = wait_flag<WaitCmp::GE, true>(c, mine + threadIdx.x, epoch, threadIdx.x, __LINE__);
  }
  return __syncthreads_and(ok);
}

// Block-wide sum of one float per thread (kArThreads threads).
__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) smem[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? smem[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) smem[0] = t;
  }
  __syncthreads();
  return smem[0];
}

// Residual add + RMSNorm of one reduced row held as `nv` vectors spread over the CTA.
// Writes the new residual and the normalised row through `store(vec_index, residual_vec, normed_vec)`.
template <int DT, typename LoadSum, typename Store>
__device__ __forceinline__ void finish_row(const ArParams& p, uint64_t row, LoadSum load_sum, Store store, float* red) {
  using V = Vec<DT>;
  const int nv = p.hidden / V::kElems;
  // hidden <= 2 * kArThreads * kElems is enforced on the host: at most two vectors per thread
  float x[2][V::kElems];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = threadIdx.x + u * kArThreads;
    if (i < nv) {
      load_sum(i, x[u]);
      if (p.residual_in) {
        float r[V::kElems];
        V::unpack(ld_v4_nc(static_cast<const uint4*>(p.residual_in) + row * nv + i), r);
#pragma unroll
        for (int e = 0; e < V::kElems; ++e) x[u][e] += r[e];
      }
      // the residual stream is kept in the storage dtype, so normalise what is actually stored
      float q[V::kElems];
      V::unpack(V::pack(x[u]), q);
#pragma unroll
      for (int e = 0; e < V::kElems; ++e) { x[u][e] = q[e]; ss += q[e] * q[e]; }
    }
  }
  const float total = block_sum(ss, red);
  const float inv = rsqrtf(total / static_cast<float>(p.hidden) + p.eps);
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = threadIdx.x + u * kArThreads;
    if (i < nv) {
      float g[V::kElems], y[V::kElems];
      V::unpack(ld_v4_nc(static_cast<const uint4*>(p.gamma) + i), g);
#pragma unroll
      for (int e = 0; e < V::kElems; ++e) y[e] = x[u][e] * inv * g[e];
      store(i, V::pack(x[u]), V::pack(y));
    }
  }
}

// acc = sum over s < world of the vector at addr(s), in rank order. All loads are issued before the first add, so the
// sum costs one memory latency instead of `world` of them (these vectors sit on the critical path of a decode step).
template <int DT, typename Addr>
__device__ __forceinline__ void sum_over_ranks(int world, Addr addr, float* acc) {
  using V = Vec<DT>;
  uint4 v[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    if (s < world) v[s] = ld_v4_relaxed_sys(addr(s));
#pragma unroll
  for (int e = 0; e < V::kElems; ++e) acc[e] = 0.f;
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s)
    if (s < world) {
      float f[V::kElems];
      V::unpack(v[s], f);
#pragma unroll
      for (int e = 0; e < V::kElems; ++e) acc[e] += f[e];
    }
}

// Work maps. A CTA must consume only data that CTA b of the peers staged, because it synchronises with
// nobody else. "global": unit i belongs to CTA (i / T) % G. "slice": the data is cut into `world` equal
// slices and unit s * slice + i belongs to the CTA that owns i in the global map of [0, slice).
template <typename F>
__device__ __forceinline__ void for_units_global(uint64_t n, F f) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) f(i);
}

// Launched with kArThreads threads. The register cap (instead of a launch bound, which would let the compiler take
// 128) keeps a CTA of this kernel small enough to become resident next to a CTA of the preceding decode GEMM when
// the two are chained by programmatic dependent launch.
template <int DT>
__global__ void __maxnreg__(80) allreduce_kernel(const ArParams p, const SymmCtx ctx) {
  using V = Vec<DT>;
  __shared__ float red[32];
  griddep_launch_dependents();
  griddep_wait();
  const uint32_t epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  const int world = ctx.world, me = ctx.rank;
  const uint64_t nvec = p.n / V::kElems;
  uint4* ws = static_cast<uint4*>(p.ws[par]);
  const uint4* in = static_cast<const uint4*>(p.in);
  uint4* out = static_cast<uint4*>(p.out);
  const bool fused = p.hidden > 0;
  const uint64_t row_vecs = fused ? p.hidden / V::kElems : 1;
  const uint64_t rows = fused ? p.n / p.hidden : 0;
  const bool mc = p.method == kOneShotMc || p.method == kTwoShotMc;
  bool ok = true;

  auto peer_of = [&](int k) { int q = me + k; return q >= world ? q - world : q; };
  auto write_row_outputs = [&](uint64_t row, int i, uint4 res, uint4 nrm) {
    if (p.residual_out) static_cast<uint4*>(p.residual_out)[row * row_vecs + i] = res;
    static_cast<uint4*>(p.normed_out)[row * row_vecs + i] = nrm;
  };

  if (p.method == kOneShot) {
    // ---- push my data into slot[me] of every rank, meet, sum the slots -------------------------
    if (!fused) {
      for_units_global(nvec, [&](uint64_t i) {
        const uint4 v = in[i];
        for (int k = 0; k < world; ++k) st_v4(symm_at(ctx, ws + me * nvec + i, peer_of(k)), v);
      });
    } else {
      for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x)
        for (uint64_t i = threadIdx.x; i < row_vecs; i += blockDim.x) {
          const uint4 v = in[r * row_vecs + i];
          for (int k = 0; k < world; ++k) st_v4(symm_at(ctx, ws + me * nvec + r * row_vecs + i, peer_of(k)), v);
        }
    }
    ok = cta_peer_barrier(ctx, p.flags, 0, epoch);
    if (ok && !fused) {
      for_units_global(nvec, [&](uint64_t i) {
        float acc[V::kElems];
        sum_over_ranks<DT>(world, [&](int s) { return ws + s * nvec + i; }, acc);
        out[i] = V::pack(acc);
      });
    } else if (ok) {
      for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        auto load_sum = [&](int i, float* acc) {
          sum_over_ranks<DT>(world, [&](int s) { return ws + s * nvec + r * row_vecs + i; }, acc);
        };
        finish_row<DT>(p, r, load_sum, [&](int i, uint4 res, uint4 nrm) { write_row_outputs(r, i, res, nrm); }, red);
      }
    }
  } else if (p.method == kOneShotMc) {
    // ---- stage, meet, let the switch sum every vector for every rank ---------------------------
    if (!fused) {
      for_units_global(nvec, [&](uint64_t i) { ws[i] = in[i]; });
    } else {
      for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x)
        for (uint64_t i = threadIdx.x; i < row_vecs; i += blockDim.x) ws[r * row_vecs + i] = in[r * row_vecs + i];
    }
    ok = cta_peer_barrier(ctx, p.flags, 0, epoch);
    if (ok && !fused) {
      for_units_global(nvec, [&](uint64_t i) { out[i] = V::mc_reduce(mc_ptr(ctx, ws + i)); });
    } else if (ok) {
      for (uint64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        auto load_sum = [&](int i, float* acc) { V::unpack(V::mc_reduce(mc_ptr(ctx, ws + r * row_vecs + i)), acc); };
        finish_row<DT>(p, r, load_sum, [&](int i, uint4 res, uint4 nrm) { write_row_outputs(r, i, res, nrm); }, red);
      }
    }
  } else {
    // ---- two-shot: rank r reduces slice r and broadcasts the result ----------------------------
    // workspace: [0, nvec) staging; [nvec, 2 nvec) results (new residual when fused); [2 nvec, 3 nvec) normed rows
    const uint64_t slice = nvec / world;           // vectors per rank
    const uint64_t rpr = fused ? rows / world : 0;  // rows per rank
    if (!fused) {
      for (int s = 0; s < world; ++s)
        for_units_global(slice, [&](uint64_t i) { ws[s * slice + i] = in[s * slice + i]; });
    } else {
      for (int s = 0; s < world; ++s)
        for (uint64_t r = blockIdx.x; r < rpr; r += gridDim.x)
          for (uint64_t i = threadIdx.x; i < row_vecs; i += blockDim.x) {
            const uint64_t idx = (s * rpr + r) * row_vecs + i;
            ws[idx] = in[idx];
          }
    }
    ok = cta_peer_barrier(ctx, p.flags, 0, epoch);
    auto pull_sum = [&](const uint4* addr, float* acc) {
      sum_over_ranks<DT>(world, [&](int k) { return symm_at(ctx, addr, peer_of(k)); }, acc);
    };
    auto broadcast = [&](uint4* addr, uint4 v) {
      if (mc) {
        multimem_st_v4(mc_ptr(ctx, addr), v);
      } else {
        for (int k = 0; k < world; ++k) st_v4(symm_at(ctx, addr, peer_of(k)), v);
      }
    };
    if (ok && !fused) {
      for_units_global(slice, [&](uint64_t i) {
        uint4* src = ws + me * slice + i;
        uint4 r;
        if (mc) {
          r = V::mc_reduce(mc_ptr(ctx, src));
        } else {
          float acc[V::kElems];
          pull_sum(src, acc);
          r = V::pack(acc);
        }
        broadcast(ws + nvec + me * slice + i, r);
      });
    } else if (ok) {
      for (uint64_t r = blockIdx.x; r < rpr; r += gridDim.x) {
        const uint64_t row = me * rpr + r;
        auto load_sum = [&](int i, float* acc) {
          uint4* src = ws + row * row_vecs + i;
          if (mc) V::unpack(V::mc_reduce(mc_ptr(ctx, src)), acc);
          else pull_sum(src, acc);
        };
        auto store = [&](int i, uint4 res, uint4 nrm) {
          broadcast(ws + nvec + row * row_vecs + i, res);
          broadcast(ws + 2 * nvec + row * row_vecs + i, nrm);
        };
        finish_row<DT>(p, row, load_sum, store, red);
      }
    }
    if (ok) ok = cta_peer_barrier(ctx, p.flags, 1, epoch);
    if (ok && !fused) {
      for (int s = 0; s < world; ++s)
        for_units_global(slice, [&](uint64_t i) { out[s * slice + i] = ld_v4_relaxed_sys(ws + nvec + s * slice + i); });
    } else if (ok) {
      for (int s = 0; s < world; ++s)
        for (uint64_t r = blockIdx.x; r < rpr; r += gridDim.x)
          for (uint64_t i = threadIdx.x; i < row_vecs; i += blockDim.x) {
            const uint64_t idx = (s * rpr + r) * row_vecs + i;
            if (p.residual_out) static_cast<uint4*>(p.residual_out)[idx] = ld_v4_relaxed_sys(ws + nvec + idx);
            static_cast<uint4*>(p.normed_out)[idx] = ld_v4_relaxed_sys(ws + 2 * nvec + idx);
          }
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

__global__ void barrier_all_kernel(const SymmCtx ctx, uint32_t* flags, uint32_t* sync) {
  const uint32_t epoch = epoch_begin(sync);
  barrier_all_block(ctx, flags, epoch);
  if (threadIdx.x == 0) epoch_end(sync, sync + 1, epoch, 1);
}

}  // namespace b200

using namespace b200;

B200_API int b200_barrier_all(const void* symm_ctx, uint32_t* flags, uint32_t* sync, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  barrier_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx, flags, sync);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
B200_API int b200_allreduce_max_ctas() { return kArMaxCtas; }

// Workspace elements needed per parity buffer, as a multiple of n.
B200_API int b200_allreduce_ws_factor(int method, int world, int fused) {
  switch (method) {
    case kOneShot: return world;
    case kOneShotMc: return 1;
    default: return fused ? 3 : 2;
  }
}

// in/out: [n] elements of `dtype` (16-byte aligned). ws0/ws1: symmetric parity buffers of
// ws_factor * n elements. flags: symmetric u32[2 * kArMaxCtas * kMaxRanks]; sync: local u32[4]; both
// zero-initialised once. hidden > 0 selects the fused residual + RMSNorm form over [n / hidden, hidden].
B200_API int b200_allreduce(const void* symm_ctx, const void* in, void* out, uint64_t n, int dtype, int method,
                            void* ws0, void* ws1, uint32_t* flags, uint32_t* sync, int hidden,
                            const void* residual_in, void* residual_out, const void* gamma, void* normed_out,
                            float eps, int num_ctas, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(dtype == kBF16 || dtype == kF16 || dtype == kF32, "allreduce supports bf16/f16/f32");
  const uint64_t ve = 16 / dtype_size(dtype);
  B200_REQUIRE(method >= kOneShot && method <= kTwoShotMc, "unknown allreduce method %d", method);
  B200_REQUIRE(n % ve == 0, "element count %llu is not a multiple of %llu", (unsigned long long)n, (unsigned long long)ve);
  if (method == kTwoShot || method == kTwoShotMc)
    B200_REQUIRE((n / ve) % ctx.world == 0, "two-shot methods need n / %llu divisible by the world size",
                 (unsigned long long)ve);
  if (method == kOneShotMc || method == kTwoShotMc)
    B200_REQUIRE(ctx.mc_base != 0, "multimem methods need an NVLS multicast mapping");
  B200_REQUIRE(((reinterpret_cast<uint64_t>(in) | reinterpret_cast<uint64_t>(out)) & 15u) == 0 || hidden > 0,
               "allreduce buffers must be 16-byte aligned");
  if (hidden > 0) {
    B200_REQUIRE(hidden % ve == 0 && n % hidden == 0, "hidden (%d) must divide n and be a multiple of %llu", hidden,
                 (unsigned long long)ve);
    B200_REQUIRE(static_cast<uint64_t>(hidden) / ve <= 2 * kArThreads, "hidden (%d) too large for the fused kernel", hidden);
    B200_REQUIRE(gamma != nullptr && normed_out != nullptr, "fused allreduce needs gamma and normed_out");
    if (method == kTwoShot || method == kTwoShotMc)
      B200_REQUIRE((n / hidden) % ctx.world == 0, "fused two-shot needs rows divisible by the world size");
  }
  ArParams p;
  memset(&p, 0, sizeof(p));
  p.in = in; p.out = out; p.ws[0] = ws0; p.ws[1] = ws1; p.flags = flags; p.sync = sync; p.n = n;
  p.method = method; p.dtype = dtype; p.hidden = hidden; p.residual_in = residual_in; p.residual_out = residual_out;
  p.gamma = gamma; p.normed_out = normed_out; p.eps = eps;
  int grid = num_ctas > 0 ? num_ctas : 8;
  if (grid > kArMaxCtas) grid = kArMaxCtas;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case kBF16: B200_CHECK_CUDA(launch_pdl(allreduce_kernel<kBF16>, grid, kArThreads, 0, s, p, ctx)); break;
    case kF16: B200_CHECK_CUDA(launch_pdl(allreduce_kernel<kF16>, grid, kArThreads, 0, s, p, ctx)); break;
    default: B200_CHECK_CUDA(launch_pdl(allreduce_kernel<kF32>, grid, kArThreads, 0, s, p, ctx)); break;
  }
  return kOk;
}
