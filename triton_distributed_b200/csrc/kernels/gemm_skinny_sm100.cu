// Decode-time GEMM for few tokens (M <= 256): C[M,N] = X[M,K] * W[N,K]^T, optionally with the SwiGLU
// gate fused (W = [gate; up], C[M, N/2] = silu(X gate^T) * (X up^T)).
//
// With M this small the op is a stream of the weight matrix through the SM, so the kernel is built
// to keep HBM busy rather than the tensor cores:
//   * swap-AB: the 128 weight rows of a tile are the M side of tcgen05.mma (M128, K16) and the tokens,
//     padded to a multiple of 16, are the N side, so no tensor-core rows are wasted on padding and the
//     weights are read exactly once;
//   * stream-K: the (tile, k-block) work units are cut into one equal contiguous range per SM, so every
//     SM streams the same number of weight bytes for any shape (no wave quantisation); each CTA runs a
//     deep TMA ring (up to 12 stages, ~190 KB in flight per SM) and double-buffers its accumulator;
//   * a tile covered by several CTAs is summed in an fp32 scratch tile through red.global.add; the CTA
//     that takes the last ticket of a tile converts (and applies SwiGLU), writes C, and re-zeroes scratch and ticket, so the
//     scratch is clean for the next launch without a memset.
// The tokens are the TMEM columns, so an epilogue thread owns one output feature for all tokens and a
// warp writes 32 consecutive features of one token: coalesced without a shared-memory transpose.
//
// Fused epilogues (at most 16 tokens, i.e. one accumulator chunk per epilogue thread), applied by whichever CTA holds
// the finished tile:
//   row scale     out[m, :] *= rsqrt(sumsq[m] / dim + eps): the RMSNorm of the GEMM's input, whose gain the producer
//                 of the input already multiplied in, so no normalisation kernel runs between two GEMMs
//   qkv heads     a 128-feature tile is one attention head: per-head RMSNorm, neox RoPE, and the write of q to its
//                 buffer and of k / v into the paged KV cache (replaces a separate norm + rope + cache-write kernel)
//   residual      h = out + residual; writes h, h * gain_of_the_next_norm and adds sum(h^2) per token to a buffer
//
// Role in the reference: the cuBLAS F.linear calls of the AllReduce forward mode
// (python/triton_dist/layers/nvidia/tp_mlp.py:177-191, tp_attn.py:240-271) and the unfused
// act_fn(gate) * up (tp_mlp.py:159-160).
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/tcgen05.cuh"

#include <cstdlib>
#include <cstring>

namespace b200 {

constexpr int kSkBN = 128;  // weight rows per tile
constexpr int kSkBK = 64;
constexpr int kSkWBytes = kSkBN * kSkBK * 2;
constexpr int kSkMaxStages = 12;
constexpr int kSkSmemBudget = 216 * 1024;  // ring; the kernel's static shared memory (8.7 KB) comes on top

enum SkinnyEpilogueKind : int { kEpNone = 0, kEpQkvHeads = 1, kEpResidual = 2 };

struct SkinnyEpilogue {
  int kind;
  // row scale (any kind, nullable): per-token sum of squares of the un-normalised input
  const float* sumsq_in;
  float scale_dim, eps;
  // kEpQkvHeads: tile t is head t of [q heads | k heads | v heads]
  int Hq, Hkv;
  const int* positions;      // [M]
  const long long* slots;    // [M] cache slot of every token, null = identity
  const float* cos_sin;      // [max_pos, 128] = cos | sin
  const void* q_gamma;       // [128] or null (no per-head norm)
  const void* k_gamma;
  void* q_out;               // [M, Hq, 128]
  void* k_cache;             // [slots, Hkv, 128]
  void* v_cache;
  float head_eps;
  // kEpResidual
  const void* residual_in;   // [M, N] (row pitch ldc), may alias residual_out
  void* residual_out;        // [M, N] (row pitch ldc)
  const void* next_gamma;    // [N] gain of the norm that follows, or null
  void* scaled_out;          // [M, N] (row pitch ldc) = h * next_gamma (with next_gamma)
  float* sumsq_out;          // [M], accumulated with atomics (zero it before the first producer of a step)
};

struct SkinnyParams {
  int M, N, K;        // N = weight rows per projection (the output features)
  int MB;             // tokens padded to a multiple of 16
  int stages;
  int stage_bytes;
  int num_kb;         // k-blocks per tile
  int units_total;    // tiles * num_kb
  int units_per_cta;  // contiguous (tile, k-block) units owned by one CTA
  int up_row0;        // dual: first row of the `up` projection inside W
  int bf16;
  void* C;
  int ldc;
  float* scratch;     // [tiles][dual ? 2 : 1][MB][128] fp32, zero on entry and on exit
  uint32_t* tickets;  // [tiles], zero on entry and on exit
  SkinnyEpilogue ep;
  unsigned long long* trace;  // optional [gridDim.x][8] %globaltimer checkpoints of every CTA (tuning aid), else null
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// Stream-K: the (tile, k-block) units are numbered tile-major and cut into gridDim.x equal contiguous
// ranges, so every SM streams the same number of weight bytes whatever the shape. A CTA's range is a
// sequence of segments, each inside one tile; a tile covered by several CTAs is summed in scratch.
struct Segment {
  int tile, kb0, kb1;
};
__device__ __forceinline__ bool next_segment(const SkinnyParams& p, int& u, int u1, Segment& s) {
  if (u >= u1) return false;
  s.tile = u / p.num_kb;
  s.kb0 = u - s.tile * p.num_kb;
  s.kb1 = min(p.num_kb, s.kb0 + (u1 - u));
  u += s.kb1 - s.kb0;
  return true;
}

__device__ __forceinline__ float ld_elem(const void* p, size_t i, bool bf16) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : __half2float(static_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ float round_elem(float v, bool bf16) {
  return bf16 ? __bfloat162float(__float2bfloat16(v)) : __half2float(__float2half(v));
}
__device__ __forceinline__ void st_elem(void* p, size_t i, float v, bool bf16) {
  if (bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else static_cast<__half*>(p)[i] = __float2half(v);
}

// Finishes one 128-feature tile for up to 16 tokens. Executed by the 128 epilogue threads together (thread et owns
// feature et of the tile for every token); g / uu hold the complete sums. `xch` is [16][128] floats and `red` [4][16]
// floats of shared memory.
template <bool kDual>
__device__ __forceinline__ void finish_tile16(const SkinnyParams& p, int tile, int et, float (&g)[16], float (&uu)[16],
                                              float* xch, float* red) {
  const SkinnyEpilogue& ep = p.ep;
  const bool bf16 = p.bf16 != 0;
  const int n = tile * kSkBN + et;
  const int w = et >> 5, lane = et & 31;
  if (ep.sumsq_in != nullptr) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float sc = j < p.M ? rsqrtf(__ldcg(ep.sumsq_in + j) / ep.scale_dim + ep.eps) : 0.f;
      g[j] *= sc;
      if (kDual) uu[j] *= sc;
    }
  }
  if (ep.kind == kEpQkvHeads) {
    const int head = tile;
    const bool is_q = head < ep.Hq, is_k = !is_q && head < ep.Hq + ep.Hkv;
    const void* gamma = is_q ? ep.q_gamma : is_k ? ep.k_gamma : nullptr;
    // rotary factors are fetched first so that their two dependent loads overlap the per-head norm
    float cj[16], sj[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      cj[j] = 1.f, sj[j] = 0.f;
      if ((is_q || is_k) && j < p.M) {
        const float* cs = ep.cos_sin + static_cast<size_t>(__ldg(ep.positions + j)) * 128;
        cj[j] = __ldg(cs + (et & 63)), sj[j] = __ldg(cs + 64 + (et & 63));
      }
    }
    if (gamma != nullptr) {  // per-head RMSNorm over the 128 features of the tile
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float t = warp_sum(g[j] * g[j]);
        if (lane == 0) red[w * 16 + j] = t;
      }
      epi_bar();
      const float gm = ld_elem(gamma, et, bf16);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float tot = red[j] + red[16 + j] + red[32 + j] + red[48 + j];
        g[j] *= rsqrtf(tot / 128.f + ep.head_eps) * gm;
      }
    }
    if (is_q || is_k) {  // neox rotary embedding: feature i pairs with feature i +- 64
#pragma unroll
      for (int j = 0; j < 16; ++j) xch[j * kSkBN + et] = g[j];
      epi_bar();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float other = xch[j * kSkBN + (et ^ 64)];
        g[j] = et < 64 ? g[j] * cj[j] - other * sj[j] : g[j] * cj[j] + other * sj[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < p.M) {
        if (is_q) {
          st_elem(ep.q_out, (static_cast<size_t>(j) * ep.Hq + head) * 128 + et, g[j], bf16);
        } else {
          const size_t slot = ep.slots ? static_cast<size_t>(ep.slots[j]) : static_cast<size_t>(j);
          const int kvh = is_k ? head - ep.Hq : head - ep.Hq - ep.Hkv;
          st_elem(is_k ? ep.k_cache : ep.v_cache, (slot * ep.Hkv + kvh) * 128 + et, g[j], bf16);
        }
      }
    }
    epi_bar();  // red / xch are reused by the next tile
    return;
  }
  if (ep.kind == kEpResidual) {
    const float gm = (ep.next_gamma != nullptr && n < p.N) ? ld_elem(ep.next_gamma, n, bf16) : 0.f;
    // every residual element is loaded before the first store: residual_in may alias residual_out, so the compiler
    // keeps loads behind earlier stores, which would make this one memory round trip per token
    float res[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
      res[j] = (j < p.M && n < p.N) ? ld_elem(ep.residual_in, static_cast<size_t>(j) * p.ldc + n, bf16) : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float sq = 0.f;
      if (j < p.M && n < p.N) {
        const size_t o = static_cast<size_t>(j) * p.ldc + n;
        const float h = round_elem(g[j] + res[j], bf16);  // the stream is kept in storage type
        st_elem(ep.residual_out, o, h, bf16);
        if (ep.scaled_out != nullptr) st_elem(ep.scaled_out, o, h * gm, bf16);
        sq = h * h;
      }
      sq = warp_sum(sq);
      if (lane == 0 && j < p.M && ep.sumsq_out != nullptr) atomicAdd(ep.sumsq_out + j, sq);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (j < p.M && n < p.N) {
      const float v = kDual ? g[j] / (1.f + __expf(-g[j])) * uu[j] : g[j];
      st_elem(p.C, static_cast<size_t>(j) * p.ldc + n, v, bf16);
    }
  }
}

template <bool kDual>
__global__ void __launch_bounds__(256, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kSkMaxStages];
  __shared__ uint64_t empty_bar[kSkMaxStages];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_word;
  __shared__ uint32_t last_flag;
  __shared__ uint32_t armed_count;  // k-blocks whose stage barrier the weight producer has armed
  __shared__ float ep_xch[16 * kSkBN];  // fused epilogues: partner exchange of the rotary embedding
  __shared__ float ep_red[4 * 16];      //                  per-warp partial sums of the per-head norm
  volatile uint32_t* abort_flag = &abort_word;
  const bool fused_ep = p.ep.kind != kEpNone || p.ep.sumsq_in != nullptr;  // host guarantees MB == 16 then

  const int warp = threadIdx.x >> 5;
  constexpr int kW = kDual ? 2 : 1;
  const int acc_cols = kW * p.MB;  // TMEM columns of one accumulator set
  const uint32_t need = 2 * acc_cols;
  const uint32_t tmem_cols = need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
  const uint64_t timeout_ns = 4000000000ull;
  const int u_begin = blockIdx.x * p.units_per_cta;
  const int u_end = min(p.units_total, u_begin + p.units_per_cta);
  griddep_launch_dependents();  // the next kernel may set itself up while this one streams
  auto stamp = [&](int slot) {
    if (p.trace != nullptr) p.trace[blockIdx.x * 8 + slot] = globaltimer_ns();
  };
  if (threadIdx.x == 0) stamp(0);  // CTA start

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(full_bar + i, 1);
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar + i, 1);
      mbar_init(tempty_bar + i, 4);
    }
    abort_word = 0;
    armed_count = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 2) tmem_alloc(&tmem_slot, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0) stamp(1);  // barriers initialised, TMEM allocated

  if (warp == 0) {
    if (elect_one()) {
      // Weight producer. The weights do not depend on the previous kernel, so this thread never waits for it: it
      // arms each stage's barrier for the whole stage (weights + activations), requests the weight tiles and
      // publishes how many k-blocks are armed. The activation tiles are requested by the thread below.
      uint32_t stage = 0, phase = 0, armed = 0;
      int u = u_begin;
      Segment sg;
      bool ok = true;
      while (ok && next_segment(p, u, u_end, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, timeout_ns)) { ok = false; break; }
          uint8_t* s = smem + stage * p.stage_bytes;
          mbar_expect_tx(full_bar + stage, p.stage_bytes);
          tma_load_2d(s, &tmW, full_bar + stage, kb * kSkBK, sg.tile * kSkBN);
          if (kDual) tma_load_2d(s + kSkWBytes, &tmW, full_bar + stage, kb * kSkBK, p.up_row0 + sg.tile * kSkBN);
          ++armed;
          asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&armed_count)), "r"(armed) : "memory");
          if (++stage == static_cast<uint32_t>(p.stages)) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    if (elect_one()) {
      // Activation producer. The activations are the previous kernel's output: wait for it once, then request the
      // tile of every k-block as soon as the weight producer has armed its stage. Because the two producers are
      // separate threads, a CTA that starts late (the previous kernel is already complete) gets its activations at
      // once instead of after the whole first ring of weight requests, and a CTA that starts early keeps prefetching
      // weights for as long as the previous kernel runs.
      griddep_wait();
      stamp(2);  // the previous kernel has completed: activations may be loaded
      fence_proxy_async();
      uint32_t stage = 0, done = 0;
      int u = u_begin;
      Segment sg;
      bool ok = true;
      while (ok && next_segment(p, u, u_end, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1 && ok; ++kb) {
          uint64_t t0 = 0;
          uint32_t spins = 0;
          while (true) {
            uint32_t seen;
            asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(seen) : "r"(smem_u32(&armed_count)) : "memory");
            if (seen > done) break;
            if ((++spins & 255u) == 0u) {
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              if (*abort_flag != 0u || now - t0 > timeout_ns) { *abort_flag = 1u; ok = false; break; }
            }
          }
          if (!ok) break;
          tma_load_2d(smem + stage * p.stage_bytes + kW * kSkWBytes, &tmX, full_bar + stage, kb * kSkBK, 0);
          ++done;
          if (++stage == static_cast<uint32_t>(p.stages)) stage = 0;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_f16(kSkBN, p.MB, p.bf16 != 0);
      uint32_t stage = 0, phase = 0, it = 0;
      int u = u_begin;
      Segment sg;
      bool ok = true;
      while (ok && next_segment(p, u, u_end, sg)) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar + acc, acc_phase ^ 1, abort_flag, timeout_ns)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * acc_cols;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(full_bar + stage, phase, abort_flag, timeout_ns)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t s = smem_u32(smem + stage * p.stage_bytes);
          const uint64_t dw = umma_desc_sw128_kmajor(s);
          const uint64_t dx = umma_desc_sw128_kmajor(s + kW * kSkWBytes);
#pragma unroll
          for (int k = 0; k < kSkBK / 16; ++k) {
            const uint32_t accum = (kb > sg.kb0 || k > 0) ? 1u : 0u;
            umma_f16(d_tmem, dw + 2 * k, dx + 2 * k, idesc, accum);
            if (kDual) umma_f16(d_tmem + p.MB, umma_desc_sw128_kmajor(s + kSkWBytes) + 2 * k, dx + 2 * k, idesc, accum);
          }
          umma_commit(empty_bar + stage);
          if (++stage == static_cast<uint32_t>(p.stages)) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(tfull_bar + acc);
        ++it;
      }
      stamp(3);  // last MMA issued
    }
    __syncwarp();
  } else if (warp >= 4) {
    const int w = warp - 4;
    const int et = threadIdx.x - 128;  // 0..127 == feature index inside the tile
    const int lane = threadIdx.x & 31;
    uint32_t it = 0;
    int u = u_begin;
    Segment sg;
    griddep_wait();  // the output, the scratch tile and the tickets may still be in use by the previous kernel
    while (next_segment(p, u, u_end, sg)) {
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      ++it;
      const int n = sg.tile * kSkBN + et;
      // how many CTAs contribute to this tile
      const int first_cta = (sg.tile * p.num_kb) / p.units_per_cta;
      const int last_cta = ((sg.tile + 1) * p.num_kb - 1) / p.units_per_cta;
      const int contributors = last_cta - first_cta + 1;
      if (!mbar_wait(tfull_bar + acc, acc_phase, abort_flag, timeout_ns)) break;
      tc_fence_after_sync();
      if (et == 0 && u >= u_end) stamp(4);  // accumulator of this CTA's last segment is complete
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(w * 32) << 16) + acc * acc_cols;
      float* scratch = p.scratch + static_cast<size_t>(sg.tile) * kW * p.MB * kSkBN;
      auto store_out = [&](int m, float g, float uu) {
        if (m < p.M && n < p.N) {
          const float v = kDual ? g / (1.f + __expf(-g)) * uu : g;
          if (p.bf16) static_cast<__nv_bfloat16*>(p.C)[static_cast<size_t>(m) * p.ldc + n] = __float2bfloat16(v);
          else static_cast<__half*>(p.C)[static_cast<size_t>(m) * p.ldc + n] = __float2half(v);
        }
      };
      for (int c0 = 0; c0 < p.MB; c0 += 16) {
        uint32_t g[16], uu[16];
        tmem_ld_32x16(taddr + c0, g);
        if (kDual) tmem_ld_32x16(taddr + p.MB + c0, uu);
        tmem_ld_wait();
        if (contributors == 1 && fused_ep) {
          float gf[16], uf[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            gf[j] = __uint_as_float(g[j]);
            uf[j] = kDual ? __uint_as_float(uu[j]) : 0.f;
          }
          finish_tile16<kDual>(p, sg.tile, et, gf, uf, ep_xch, ep_red);
        } else if (contributors == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) store_out(c0 + j, __uint_as_float(g[j]), kDual ? __uint_as_float(uu[j]) : 0.f);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < p.M) {
              atomicAdd(scratch + static_cast<size_t>(c0 + j) * kSkBN + et, __uint_as_float(g[j]));
              if (kDual) atomicAdd(scratch + static_cast<size_t>(p.MB + c0 + j) * kSkBN + et, __uint_as_float(uu[j]));
            }
          }
        }
      }
      // accumulator read: give it back to the MMA warp before the (slower) ticket protocol
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar + acc);
      if (contributors > 1) {
        // the last contributor of the tile finishes it and leaves scratch + ticket zeroed
        __threadfence();
        epi_bar();
        if (et == 0) {
          if (u >= u_end) stamp(5);  // partial sums added and fenced
          const uint32_t t = atomicAdd(p.tickets + sg.tile, 1u);
          last_flag = (t == static_cast<uint32_t>(contributors - 1)) ? 1u : 0u;
          if (u >= u_end) stamp(6);  // ticket drawn
        }
        epi_bar();
        if (last_flag && fused_ep) {
          __threadfence();
          float gf[16], uf[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {  // all loads first (one round trip), then the zeroing stores
            gf[j] = uf[j] = 0.f;
            if (j < p.M) {
              gf[j] = __ldcg(scratch + static_cast<size_t>(j) * kSkBN + et);
              if (kDual) uf[j] = __ldcg(scratch + static_cast<size_t>(p.MB + j) * kSkBN + et);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < p.M) {
              __stcg(scratch + static_cast<size_t>(j) * kSkBN + et, 0.f);
              if (kDual) __stcg(scratch + static_cast<size_t>(p.MB + j) * kSkBN + et, 0.f);
            }
          }
          finish_tile16<kDual>(p, sg.tile, et, gf, uf, ep_xch, ep_red);
          if (et == 0) p.tickets[sg.tile] = 0;
        } else if (last_flag) {
          __threadfence();
          // eight tokens at a time, all loads issued before the first use: one L2 round trip per batch instead of one
          // per token (this loop is the tail of the kernel; at 8 tokens it used to cost ~4 us, now ~1 us)
          for (int m0 = 0; m0 < p.M; m0 += 8) {
            float gv[8], uv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              gv[j] = uv[j] = 0.f;
              if (m0 + j < p.M) {
                gv[j] = __ldcg(scratch + static_cast<size_t>(m0 + j) * kSkBN + et);
                if (kDual) uv[j] = __ldcg(scratch + static_cast<size_t>(p.MB + m0 + j) * kSkBN + et);
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (m0 + j < p.M) {
                __stcg(scratch + static_cast<size_t>(m0 + j) * kSkBN + et, 0.f);
                if (kDual) __stcg(scratch + static_cast<size_t>(p.MB + m0 + j) * kSkBN + et, 0.f);
                store_out(m0 + j, gv[j], uv[j]);
              }
            }
          }
          if (et == 0) p.tickets[sg.tile] = 0;
        }
        epi_bar();  // last_flag is reused by the next segment
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, tmem_cols);
  if (threadIdx.x == 0) stamp(7);  // CTA done
}

// Shared memory per CTA for the weight ring. At about half of an SM's shared memory the first CTAs of the next
// kernel of a programmatic-dependent-launch chain become resident (and prefetch their weights) while this kernel's
// last tiles are still streaming. B200DIST_SKINNY_SMEM_KB overrides it.
static int skinny_smem_budget() {
  static int budget = -1;
  if (budget < 0) {
    const char* e = getenv("B200DIST_SKINNY_SMEM_KB");
    int kb = e ? atoi(e) : 0;
    budget = (kb >= 16 && kb * 1024 <= kSkSmemBudget) ? kb * 1024 : kSkSmemBudget;
  }
  return budget;
}

template <bool kDual>
static int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, dim3 grid, int smem,
                         cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel<kDual>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSkSmemBudget + 1024));
    configured[dev & 63] = true;
  }
  B200_CHECK_CUDA(launch_pdl(gemm_skinny_kernel<kDual>, grid, dim3(256), static_cast<size_t>(smem), stream, tw, tx, p));
  return kOk;
}

}  // namespace b200

using namespace b200;

// Scratch floats / tickets needed for a call (independent of the split count).
B200_API long long b200_gemm_skinny_scratch_floats(int M, int N, int dual) {
  const int MB = (M + 15) / 16 * 16;
  const long long tiles = (N + kSkBN - 1) / kSkBN;
  return tiles * (dual ? 2 : 1) * MB * kSkBN;
}

// X [M, K] (row pitch ldx), W [Nw, K] (row pitch ldw), C [M, N] (row pitch ldc).
// dual == 0: N = Nw. dual == 1: W = [gate (N rows); up (N rows)], C = silu(X gate^T) * (X up^T).
// scratch / tickets: zero-initialised once by the caller; every call leaves them zeroed.
// splits <= 0: one CTA per SM (stream-K); splits > 0 forces tiles * splits CTAs.
static unsigned long long* g_skinny_trace = nullptr;

static int skinny_impl(const void* X, const void* W, void* C, int M, int N, int K, int ldx, int ldw, int ldc, int dual,
                       int dtype, float* scratch, uint32_t* tickets, int splits, const SkinnyEpilogue* ep, void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "gemm_skinny supports bf16/f16");
  B200_REQUIRE(M >= 1 && M <= 256, "gemm_skinny handles 1..256 tokens, got %d", M);
  B200_REQUIRE(K % 8 == 0, "K (%d) must be a multiple of 8", K);
  SkinnyParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.MB = (M + 15) / 16 * 16;
  B200_REQUIRE(!dual || p.MB <= 128, "fused SwiGLU handles at most 128 tokens");
  const int kw = dual ? 2 : 1;
  p.stage_bytes = kw * kSkWBytes + p.MB * 128;
  p.stages = skinny_smem_budget() / p.stage_bytes;
  if (p.stages > kSkMaxStages) p.stages = kSkMaxStages;
  if (p.stages < 2) p.stages = kSkSmemBudget / p.stage_bytes < 2 ? 0 : 2;
  B200_REQUIRE(p.stages >= 2, "tile does not fit in shared memory");
  p.up_row0 = N;
  p.bf16 = dtype == kBF16;
  p.C = C; p.ldc = ldc; p.scratch = scratch; p.tickets = tickets;
  p.trace = g_skinny_trace;
  if (ep != nullptr) {
    p.ep = *ep;
    const bool fused = ep->kind != kEpNone || ep->sumsq_in != nullptr;
    B200_REQUIRE(!fused || M <= 16, "the fused epilogues handle at most 16 tokens, got %d", M);
    if (ep->kind == kEpQkvHeads) {
      B200_REQUIRE(!dual && N == (ep->Hq + 2 * ep->Hkv) * kSkBN, "qkv epilogue: N (%d) must be (Hq + 2 Hkv) * 128", N);
      B200_REQUIRE(ep->positions && ep->cos_sin && ep->q_out && ep->k_cache && ep->v_cache, "qkv epilogue: missing buffers");
    } else if (ep->kind == kEpResidual) {
      B200_REQUIRE(!dual && ep->residual_in && ep->residual_out, "residual epilogue: missing buffers");
      B200_REQUIRE(ep->scaled_out == nullptr || ep->next_gamma != nullptr, "residual epilogue: scaled_out needs next_gamma");
    } else {
      B200_REQUIRE(ep->kind == kEpNone, "unknown epilogue kind %d", ep->kind);
      B200_REQUIRE(C != nullptr, "gemm_skinny needs an output");
    }
  }
  const int tiles = (N + kSkBN - 1) / kSkBN;
  p.num_kb = (K + kSkBK - 1) / kSkBK;
  p.units_total = tiles * p.num_kb;
  // `splits` > 0 forces that many CTAs per tile (tests); otherwise one CTA per SM
  int ctas = splits > 0 ? tiles * splits : sm_count();
  if (ctas > p.units_total) ctas = p.units_total;
  p.units_per_cta = (p.units_total + ctas - 1) / ctas;
  ctas = (p.units_total + p.units_per_cta - 1) / p.units_per_cta;
  // no more ring stages than a CTA has k-blocks to stream: a small GEMM then keeps little shared memory, and the first
  // CTAs of the next kernel of a programmatic-dependent-launch chain can become resident next to it
  if (p.stages > p.units_per_cta) p.stages = p.units_per_cta < 2 ? 2 : p.units_per_cta;
  B200_REQUIRE(scratch && tickets, "gemm_skinny needs scratch and tickets");
  CUtensorMap tw, tx;
  int rc = make_tma_2d(&tw, W, dtype, static_cast<uint64_t>(kw) * N, K, ldw, kSkBN, kSkBK, true);
  if (rc != kOk) return rc;
  rc = make_tma_2d(&tx, X, dtype, M, K, ldx, p.MB, kSkBK, true);
  if (rc != kOk) return rc;
  const int smem = p.stages * p.stage_bytes + 1024;
  dim3 grid(ctas);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dual ? launch_skinny<true>(tw, tx, p, grid, smem, s) : launch_skinny<false>(tw, tx, p, grid, smem, s);
}

B200_API int b200_gemm_skinny(const void* X, const void* W, void* C, int M, int N, int K, int ldx, int ldw, int ldc,
                              int dual, int dtype, float* scratch, uint32_t* tickets, int splits, void* stream) {
  return skinny_impl(X, W, C, M, N, K, ldx, ldw, ldc, dual, dtype, scratch, tickets, splits, nullptr, stream);
}

// As b200_gemm_skinny with a fused epilogue (M <= 16). `epilogue` points to a SkinnyEpilogue (see the top of this file;
// the Python binding mirrors its layout). C may be null for the kinds that write their own outputs.
B200_API int b200_gemm_skinny_fused(const void* X, const void* W, void* C, int M, int N, int K, int ldx, int ldw, int ldc,
                                    int dual, int dtype, float* scratch, uint32_t* tickets, const void* epilogue,
                                    void* stream) {
  B200_REQUIRE(epilogue != nullptr, "b200_gemm_skinny_fused needs an epilogue description");
  return skinny_impl(X, W, C, M, N, K, ldx, ldw, ldc, dual, dtype, scratch, tickets, 0,
                     static_cast<const SkinnyEpilogue*>(epilogue), stream);
}
// Tuning aid: while `buf` (device memory, 8 x u64 per CTA, at least 148 CTAs) is set, every decode GEMM launch writes
// %globaltimer checkpoints of each CTA there (0 start, 1 set-up done, 2 previous kernel complete, 3 last MMA issued,
// 4 last accumulator complete, 5 partial sums fenced, 6 ticket drawn, 7 CTA done). Pass null to switch it off.
B200_API int b200_gemm_skinny_set_trace(void* buf) {
  g_skinny_trace = static_cast<unsigned long long*>(buf);
  return kOk;
}
B200_API int b200_gemm_skinny_epilogue_bytes() { return static_cast<int>(sizeof(SkinnyEpilogue)); }

// ------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared and documented in b200/no_alloc_api.h).
// ------------------------------------------------------------------------------------------------
#include "b200/no_alloc_api.h"

#include <mutex>

namespace b200 {
constexpr long long kStaticScratchFloats = 1 << 20;
constexpr int kStaticTickets = 4096;
// The split accumulation area and the tickets, part of the library image on every device that loads it.
// In host code these names are stand-ins, not device addresses: the address a kernel may use comes from
// cudaGetSymbolAddress on the device in question.
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) uint32_t g_static_tickets[kStaticTickets];

struct StaticArea {
  float* scratch = nullptr;
  uint32_t* tickets = nullptr;
};
// Resolved once per device, with that device current. The table is filled under a lock, so host threads that make
// their first call on a device at the same time see either nothing or a complete entry.
static int static_area(StaticArea** out) {
  static StaticArea areas[64];
  static std::mutex mu;
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  StaticArea& a = areas[dev];
  if (a.scratch == nullptr) {
    void* ps = nullptr;
    void* pt = nullptr;
    B200_CHECK_CUDA(cudaGetSymbolAddress(&ps, g_static_scratch));
    B200_CHECK_CUDA(cudaGetSymbolAddress(&pt, g_static_tickets));
    a.tickets = static_cast<uint32_t*>(pt);
    a.scratch = static_cast<float*>(ps);
  }
  *out = &a;
  return kOk;
}
}  // namespace b200

B200_API long long b200_gemm_skinny_static_capacity_floats() { return b200::kStaticScratchFloats; }

B200_API int b200_gemm_skinny_static(const void* X, const void* W, void* C, int M, int N, int K, int ldx, int ldw,
                                     int ldc, int dual, int dtype, void* stream) {
  B200_REQUIRE(M >= 1 && M <= 256 && N >= 1, "b200_gemm_skinny_static: M must be in [1, 256] and N >= 1");
  const long long need = b200_gemm_skinny_scratch_floats(M, N, dual);
  const long long tiles = (N + kSkBN - 1) / kSkBN;
  B200_REQUIRE(need <= kStaticScratchFloats && tiles <= kStaticTickets,
               "b200_gemm_skinny_static: problem needs %lld scratch floats and %lld tiles; the built-in area holds "
               "%lld floats and %d tiles (use b200_gemm_skinny with caller-provided scratch instead)",
               need, tiles, kStaticScratchFloats, kStaticTickets);
  StaticArea* area = nullptr;
  int rc = static_area(&area);
  if (rc != kOk) return rc;
  return b200_gemm_skinny(X, W, C, M, N, K, ldx, ldw, ldc, dual, dtype, area->scratch, area->tickets, 0, stream);
}

B200_API int b200_gemm_skinny_static_reset(void* stream) {
  StaticArea* area = nullptr;
  int rc = static_area(&area);
  if (rc != kOk) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_CHECK_CUDA(cudaMemsetAsync(area->scratch, 0, sizeof(float) * kStaticScratchFloats, s));
  B200_CHECK_CUDA(cudaMemsetAsync(area->tickets, 0, sizeof(uint32_t) * kStaticTickets, s));
  return kOk;
}
