// Paged GQA decode attention with split-KV (flash-decoding) and the LSE-weighted combine used both
// inside a rank (over splits) and across ranks (sequence-parallel decode).
//
// Reference semantics: python/triton_dist/kernels/nvidia/flash_decode.py:130-239 (split-KV kernel: one
// program per (batch, head group, split), paged block_table, soft-cap, partial output + natural-log LSE),
// :308-360 / :393-449 / :482-532 (combine kernels; empty partials are skipped).
//
// Decode is bound by reading the KV cache once, so the design goal is HBM bandwidth, not tensor
// throughput: the <=16 query heads that share a KV head form the M=16 operand of warp-level
// m16n8k16 MMAs (a tcgen05 tile would be M>=64 and mostly padding), K/V stream through a
// double-buffered cp.async pipeline in 64-token tiles with a 16-byte XOR swizzle, and the four warps of
// a CTA each own 16 tokens of the tile and merge their running (max, sum, O) once at the end.
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/attn_merge.cuh"

#include <cstdlib>
#include <cstring>

namespace b200 {

constexpr int kD = 128;          // head dim
constexpr int kTile = 64;        // tokens per pipeline stage
constexpr int kAttnThreads = 128;
constexpr int kTileBytes = kTile * kD * 2;  // 16 KB
constexpr int kAttnSmem = 4 * kTileBytes;   // K,V x 2 stages

struct DecodeParams {
  const void* q;        // [B, Hq, D]
  const void* k_cache;  // [slots, Hkv, D], slot = block * page + offset
  const void* v_cache;
  const int* block_table;  // [B, bt_stride]
  const int* kv_lens;      // [B]
  float* o_part;           // [B, Hq, S, D]
  float* lse_part;         // [B, Hq, S]
  void* out;               // [B, Hq, D] when S == 1 and direct output is requested
  float* out_lse;          // [B, Hq] or null
  int bt_stride, Hq, Hkv, page, S;
  float scale, soft_cap;
  int direct;
  uint32_t* tickets;    // fused combine only: one self-resetting counter per (batch, head group)
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Fused combine: every CTA of a (batch, head group) draws a ticket after its partial is visible; the CTA
// that draws the last one merges all S partials (the arithmetic of decode_combine_kernel) and writes the final rows,
// so the separate combine launch disappears. The ticket resets itself for the next call.
template <bool BF16>
__device__ __forceinline__ void combine_by_last_cta(const DecodeParams& p, int b, int head0, int nrows) {
  __shared__ uint32_t is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ticket = p.tickets + static_cast<size_t>(b) * gridDim.y + blockIdx.y;
    const uint32_t t = atomicAdd(ticket, 1u);
    is_last = t == static_cast<uint32_t>(p.S - 1) ? 1u : 0u;
    if (is_last) *ticket = 0u;  // every CTA of the group has arrived
  }
  __syncthreads();
  if (is_last == 0u) return;
  __threadfence();
  for (int i = threadIdx.x; i < nrows * kD; i += blockDim.x) {
    const int r = i / kD, c = i - r * kD;
    const size_t bh = static_cast<size_t>(b) * p.Hq + head0 + r;
    float o, lse;
    merge_splits(p.lse_part + bh * p.S, 1, p.o_part + bh * p.S * kD + c, kD, p.S, o, lse);
    if (BF16) static_cast<__nv_bfloat16*>(p.out)[bh * kD + c] = __float2bfloat16(o);
    else static_cast<__half*>(p.out)[bh * kD + c] = __float2half(o);
    if (c == 0 && p.out_lse) p.out_lse[bh] = lse;
  }
}

template <bool BF16, bool FUSE = false>
__global__ void __launch_bounds__(kAttnThreads) decode_split_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  griddep_launch_dependents();
  griddep_wait();
  const int split = blockIdx.x, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int hgroups = (G + 15) / 16;
  const int kvh = blockIdx.y / hgroups, hg = blockIdx.y - kvh * hgroups;
  const int head0 = kvh * G + hg * 16;
  const int nrows = min(16, G - hg * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = p.kv_lens[b];
  int chunk = (kv_len + p.S - 1) / p.S;
  chunk = (chunk + kTile - 1) / kTile * kTile;
  const int t0 = split * chunk;
  const int t1 = min(kv_len, t0 + chunk);
  const int r_lo = lane >> 2, r_hi = r_lo + 8;

  if (t0 >= t1) {  // empty split: mark it so that the combine skips it
    if (!p.direct) {
      for (int r = threadIdx.x; r < nrows; r += blockDim.x)
        p.lse_part[(static_cast<size_t>(b) * p.Hq + head0 + r) * p.S + split] = -INFINITY;
      if (FUSE) combine_by_last_cta<BF16>(p, b, head0, nrows);
    } else {
      for (int i = threadIdx.x; i < nrows * kD; i += blockDim.x) {
        const size_t o = (static_cast<size_t>(b) * p.Hq + head0 + i / kD) * kD + (i % kD);
        if (BF16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16(0.f);
        else static_cast<__half*>(p.out)[o] = __float2half(0.f);
      }
      if (p.out_lse)
        for (int r = threadIdx.x; r < nrows; r += blockDim.x) p.out_lse[static_cast<size_t>(b) * p.Hq + head0 + r] = -INFINITY;
    }
    return;
  }

  // ---- Q fragments (A operand), rows >= nrows are zero ----
  uint32_t qa[8][4];
  {
    const uint32_t* q32 = static_cast<const uint32_t*>(p.q);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int c = kk * 16 + (lane & 3) * 2;
      const size_t base_lo = ((static_cast<size_t>(b) * p.Hq + head0 + r_lo) * kD + c) / 2;
      const size_t base_hi = ((static_cast<size_t>(b) * p.Hq + head0 + r_hi) * kD + c) / 2;
      qa[kk][0] = r_lo < nrows ? q32[base_lo] : 0u;
      qa[kk][1] = r_hi < nrows ? q32[base_hi] : 0u;
      qa[kk][2] = r_lo < nrows ? q32[base_lo + 4] : 0u;
      qa[kk][3] = r_hi < nrows ? q32[base_hi + 4] : 0u;
    }
  }

  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  auto k_stage = [&](int s) { return smem_base + s * kTileBytes; };
  auto v_stage = [&](int s) { return smem_base + (2 + s) * kTileBytes; };
  const uint8_t* kc = static_cast<const uint8_t*>(p.k_cache);
  const uint8_t* vc = static_cast<const uint8_t*>(p.v_cache);

  auto load_tile = [&](int tile_t0, int s) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int tok_in = i * 8 + (threadIdx.x >> 4);
      const int c = threadIdx.x & 15;
      const int tok = tile_t0 + tok_in;
      const bool valid = tok < t1;
      size_t off = 0;
      if (valid) {
        const int blk = p.block_table[static_cast<size_t>(b) * p.bt_stride + tok / p.page];
        const size_t slot = static_cast<size_t>(blk) * p.page + tok % p.page;
        off = ((slot * p.Hkv + kvh) * kD + c * 8) * 2;
      }
      const uint32_t so = tok_in * 256 + ((c ^ (tok_in & 7)) * 16);
      cp_async_16(k_stage(s) + so, kc + off, valid ? 16 : 0);
      cp_async_16(v_stage(s) + so, vc + off, valid ? 16 : 0);
    }
    cp_async_commit();
  };

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;

  const float kLog2e = 1.4426950408889634f;
  const int ntiles = (t1 - t0 + kTile - 1) / kTile;
  load_tile(t0, 0);
  for (int it = 0; it < ntiles; ++it) {
    const int s = it & 1;
    if (it + 1 < ntiles) {
      load_tile(t0 + (it + 1) * kTile, s ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int wt0 = t0 + it * kTile + warp * 16;  // first token of this warp's slice
    if (wt0 < t1) {
      // ---- S = Q K^T for 16 tokens ----
      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int m = lane >> 3, r = lane & 7;
        const int tok_in = warp * 16 + (m >> 1) * 8 + r;
        const int c = 2 * kk + (m & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(k_stage(s) + tok_in * 256 + ((c ^ (tok_in & 7)) * 16), b0, b1, b2, b3);
        mma16816<BF16>(sacc[0], qa[kk], b0, b1);
        mma16816<BF16>(sacc[1], qa[kk], b2, b3);
      }
      // ---- scale, soft-cap, mask, online softmax (base-2 domain) ----
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sacc[nb][e] * p.scale;
          if (p.soft_cap > 0.f) v = p.soft_cap * tanhf(v / p.soft_cap);
          v *= kLog2e;
          const int tok = wt0 + nb * 8 + (lane & 3) * 2 + (e & 1);
          v = tok < t1 ? v : -INFINITY;
          sacc[nb][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      uint32_t pa[4];
      float pr[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h]);
        const float base = m_new == -INFINITY ? 0.f : m_new;
        const float corr = exp2f(m_run[h] - base);  // m_run = -inf -> 0
        m_run[h] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float pv = exp2f(sacc[nb][2 * h + e] - base);
            pr[nb][2 * h + e] = pv;
            sum += pv;
          }
        l_run[h] = l_run[h] * corr + sum;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          oacc[i][2 * h] *= corr;
          oacc[i][2 * h + 1] *= corr;
        }
      }
      if (BF16) {
        pa[0] = pack_bf16x2(pr[0][0], pr[0][1]); pa[1] = pack_bf16x2(pr[0][2], pr[0][3]);
        pa[2] = pack_bf16x2(pr[1][0], pr[1][1]); pa[3] = pack_bf16x2(pr[1][2], pr[1][3]);
      } else {
        pa[0] = pack_f16x2(pr[0][0], pr[0][1]); pa[1] = pack_f16x2(pr[0][2], pr[0][3]);
        pa[2] = pack_f16x2(pr[1][0], pr[1][1]); pa[3] = pack_f16x2(pr[1][2], pr[1][3]);
      }
      // ---- O += P V ----
#pragma unroll
      for (int dn = 0; dn < 8; ++dn) {
        const int m = lane >> 3, r = lane & 7;
        const int tok_in = warp * 16 + (m & 1) * 8 + r;
        const int c = 2 * dn + (m >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(v_stage(s) + tok_in * 256 + ((c ^ (tok_in & 7)) * 16), b0, b1, b2, b3);
        mma16816<BF16>(oacc[2 * dn], pa, b0, b1);
        mma16816<BF16>(oacc[2 * dn + 1], pa, b2, b3);
      }
    }
    __syncthreads();
  }

  // ---- merge the four warps ----
  float* red_m = reinterpret_cast<float*>(smem);            // [4][16]
  float* red_l = red_m + 64;                                // [4][16]
  float* red_o = red_l + 64;                                // [4][16][128]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  if ((lane & 3) == 0) {
    red_m[warp * 16 + r_lo] = m_run[0];
    red_m[warp * 16 + r_hi] = m_run[1];
    red_l[warp * 16 + r_lo] = l_run[0];
    red_l[warp * 16 + r_hi] = l_run[1];
  }
  __syncthreads();
  float scale_w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h ? r_hi : r_lo;
    float mg = fmaxf(fmaxf(red_m[r], red_m[16 + r]), fmaxf(red_m[32 + r], red_m[48 + r]));
    scale_w[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - mg);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int c = i * 8 + (lane & 3) * 2;
    float* lo = red_o + (warp * 16 + r_lo) * kD + c;
    float* hi = red_o + (warp * 16 + r_hi) * kD + c;
    lo[0] = oacc[i][0] * scale_w[0];
    lo[1] = oacc[i][1] * scale_w[0];
    hi[0] = oacc[i][2] * scale_w[1];
    hi[1] = oacc[i][3] * scale_w[1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * kD; i += blockDim.x) {
    const int r = i / kD, c = i - r * kD;
    float mg = fmaxf(fmaxf(red_m[r], red_m[16 + r]), fmaxf(red_m[32 + r], red_m[48 + r]));
    float lg = 0.f, og = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_m[w * 16 + r];
      lg += mw == -INFINITY ? 0.f : red_l[w * 16 + r] * exp2f(mw - mg);
      og += red_o[(w * 16 + r) * kD + c];
    }
    const float o = lg > 0.f ? og / lg : 0.f;
    const size_t bh = static_cast<size_t>(b) * p.Hq + head0 + r;
    const float lse = lg > 0.f ? mg * 0.6931471805599453f + logf(lg) : -INFINITY;
    if (p.direct) {
      if (BF16) static_cast<__nv_bfloat16*>(p.out)[bh * kD + c] = __float2bfloat16(o);
      else static_cast<__half*>(p.out)[bh * kD + c] = __float2half(o);
      if (c == 0 && p.out_lse) p.out_lse[bh] = lse;
    } else {
      p.o_part[(bh * p.S + split) * kD + c] = o;
      if (c == 0) p.lse_part[bh * p.S + split] = lse;
    }
  }
  if (FUSE && !p.direct) combine_by_last_cta<BF16>(p, b, head0, nrows);
}

// ------------------------------------------------------------------------------------------------
// Variant with one private cp.async ring per warp.
//
// The kernel above keeps at most one 32 KB tile per CTA in flight while it computes the other one; with three CTAs
// per SM that is ~96 KB in flight per SM, and the measured 0.57 of the copy peak is what Little's law gives for that
// at the loaded HBM latency (the decode GEMM needs its 216 KB ring to reach 0.87). Here every warp streams its own
// 16-token slices (4 KB of K + 4 KB of V) through a ring of kNST slots without any CTA-wide barrier in the loop:
// 4 warps x (kNST - 1) slices x 8 KB in flight per CTA (160 KB with kNST = 6 and one CTA per SM, 2 x 64 KB with
// kNST = 3 and two). Warp w takes slices w, w + 4, w + 8, ... so that the four warps together read consecutive
// 64-token tiles. The arithmetic per slice and the final merge of the four warps are those of the kernel above.
template <bool BF16, int kNST, bool FUSE = false>
__global__ void __launch_bounds__(kAttnThreads) decode_split_ring_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  griddep_launch_dependents();
  griddep_wait();
  constexpr int kSlice = 16;                      // tokens per slice
  constexpr int kSliceBytes = kSlice * kD * 2;    // 4 KB (K or V)
  const int split = blockIdx.x, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int hgroups = (G + 15) / 16;
  const int kvh = blockIdx.y / hgroups, hg = blockIdx.y - kvh * hgroups;
  const int head0 = kvh * G + hg * 16;
  const int nrows = min(16, G - hg * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = p.kv_lens[b];
  int chunk = (kv_len + p.S - 1) / p.S;
  chunk = (chunk + kTile - 1) / kTile * kTile;
  const int t0 = split * chunk;
  const int t1 = min(kv_len, t0 + chunk);
  const int r_lo = lane >> 2, r_hi = r_lo + 8;

  if (t0 >= t1) {  // empty split: mark it so that the combine skips it
    if (!p.direct) {
      for (int r = threadIdx.x; r < nrows; r += blockDim.x)
        p.lse_part[(static_cast<size_t>(b) * p.Hq + head0 + r) * p.S + split] = -INFINITY;
      if (FUSE) combine_by_last_cta<BF16>(p, b, head0, nrows);
    } else {
      for (int i = threadIdx.x; i < nrows * kD; i += blockDim.x) {
        const size_t o = (static_cast<size_t>(b) * p.Hq + head0 + i / kD) * kD + (i % kD);
        if (BF16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16(0.f);
        else static_cast<__half*>(p.out)[o] = __float2half(0.f);
      }
      if (p.out_lse)
        for (int r = threadIdx.x; r < nrows; r += blockDim.x) p.out_lse[static_cast<size_t>(b) * p.Hq + head0 + r] = -INFINITY;
    }
    return;
  }

  uint32_t qa[8][4];
  {
    const uint32_t* q32 = static_cast<const uint32_t*>(p.q);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int c = kk * 16 + (lane & 3) * 2;
      const size_t base_lo = ((static_cast<size_t>(b) * p.Hq + head0 + r_lo) * kD + c) / 2;
      const size_t base_hi = ((static_cast<size_t>(b) * p.Hq + head0 + r_hi) * kD + c) / 2;
      qa[kk][0] = r_lo < nrows ? q32[base_lo] : 0u;
      qa[kk][1] = r_hi < nrows ? q32[base_hi] : 0u;
      qa[kk][2] = r_lo < nrows ? q32[base_lo + 4] : 0u;
      qa[kk][3] = r_hi < nrows ? q32[base_hi + 4] : 0u;
    }
  }

  // this warp's ring: slot s holds K at +0 and V at +kSliceBytes
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * (kNST * 2 * kSliceBytes);
  const uint8_t* kc = static_cast<const uint8_t*>(p.k_cache);
  const uint8_t* vc = static_cast<const uint8_t*>(p.v_cache);
  const int nslices_cta = (t1 - t0 + kSlice - 1) / kSlice;
  const int my_slices = nslices_cta > warp ? (nslices_cta - warp + 3) / 4 : 0;   // slices warp, warp + 4, ...
  const bool page_fast = (p.page % kSlice) == 0;   // a 16-token slice never crosses a page (t0 is a multiple of 64)

  auto load_slice = [&](int j) {   // j-th slice of this warp; always commits a group so that the counting stays uniform
    if (j < my_slices) {
      const int st0 = t0 + (warp + 4 * j) * kSlice;
      const uint32_t slot = ring + (j % kNST) * (2 * kSliceBytes);
      size_t slot0 = 0;
      if (page_fast) {
        const int blk = p.block_table[static_cast<size_t>(b) * p.bt_stride + st0 / p.page];
        slot0 = static_cast<size_t>(blk) * p.page + st0 % p.page;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int tok_in = i * 2 + (lane >> 4);
        const int c = lane & 15;
        const int tok = st0 + tok_in;
        const bool valid = tok < t1;
        size_t off = 0;
        if (valid) {
          size_t sl;
          if (page_fast) {
            sl = slot0 + tok_in;
          } else {
            const int blk = p.block_table[static_cast<size_t>(b) * p.bt_stride + tok / p.page];
            sl = static_cast<size_t>(blk) * p.page + tok % p.page;
          }
          off = ((sl * p.Hkv + kvh) * kD + c * 8) * 2;
        }
        const uint32_t so = tok_in * 256 + ((c ^ (tok_in & 7)) * 16);
        cp_async_16(slot + so, kc + off, valid ? 16 : 0);
        cp_async_16(slot + kSliceBytes + so, vc + off, valid ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;

  const float kLog2e = 1.4426950408889634f;
#pragma unroll
  for (int j = 0; j < kNST - 1; ++j) load_slice(j);
  for (int j = 0; j < my_slices; ++j) {
    load_slice(j + kNST - 1);        // into the slot that was computed in the previous iteration
    cp_async_wait<kNST - 1>();       // slice j has landed (for this lane); the barrier below covers the other lanes
    __syncwarp();
    const uint32_t ks = ring + (j % kNST) * (2 * kSliceBytes), vs = ks + kSliceBytes;
    const int wt0 = t0 + (warp + 4 * j) * kSlice;  // first token of this slice
    // ---- S = Q K^T for 16 tokens ----
    float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const int m = lane >> 3, r = lane & 7;
      const int tok_in = (m >> 1) * 8 + r;
      const int c = 2 * kk + (m & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(ks + tok_in * 256 + ((c ^ (tok_in & 7)) * 16), b0, b1, b2, b3);
      mma16816<BF16>(sacc[0], qa[kk], b0, b1);
      mma16816<BF16>(sacc[1], qa[kk], b2, b3);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = sacc[nb][e] * p.scale;
        if (p.soft_cap > 0.f) v = p.soft_cap * tanhf(v / p.soft_cap);
        v *= kLog2e;
        const int tok = wt0 + nb * 8 + (lane & 3) * 2 + (e & 1);
        v = tok < t1 ? v : -INFINITY;
        sacc[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    uint32_t pa[4];
    float pr[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m_run[h] - base);  // m_run = -inf -> 0
      m_run[h] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(sacc[nb][2 * h + e] - base);
          pr[nb][2 * h + e] = pv;
          sum += pv;
        }
      l_run[h] = l_run[h] * corr + sum;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        oacc[i][2 * h] *= corr;
        oacc[i][2 * h + 1] *= corr;
      }
    }
    if (BF16) {
      pa[0] = pack_bf16x2(pr[0][0], pr[0][1]); pa[1] = pack_bf16x2(pr[0][2], pr[0][3]);
      pa[2] = pack_bf16x2(pr[1][0], pr[1][1]); pa[3] = pack_bf16x2(pr[1][2], pr[1][3]);
    } else {
      pa[0] = pack_f16x2(pr[0][0], pr[0][1]); pa[1] = pack_f16x2(pr[0][2], pr[0][3]);
      pa[2] = pack_f16x2(pr[1][0], pr[1][1]); pa[3] = pack_f16x2(pr[1][2], pr[1][3]);
    }
#pragma unroll
    for (int dn = 0; dn < 8; ++dn) {
      const int m = lane >> 3, r = lane & 7;
      const int tok_in = (m & 1) * 8 + r;
      const int c = 2 * dn + (m >> 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vs + tok_in * 256 + ((c ^ (tok_in & 7)) * 16), b0, b1, b2, b3);
      mma16816<BF16>(oacc[2 * dn], pa, b0, b1);
      mma16816<BF16>(oacc[2 * dn + 1], pa, b2, b3);
    }
    __syncwarp();  // every lane is done with this slot before the next iteration's copies overwrite the previous one
  }
  cp_async_wait<0>();
  __syncthreads();   // all rings are idle: their memory becomes the merge area

  // ---- merge the four warps ----
  float* red_m = reinterpret_cast<float*>(smem);            // [4][16]
  float* red_l = red_m + 64;                                // [4][16]
  float* red_o = red_l + 64;                                // [4][16][128]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  if ((lane & 3) == 0) {
    red_m[warp * 16 + r_lo] = m_run[0];
    red_m[warp * 16 + r_hi] = m_run[1];
    red_l[warp * 16 + r_lo] = l_run[0];
    red_l[warp * 16 + r_hi] = l_run[1];
  }
  __syncthreads();
  float scale_w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h ? r_hi : r_lo;
    float mg = fmaxf(fmaxf(red_m[r], red_m[16 + r]), fmaxf(red_m[32 + r], red_m[48 + r]));
    scale_w[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - mg);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int c = i * 8 + (lane & 3) * 2;
    float* lo = red_o + (warp * 16 + r_lo) * kD + c;
    float* hi = red_o + (warp * 16 + r_hi) * kD + c;
    lo[0] = oacc[i][0] * scale_w[0];
    lo[1] = oacc[i][1] * scale_w[0];
    hi[0] = oacc[i][2] * scale_w[1];
    hi[1] = oacc[i][3] * scale_w[1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * kD; i += blockDim.x) {
    const int r = i / kD, c = i - r * kD;
    float mg = fmaxf(fmaxf(red_m[r], red_m[16 + r]), fmaxf(red_m[32 + r], red_m[48 + r]));
    float lg = 0.f, og = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_m[w * 16 + r];
      lg += mw == -INFINITY ? 0.f : red_l[w * 16 + r] * exp2f(mw - mg);
      og += red_o[(w * 16 + r) * kD + c];
    }
    const float o = lg > 0.f ? og / lg : 0.f;
    const size_t bh = static_cast<size_t>(b) * p.Hq + head0 + r;
    const float lse = lg > 0.f ? mg * 0.6931471805599453f + logf(lg) : -INFINITY;
    if (p.direct) {
      if (BF16) static_cast<__nv_bfloat16*>(p.out)[bh * kD + c] = __float2bfloat16(o);
      else static_cast<__half*>(p.out)[bh * kD + c] = __float2half(o);
      if (c == 0 && p.out_lse) p.out_lse[bh] = lse;
    } else {
      p.o_part[(bh * p.S + split) * kD + c] = o;
      if (c == 0) p.lse_part[bh * p.S + split] = lse;
    }
  }
  if (FUSE && !p.direct) combine_by_last_cta<BF16>(p, b, head0, nrows);
}

// out[bh, :] = sum_s w_s o[bh, s, :] / sum_s w_s with w_s = exp(lse_s - max lse); partials with
// lse = -inf are skipped. Strides are in elements so the same kernel merges split partials
// ([B*Hq, S, D]) and the all-gathered per-rank partials of sequence-parallel decode ([R, B*Hq, D(+1)]).
template <bool BF16>
__global__ void __launch_bounds__(kD) decode_combine_kernel(const float* o_part, const float* lse_part, long long o_stride_bh,
                                                            long long o_stride_s, long long lse_stride_bh,
                                                            long long lse_stride_s, int S, void* out, float* out_f32,
                                                            float* out_lse) {
  const int bh = blockIdx.x, c = threadIdx.x;
  griddep_launch_dependents();
  griddep_wait();
  float o, lse;
  merge_splits(lse_part + bh * lse_stride_bh, lse_stride_s, o_part + bh * o_stride_bh + c, o_stride_s, S, o, lse);
  if (out) {
    if (BF16) static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(bh) * kD + c] = __float2bfloat16(o);
    else static_cast<__half*>(out)[static_cast<size_t>(bh) * kD + c] = __float2half(o);
  }
  if (out_f32) out_f32[static_cast<size_t>(bh) * kD + c] = o;
  if (c == 0 && out_lse) out_lse[bh] = lse;
}

// Pipeline variant when the caller passes ring < 0: B200DIST_ATTN_V2 = 0 (two-stage CTA-wide pipeline), 3 or 6
// (per-warp rings of that depth) forces one; unset picks the three-deep rings (two CTAs of 96 KB per SM), which
// measured fastest from 2 K to 128 K tokens per sequence: 4.7-4.9 TB/s at batch 8 x 16 K and batch 32 x 4 K against
// 3.7-3.8 TB/s for the CTA-wide pipeline and 3.1-3.2 TB/s for six-deep rings (one CTA per SM).
static int attn_ring_default() {
  static int stages = -1;
  if (stages < 0) {
    const char* e = getenv("B200DIST_ATTN_V2");
    if (!e) stages = 3;
    else {
      const int v = atoi(e);
      stages = v == 3 ? 3 : (v == 6 || v == 1) ? 6 : 0;
    }
  }
  return stages;
}

template <typename K>
static int set_smem(K kernel, int bytes) {
  B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return kOk;
}

}  // namespace b200

using namespace b200;

// Paged GQA decode attention with split-KV.
//   q [B,Hq,128]; caches [num_blocks, page, Hkv, 128]; block_table [B, bt_stride] int32; kv_lens [B] int32.
//   num_splits == 1 writes `out` (and out_lse) directly.
//   num_splits > 1 fills o_part [B,Hq,S,128] / lse_part [B,Hq,S] (fp32 scratch). With `tickets` (u32
//   [B * Hkv * ceil(G / 16)], zero-initialised once; the kernel leaves it zeroed) the CTA that finishes last in a
//   (batch, head group) merges the partials and writes `out` / `out_lse`, so no combine launch follows; without
//   tickets the caller merges them (b200_decode_combine, or the cross-rank merge of sequence-parallel decode).
//   ring: 0 = two-stage CTA-wide cp.async pipeline, 3 / 6 = one private ring of that depth per warp, < 0 = default.
B200_API int b200_decode_attn(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                              int bt_stride, const int* kv_lens, int B, int Hq, int Hkv, int head_dim, int page,
                              float scale, float soft_cap, int num_splits, float* o_part, float* lse_part,
                              uint32_t* tickets, void* out, float* out_lse, int dtype, int ring, void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "decode attention supports bf16/f16");
  B200_REQUIRE(head_dim == kD, "decode attention is specialised for head_dim 128, got %d", head_dim);
  B200_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "Hq (%d) must be a multiple of Hkv (%d)", Hq, Hkv);
  B200_REQUIRE(num_splits >= 1 && page >= 1, "bad num_splits/page");
  if (ring < 0) ring = attn_ring_default();
  B200_REQUIRE(ring == 0 || ring == 3 || ring == 6, "ring must be 0, 3 or 6, got %d", ring);
  if (B == 0) return kOk;
  const bool fuse = tickets != nullptr && num_splits > 1;
  B200_REQUIRE(!fuse || out != nullptr, "the fused combine writes `out`");
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  static bool configured[64] = {false};
  if (!configured[dev & 63]) {
    int rc = kOk;
#define B200_ATTN_SMEM(BF, FU)                                                                \
    if (rc == kOk) rc = set_smem(decode_split_kernel<BF, FU>, kAttnSmem);                       \
    if (rc == kOk) rc = set_smem(decode_split_ring_kernel<BF, 3, FU>, 96 * 1024);               \
    if (rc == kOk) rc = set_smem(decode_split_ring_kernel<BF, 6, FU>, 192 * 1024);
    B200_ATTN_SMEM(true, false) B200_ATTN_SMEM(false, false) B200_ATTN_SMEM(true, true) B200_ATTN_SMEM(false, true)
#undef B200_ATTN_SMEM
    if (rc != kOk) return rc;
    configured[dev & 63] = true;
  }
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.kv_lens = kv_lens;
  p.o_part = o_part; p.lse_part = lse_part; p.out = out; p.out_lse = out_lse; p.tickets = tickets;
  p.bt_stride = bt_stride; p.Hq = Hq; p.Hkv = Hkv; p.page = page; p.S = num_splits;
  p.scale = scale; p.soft_cap = soft_cap; p.direct = num_splits == 1 && out != nullptr;
  B200_REQUIRE(p.direct || (o_part && lse_part), "split partial buffers are required when num_splits > 1");
  const int G = Hq / Hkv;
  dim3 grid(num_splits, Hkv * ((G + 15) / 16), B);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf = dtype == kBF16;
  const int smem = ring == 0 ? kAttnSmem : ring == 3 ? 96 * 1024 : 192 * 1024;
#define B200_ATTN_LAUNCH(KERNEL) B200_CHECK_CUDA(launch_pdl(KERNEL, grid, kAttnThreads, smem, s, p))
  if (ring == 0) {
    if (bf && fuse) B200_ATTN_LAUNCH((decode_split_kernel<true, true>));
    else if (bf) B200_ATTN_LAUNCH((decode_split_kernel<true, false>));
    else if (fuse) B200_ATTN_LAUNCH((decode_split_kernel<false, true>));
    else B200_ATTN_LAUNCH((decode_split_kernel<false, false>));
  } else if (ring == 3) {
    if (bf && fuse) B200_ATTN_LAUNCH((decode_split_ring_kernel<true, 3, true>));
    else if (bf) B200_ATTN_LAUNCH((decode_split_ring_kernel<true, 3, false>));
    else if (fuse) B200_ATTN_LAUNCH((decode_split_ring_kernel<false, 3, true>));
    else B200_ATTN_LAUNCH((decode_split_ring_kernel<false, 3, false>));
  } else {
    if (bf && fuse) B200_ATTN_LAUNCH((decode_split_ring_kernel<true, 6, true>));
    else if (bf) B200_ATTN_LAUNCH((decode_split_ring_kernel<true, 6, false>));
    else if (fuse) B200_ATTN_LAUNCH((decode_split_ring_kernel<false, 6, true>));
    else B200_ATTN_LAUNCH((decode_split_ring_kernel<false, 6, false>));
  }
#undef B200_ATTN_LAUNCH
  return kOk;
}

// Earlier entry points, kept for callers of the C ABI: split only (the caller merges), and split with the fused merge.
B200_API int b200_decode_attn_split(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                    int bt_stride, const int* kv_lens, int B, int Hq, int Hkv, int head_dim, int page,
                                    float scale, float soft_cap, int num_splits, float* o_part, float* lse_part,
                                    void* out, float* out_lse, int dtype, void* stream) {
  return b200_decode_attn(q, k_cache, v_cache, block_table, bt_stride, kv_lens, B, Hq, Hkv, head_dim, page, scale, soft_cap,
                          num_splits, o_part, lse_part, nullptr, out, out_lse, dtype, -1, stream);
}
B200_API int b200_decode_attn_fused(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                    int bt_stride, const int* kv_lens, int B, int Hq, int Hkv, int head_dim, int page,
                                    float scale, float soft_cap, int num_splits, float* o_part, float* lse_part,
                                    uint32_t* tickets, void* out, float* out_lse, int dtype, void* stream) {
  B200_REQUIRE(num_splits >= 2 && tickets, "the fused combine is for num_splits >= 2 and needs tickets");
  return b200_decode_attn(q, k_cache, v_cache, block_table, bt_stride, kv_lens, B, Hq, Hkv, head_dim, page, scale, soft_cap,
                          num_splits, o_part, lse_part, tickets, out, out_lse, dtype, -1, stream);
}

B200_API int b200_decode_combine(const float* o_part, const float* lse_part, long long o_stride_bh, long long o_stride_s,
                                 long long lse_stride_bh, long long lse_stride_s, int BH, int S, void* out, float* out_f32,
                                 float* out_lse, int dtype, void* stream) {
  if (BH == 0) return kOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == kBF16)
    B200_CHECK_CUDA(launch_pdl(decode_combine_kernel<true>, BH, kD, 0, s, o_part, lse_part, o_stride_bh, o_stride_s,
                               lse_stride_bh, lse_stride_s, S, out, out_f32, out_lse));
  else
    B200_CHECK_CUDA(launch_pdl(decode_combine_kernel<false>, BH, kD, 0, s, o_part, lse_part, o_stride_bh, o_stride_s,
                               lse_stride_bh, lse_stride_s, S, out, out_f32, out_lse));
  return kOk;
}
