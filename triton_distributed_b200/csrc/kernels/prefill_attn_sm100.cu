// Causal (or full) variable-length prefill attention for sm_100a, head dim 128, GQA, bf16 / f16.
//
//   out[q, h, :] = softmax(scale * Q[q, h, :] . K[keys of q's sequence, kvh(h), :]^T) V[...]     (bottom-right causal mask)
//
// One CTA owns 128 query rows of one head and walks the keys in steps of 128:
//   warp 0     TMA producer: the Q tile once, then K and V^T tiles through two-stage rings (128-byte swizzle)
//   warp 1     one elected thread issues tcgen05.mma: S = Q K^T into one of two 128-column TMEM buffers (so the
//              scores of step j + 1 are computed while step j is in the softmax), then O_step = P V into a third
//   warps 4-11 softmax, two threads per query row (each owns 64 of the 128 score / output columns; the row maximum is
//              exchanged through shared memory): read S twice from TMEM (max, then exp2), write P as 16-bit into a
//              swizzled shared-memory tile that is the A operand of the second MMA, and keep the running output row
//              in 2 x 64 fp32 registers: O = O * exp2(m_old - m_new) + O_step, so tensor memory never has to be rescaled
// V is the B operand of the second MMA and has to be K-major ([d, keys]); a small kernel transposes it once per call
// into a zero-padded [batch x kv head, 128, padded keys] buffer, O(S d) work against the O(S^2 d) of the attention.
// Every barrier wait is bounded; on expiry the CTA unwinds through an abort flag and reports a status.
//
// Role in the reference: flash_attn_with_kvcache in layers/nvidia/tp_attn.py:194-195 (prefill) and the Triton
// flash-attention consumer of the sequence-parallel all-gather path, kernels/nvidia/sp_ag_attention_intra_node.py:255-425.
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/tcgen05.cuh"

#include <cstring>

namespace b200 {

constexpr int kPD = 128;                    // head dim
constexpr int kPM = 128, kPN = 128;         // query rows per CTA, keys per step
constexpr int kPAtom = 128 * 64 * 2;        // one 128-row x 64-column 16-bit swizzle atom: 16 KB
constexpr int kPTile = 2 * kPAtom;          // a 128 x 128 tile: 32 KB
constexpr int kPSmem = kPTile /*Q*/ + 2 * kPTile /*K*/ + 2 * kPTile /*V^T*/ + kPTile /*P*/ + 1024 + 256 + 3072 /*max / sum exchange*/;
constexpr int kPThreads = 384;

struct PrefillParams {
  int Hq, Hkv, causal, bf16;
  const int* cu_q;      // [B + 1] first packed query row of every sequence
  const int* cu_k;      // [B + 1] first key row of every sequence (only [0, B) is read when k_lens is given)
  const int* k_lens;    // nullable [B]: keys of every sequence; null = cu_k[b + 1] - cu_k[b] (packed sequences)
  float scale_log2e;    // softmax scale * log2(e)
  void* out;            // [total_q, Hq, 128]
  uint32_t* status;     // nullable: set non-zero when a pipeline wait expired
};

// 2^x on the special-function unit (one instruction; -inf gives 0, which is what a masked score must contribute)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// barrier of the 256 softmax threads (warps 4-11) only
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// V [total_k, Hkv, 128] -> Vt [B * Hkv, 128, s_pad] (keys contiguous, zero beyond each sequence's length)
__global__ void __launch_bounds__(256) transpose_v_kernel(const uint16_t* __restrict__ v, uint16_t* __restrict__ vt,
                                                          const int* __restrict__ cu_k, const int* __restrict__ k_lens,
                                                          int Hkv, int s_pad) {
  __shared__ uint16_t tile[32][33];
  const int bh = blockIdx.z, b = bh / Hkv, kvh = bh - b * Hkv;
  const int k_start = cu_k[b], k_len = k_lens ? k_lens[b] : cu_k[b + 1] - k_start;
  const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    const int s = s0 + i;
    tile[i][tx] = s < k_len ? v[(static_cast<size_t>(k_start + s) * Hkv + kvh) * kPD + d0 + tx] : uint16_t(0);
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int s = s0 + tx;
    if (s < s_pad) vt[(static_cast<size_t>(bh) * kPD + d0 + i) * s_pad + s] = tile[tx][i];
  }
}

__global__ void __launch_bounds__(kPThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmVt, const PrefillParams p) {
  const int m_blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_start = p.cu_q[b], q_len = p.cu_q[b + 1] - q_start;
  const int k_start = p.cu_k[b], k_len = p.k_lens ? p.k_lens[b] : p.cu_k[b + 1] - k_start;
  if (m_blk * kPM >= q_len) return;  // uniform over the CTA, before anything is allocated
  const int kvh = h / (p.Hq / p.Hkv);
  const int offset = k_len - q_len;  // bottom-right alignment of the causal mask
  int kv_end = k_len;
  if (p.causal) kv_end = max(0, min(k_len, m_blk * kPM + kPM + offset));
  const int n_steps = (kv_end + kPN - 1) / kPN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kPTile;       // [2 stages][2 atoms]
  uint8_t* sV = sK + 2 * kPTile;   // [2 stages][2 atoms], V^T: rows = d, columns = keys
  uint8_t* sP = sV + 2 * kPTile;   // [2 atoms], rows = queries, columns = keys
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPTile);
  uint64_t* q_full = bars;          // [1]
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* s_empty = bars + 11;    // [2]
  uint64_t* p_full = bars + 13;     // [1]
  uint64_t* o_full = bars + 14;     // [1]
  uint64_t* o_empty = bars + 15;    // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* xmax = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [2 step parities][2 halves][128 rows]
  float* xsum = xmax + 4 * kPM;                                                    // [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t timeout_ns = 4000000000ull;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
      mbar_init(s_full + i, 1);
      mbar_init(s_empty + i, 8);
    }
    mbar_init(p_full, 8);
    mbar_init(o_full, 1);
    mbar_init(o_empty, 8);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmVt);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;  // columns [0,128) S0, [128,256) S1, [256,384) O_step

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_steps > 0) {  // nothing may be in flight into shared memory when nobody will wait for it
      mbar_expect_tx(q_full, kPTile);
      tma_load_3d(sQ, &tmQ, q_full, 0, h, q_start + m_blk * kPM);
      tma_load_3d(sQ + kPAtom, &tmQ, q_full, 64, h, q_start + m_blk * kPM);
      for (int j = 0; j < n_steps; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_empty + st, ph ^ 1, abort_flag, timeout_ns)) break;
        mbar_expect_tx(k_full + st, kPTile);
        tma_load_3d(sK + st * kPTile, &tmK, k_full + st, 0, kvh, k_start + j * kPN);
        tma_load_3d(sK + st * kPTile + kPAtom, &tmK, k_full + st, 64, kvh, k_start + j * kPN);
        if (!mbar_wait(v_empty + st, ph ^ 1, abort_flag, timeout_ns)) break;
        mbar_expect_tx(v_full + st, kPTile);
        tma_load_3d(sV + st * kPTile, &tmVt, v_full + st, j * kPN, 0, b * p.Hkv + kvh);
        tma_load_3d(sV + st * kPTile + kPAtom, &tmVt, v_full + st, j * kPN + 64, 0, b * p.Hkv + kvh);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_steps > 0) {
      const uint32_t idesc = umma_idesc_f16(kPM, kPN, p.bf16 != 0);
      bool ok = mbar_wait(q_full, 0, abort_flag, timeout_ns);
      auto issue_scores = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_full + st, ph, abort_flag, timeout_ns)) return false;
        if (!mbar_wait(s_empty + st, ph ^ 1, abort_flag, timeout_ns)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kPD / 16; ++kk) {
          const uint64_t da = umma_desc_sw128_kmajor(smem_u32(sQ + (kk >> 2) * kPAtom)) + 2 * (kk & 3);
          const uint64_t db = umma_desc_sw128_kmajor(smem_u32(sK + st * kPTile + (kk >> 2) * kPAtom)) + 2 * (kk & 3);
          umma_f16(tmem_base + st * kPN, da, db, idesc, kk != 0 ? 1u : 0u);
        }
        umma_commit(k_empty + st);
        umma_commit(s_full + st);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < n_steps && ok; ++j) {
        if (j + 1 < n_steps) ok = issue_scores(j + 1);
        if (!ok) break;
        const int st = j & 1;
        if (!mbar_wait(p_full, j & 1, abort_flag, timeout_ns)) break;
        if (!mbar_wait(v_full + st, (j >> 1) & 1, abort_flag, timeout_ns)) break;
        if (!mbar_wait(o_empty, (j & 1) ^ 1, abort_flag, timeout_ns)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kPN / 16; ++kk) {
          const uint64_t da = umma_desc_sw128_kmajor(smem_u32(sP + (kk >> 2) * kPAtom)) + 2 * (kk & 3);
          const uint64_t db = umma_desc_sw128_kmajor(smem_u32(sV + st * kPTile + (kk >> 2) * kPAtom)) + 2 * (kk & 3);
          umma_f16(tmem_base + 2 * kPN, da, db, idesc, kk != 0 ? 1u : 0u);
        }
        umma_commit(v_empty + st);
        umma_commit(o_full);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + output accumulation
    // Two threads per query row: warps 4-7 own score / output columns [0, 64) of the 128-wide tile, warps 8-11 columns
    // [64, 128) (two warps per scheduler instead of one, and half the serial chain per thread). The halves exchange
    // their row maxima through shared memory once per step and their row sums once at the end.
    const int sw = warp - 4;
    const int w4 = sw & 3;    // == warp % 4: the TMEM lane quarter this warp may read
    const int half = sw >> 2;
    const int col0 = half * 64;
    const int row = w4 * 32 + lane;
    const int q_pos = m_blk * kPM + row;
    const int limit = p.causal ? q_pos + offset : k_len - 1;  // last key this row may attend
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(w4 * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f, corr_prev = 1.f;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    bool ok = true;

    auto accumulate_o = [&](int j) -> bool {  // O = O * corr(j) + O_step(j), once the second MMA of step j has finished
      if (!__all_sync(0xffffffffu, mbar_wait(o_full, j & 1, abort_flag, timeout_ns))) return false;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_base + 2 * kPN + col0 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], corr_prev, __uint_as_float(r[i]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty);
      return true;
    };

    // Every softmax thread runs all n_steps iterations and meets its partner at the barrier of every step, also after
    // a pipeline wait has failed (then it skips the work and the waits): the barrier count stays the same for all.
    for (int j = 0; j < n_steps; ++j) {
      const int st = j & 1;
      if (ok) ok = mbar_wait(s_full + st, (j >> 1) & 1, abort_flag, timeout_ns);
      ok = __all_sync(0xffffffffu, ok);  // the TMEM loads below need the whole warp
      tc_fence_after_sync();
      const uint32_t s_addr = lane_base + st * kPN + col0;
      // keys of this thread's half below `visible` are unmasked for its row: only the diagonal and the last tile mask
      const int visible = min(limit + 1, k_len) - (j * kPN + col0);
      // ---- pass 1: maximum of this half of the row (raw scores; the positive scale is applied to the maximum once)
      float mx = -INFINITY;
      if (ok) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(s_addr + c * 32, r);
          tmem_ld_wait();
          if (visible >= (c + 1) * 32) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, c * 32 + i < visible ? __uint_as_float(r[i]) : -INFINITY);
          }
        }
      }
      xmax[(st * 2 + half) * kPM + row] = mx;   // double-buffered by step parity: the partner may run one step ahead
      softmax_bar();
      mx = fmaxf(mx, xmax[(st * 2 + (half ^ 1)) * kPM + row]);
      const float m_new = fmaxf(m_run, mx * p.scale_log2e);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float corr = fast_exp2(m_run - base);  // m_run == -inf -> 0
      // ---- the previous step's P V has finished (which also frees the P tile): fold it into the registers
      if (ok && j > 0) ok = accumulate_o(j - 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;
      // ---- pass 2: probabilities, row sum, P tile (A operand of the second MMA: K-major, 128-byte swizzle)
      float sum = 0.f;
      uint8_t* atom = sP + half * kPAtom + row * 128;   // keys [64 half, 64 half + 64) of the row are atom `half`
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // 16 keys at a time
        uint32_t r[16];
        tmem_ld_32x16(s_addr + c * 16, r);
        tmem_ld_wait();
        uint32_t packed[8];
        const bool all_visible = visible >= (c + 1) * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          // 2^(s * scale - base) as one fused multiply-add and one special-function instruction per score
          float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2e, -base));
          float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2e, -base));
          if (!all_visible) {
            p0 = c * 16 + i < visible ? p0 : 0.f;
            p1 = c * 16 + i + 1 < visible ? p1 : 0.f;
          }
          sum += p0 + p1;
          packed[i >> 1] = p.bf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int chunk = c * 2 + q;
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) * 16)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      tc_fence_before_sync();       // this thread's TMEM reads of S are done
      fence_view_async_shared();    // its P writes are visible to the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_empty + st);
        mbar_arrive(p_full);
      }
      l_run = l_run * corr + sum;   // this half's share of the row sum; both halves use the same maxima
      m_run = m_new;
      corr_prev = corr;
    }
    if (ok && n_steps > 0) ok = accumulate_o(n_steps - 1);
    // ---- total row sum = sum of the two halves, then normalise and store this half of the row
    xsum[half * kPM + row] = l_run;
    softmax_bar();
    l_run += xsum[(half ^ 1) * kPM + row];
    if (ok && q_pos < q_len) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint8_t* dst = static_cast<uint8_t*>(p.out) + ((static_cast<size_t>(q_start + q_pos) * p.Hq + h) * kPD + col0) * 2;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = o[c * 8 + i] * inv;
        uint4 v;
        if (p.bf16) v = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        else v = make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
        *reinterpret_cast<uint4*>(dst + c * 16) = v;
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && *abort_flag != 0u && p.status != nullptr) atomicMax(p.status, static_cast<uint32_t>(kStatusPipeTimeout));
}

}  // namespace b200

using namespace b200;

// Bytes of the transposed-V scratch that b200_prefill_attention needs: B * Hkv * 128 * s_pad elements of 2 bytes, where
// s_pad = max_k rounded up to 128.
B200_API long long b200_prefill_attention_scratch_bytes(int B, int Hkv, int max_k) {
  const long long s_pad = (static_cast<long long>(max_k) + 127) / 128 * 128;
  return static_cast<long long>(B) * Hkv * kPD * s_pad * 2;
}

// q [total_q, Hq, 128], k / v [total_k, Hkv, 128] (contiguous rows), cu_q / cu_k int32 [B + 1] on the device, out
// [total_q, Hq, 128]. Sequence b's keys are rows [cu_k[b], cu_k[b] + len) with len = k_lens[b], or cu_k[b + 1] - cu_k[b]
// when k_lens is null (packed sequences); with k_lens the key rows may sit anywhere in k / v, e.g. in the pages of a
// KV cache whose sequences own contiguous runs of slots. With causal != 0 query i of a sequence attends keys
// <= i + (k_len - q_len). vt_scratch: b200_prefill_attention_scratch_bytes(...) bytes, 16-byte aligned.
// dtype 0 = bf16, 1 = f16.
B200_API int b200_prefill_attention(const void* q, const void* k, const void* v, const int* cu_q, const int* cu_k,
                                    const int* k_lens, int B,
                                    int total_q, int total_k, int max_q, int max_k, int Hq, int Hkv, int head_dim,
                                    float scale, int causal, void* vt_scratch, void* out, int dtype, uint32_t* status,
                                    void* stream) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "prefill attention supports bf16/f16");
  B200_REQUIRE(head_dim == kPD, "prefill attention is specialised for head_dim 128, got %d", head_dim);
  B200_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "Hq (%d) must be a multiple of Hkv (%d)", Hq, Hkv);
  B200_REQUIRE(B >= 1 && max_q >= 1 && max_k >= 1 && total_q >= 1 && total_k >= 1, "empty problem");
  B200_REQUIRE(vt_scratch != nullptr, "the transposed-V scratch is required");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int s_pad = (max_k + 127) / 128 * 128;
  transpose_v_kernel<<<dim3(s_pad / 32, kPD / 32, B * Hkv), 256, 0, s>>>(static_cast<const uint16_t*>(v),
                                                                          static_cast<uint16_t*>(vt_scratch), cu_k, k_lens, Hkv, s_pad);
  B200_CHECK_CUDA(cudaGetLastError());
  CUtensorMap tq, tk, tv;
  int rc = make_tma_3d(&tq, q, dtype, kPD, Hq, total_q, kPD, static_cast<uint64_t>(Hq) * kPD, 64, 1, kPM, true);
  if (rc != kOk) return rc;
  rc = make_tma_3d(&tk, k, dtype, kPD, Hkv, total_k, kPD, static_cast<uint64_t>(Hkv) * kPD, 64, 1, kPN, true);
  if (rc != kOk) return rc;
  rc = make_tma_3d(&tv, vt_scratch, dtype, s_pad, kPD, static_cast<uint64_t>(B) * Hkv, s_pad,
                   static_cast<uint64_t>(kPD) * s_pad, 64, kPD, 1, true);
  if (rc != kOk) return rc;
  static bool configured[64] = {false};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmem));
    configured[dev & 63] = true;
  }
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.bf16 = dtype == kBF16;
  p.cu_q = cu_q; p.cu_k = cu_k; p.k_lens = k_lens;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.out = out; p.status = status;
  dim3 grid((max_q + kPM - 1) / kPM, Hq, B);
  prefill_attn_kernel<<<grid, kPThreads, kPSmem, s>>>(tq, tk, tv, p);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
