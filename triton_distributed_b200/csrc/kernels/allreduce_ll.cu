// Low-latency fused all-reduce + residual + RMSNorm for decode-sized inputs (a few rows of a few thousand channels).
//
// The one-shot all-reduce of allreduce.cu pushes the data, fences, exchanges flags and only then reads the slots: two
// dependent NVLink traversals plus a system-scope fence per call. Here every 32-bit word (two 16-bit elements) travels
// in an 8-byte packet {word, epoch}: a single aligned 8-byte store is delivered atomically, so the receiver can poll
// the payload itself and the flag exchange, the fence and the barrier disappear (the LL protocol of
// python/triton_dist/kernels/nvidia/low_latency_allgather.py:530-566 applied to the reduction). Packets are written
// into slot [source rank] of every peer's workspace; the workspace is double-buffered by the parity of the
// device-resident epoch, and the epoch is the flag value, so nothing is ever reset.
//
// One CTA of 1024 threads owns a row: it sends the row, gathers the `world` contributions of every word (all loads
// of a word issued together, summed in rank order in fp32), adds the residual, rounds to the storage type, and
// normalises. Arithmetic and rounding are those of the fused path in allreduce.cu (finish_row), so both give the
// same numbers. It serves fused calls of at most 512 KB (B200DIST_AR_LL=0 sends them to allreduce.cu instead). With an
// NVLS multicast mapping one multimem.st per packet reaches every rank through the switch, so a rank injects its row
// once instead of world - 1 times.
//
// Role in the reference: the GEMM + AllReduce decode path (layers/nvidia/tp_mlp.py:177-191, tp_attn.py:240-271), whose
// all-reduce is kernels/nvidia/allreduce.py:364-414 followed by a separate flashinfer RMSNorm.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

namespace b200 {

constexpr int kLLThreads = 1024;
constexpr int kLLMaxCtas = 256;       // copies of the call counter (the grid never exceeds the SM count)
constexpr int kLLWordsPerThread = 4;  // a row has at most 4096 words: hidden <= 8192 for 16-bit types

struct ArLLParams {
  const uint32_t* in;          // [rows, hidden / 2] words of this rank's partial result
  uint64_t* ws[2];             // symmetric, per parity: [world][rows][hidden / 2] packets
  uint32_t* sync;              // local u32[256]: one copy of the call counter per CTA
  int rows, hidden, bf16, use_mc;
  const uint32_t* residual_in; // [rows, hidden / 2] or null
  uint32_t* residual_out;      // [rows, hidden / 2] or null
  const uint32_t* gamma;       // [hidden / 2]
  uint32_t* normed_out;        // [rows, hidden / 2]
  float eps;
};

__device__ __forceinline__ float2 ll_unpack(uint32_t w, bool bf16) { return bf16 ? unpack_bf16x2(w) : unpack_f16x2(w); }
__device__ __forceinline__ uint32_t ll_pack(float a, float b, bool bf16) { return bf16 ? pack_bf16x2(a, b) : pack_f16x2(a, b); }

__global__ void __launch_bounds__(kLLThreads) allreduce_ll_kernel(const ArLLParams p, const SymmCtx ctx) {
  __shared__ float red[33];
  griddep_launch_dependents();
  const int world = ctx.world, me = ctx.rank;
  const int row_words = p.hidden / 2;
  const bool bf16 = p.bf16 != 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the gain is a weight (never an output of the kernel launched just before this one): fetched before the dependency
  // wait, past L1, so that it costs no round trip after the sum
  uint32_t gw[kLLWordsPerThread];
#pragma unroll
  for (int u = 0; u < kLLWordsPerThread; ++u) {
    const int i = tid + u * kLLThreads;
    gw[u] = i < row_words ? __ldcg(p.gamma + i) : 0u;
  }
  griddep_wait();
  // Every CTA keeps its own copy of the call counter (sync[blockIdx.x]) and advances it with one plain store when it
  // leaves; CTA 0 also advances the copies of the CTAs that this launch does not have, so all copies stay equal from
  // call to call whatever the grid sizes. Compared with one shared word that the last CTA to leave advances (a fence, an
  // atomic and a second fence per CTA), this takes ~1.3 us off the end of the kernel, which the next kernel of a
  // dependent-launch chain waits for.
  const uint32_t epoch = ld_relaxed_gpu(p.sync + blockIdx.x) + 1u;
  const int par = epoch & 1;
  uint64_t* ws = p.ws[par];
  bool ok = true;

  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    // ---- send: my word goes into slot [me] of every rank (my own copy is taken from the register below)
    // all of the row's loads (partial result and residual) are issued before the first packet leaves, so that the
    // residual's round trip overlaps the exchange instead of following every poll
    uint32_t mine[kLLWordsPerThread], resw[kLLWordsPerThread];
#pragma unroll
    for (int u = 0; u < kLLWordsPerThread; ++u) {
      const int i = tid + u * kLLThreads;
      mine[u] = resw[u] = 0u;
      if (i < row_words) {
        mine[u] = p.in[static_cast<size_t>(row) * row_words + i];
        if (p.residual_in) resw[u] = p.residual_in[static_cast<size_t>(row) * row_words + i];
      }
    }
#pragma unroll
    for (int u = 0; u < kLLWordsPerThread; ++u) {
      const int i = tid + u * kLLThreads;
      if (i < row_words) {
        const uint32_t d = mine[u];
        uint64_t* slot = ws + (static_cast<size_t>(me) * p.rows + row) * row_words + i;
        if (p.use_mc) {
          const uint64_t v = (static_cast<uint64_t>(epoch) << 32) | d;
          asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_ptr(ctx, slot)), "l"(v) : "memory");
        } else {
          for (int k = 1; k < world; ++k) {
            int peer = me + k;
            if (peer >= world) peer -= world;
            ll_store(symm_at(ctx, slot, peer), d, epoch);
          }
        }
      }
    }
    // ---- gather, sum in rank order, add the residual, round to the storage type
    float x[kLLWordsPerThread][2];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kLLWordsPerThread; ++u) {
      const int i = tid + u * kLLThreads;
      x[u][0] = x[u][1] = 0.f;
      if (i < row_words) {
        uint64_t v[kMaxRanks];
        uint32_t pending = ((1u << world) - 1u) & ~(1u << me);
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (pending != 0u && ok) {
#pragma unroll
          for (int s = 0; s < kMaxRanks; ++s)
            if ((pending >> s) & 1u) {
              const uint64_t* src = ws + (static_cast<size_t>(s) * p.rows + row) * row_words + i;
              asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v[s]) : "l"(src) : "memory");
            }
#pragma unroll
          for (int s = 0; s < kMaxRanks; ++s)
            if (((pending >> s) & 1u) && static_cast<uint32_t>(v[s] >> 32) == epoch) pending &= ~(1u << s);
          if (pending != 0u && ++spins > 4u) __nanosleep(40);
          if (pending != 0u && (spins & 31u) == 0u) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > ctx.timeout_ns) {
              report_status(ctx, kStatusWaitTimeout, __ffs(pending) - 1, epoch, 0, __LINE__);
              ok = false;
            } else if (status_is_error(ctx)) {
              ok = false;
            }
          }
        }
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s)
          if (s < world) {
            const float2 f = ll_unpack(s == me ? mine[u] : static_cast<uint32_t>(v[s]), bf16);
            a0 += f.x;
            a1 += f.y;
          }
        if (p.residual_in) {
          const float2 r = ll_unpack(resw[u], bf16);
          a0 += r.x;
          a1 += r.y;
        }
        const float2 q = ll_unpack(ll_pack(a0, a1, bf16), bf16);  // the residual stream is kept in the storage type
        x[u][0] = q.x;
        x[u][1] = q.y;
        ss += q.x * q.x + q.y * q.y;
      }
    }
    // ---- row-wide sum of squares (every thread takes part, also after a timeout)
    ss = warp_sum(ss);
    __syncthreads();
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
      float t = red[lane];
      t = warp_sum(t);
      if (lane == 0) red[32] = t;
    }
    __syncthreads();
    const float inv = rsqrtf(red[32] / static_cast<float>(p.hidden) + p.eps);
#pragma unroll
    for (int u = 0; u < kLLWordsPerThread; ++u) {
      const int i = tid + u * kLLThreads;
      if (i < row_words && ok) {
        const float2 g = ll_unpack(gw[u], bf16);
        const size_t o = static_cast<size_t>(row) * row_words + i;
        if (p.residual_out) p.residual_out[o] = ll_pack(x[u][0], x[u][1], bf16);
        p.normed_out[o] = ll_pack(x[u][0] * inv * g.x, x[u][1] * inv * g.y, bf16);
      }
    }
  }
  __syncthreads();  // every thread of the CTA is done with the packets of this call
  if (threadIdx.x == 0) p.sync[blockIdx.x] = epoch;
  if (blockIdx.x == 0)
    for (int i = gridDim.x + threadIdx.x; i < kLLMaxCtas; i += blockDim.x) p.sync[i] = epoch;
}

}  // namespace b200

using namespace b200;

// Bytes of symmetric workspace per parity buffer that a call of this shape needs.
B200_API long long b200_allreduce_ll_ws_bytes(int world, int rows, int hidden) {
  return static_cast<long long>(world) * rows * (hidden / 2) * 8;
}

// in / residual / normed_out: [rows, hidden] of bf16 (dtype 0) or f16 (1), 4-byte aligned rows (hidden even).
// ws0 / ws1: symmetric parity buffers of b200_allreduce_ll_ws_bytes each, zero-initialised once; sync: local u32[256],
// zero-initialised once and used by LL calls only (its epoch is the packet flag). residual_in / residual_out may be
// null and may alias each other. use_multimem != 0 broadcasts packets with multimem.st (needs the NVLS mapping).
B200_API int b200_allreduce_ll(const void* symm_ctx, const void* in, int rows, int hidden, int dtype, void* ws0, void* ws1,
                               uint32_t* sync, const void* residual_in, void* residual_out, const void* gamma,
                               void* normed_out, float eps, int use_multimem, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "the LL all-reduce handles bf16 and f16");
  B200_REQUIRE(rows >= 1 && hidden >= 2 && hidden % 2 == 0, "bad shape %d x %d", rows, hidden);
  B200_REQUIRE(hidden / 2 <= kLLThreads * kLLWordsPerThread, "hidden (%d) exceeds %d", hidden, 2 * kLLThreads * kLLWordsPerThread);
  B200_REQUIRE(ctx.world >= 1 && ctx.world <= kMaxRanks, "world (%d) out of range", ctx.world);
  B200_REQUIRE(in && ws0 && ws1 && sync && gamma && normed_out, "missing buffers");
  B200_REQUIRE(!use_multimem || ctx.mc_base != 0, "multimem packets need an NVLS multicast mapping");
  ArLLParams p;
  memset(&p, 0, sizeof(p));
  p.in = static_cast<const uint32_t*>(in);
  p.ws[0] = static_cast<uint64_t*>(ws0);
  p.ws[1] = static_cast<uint64_t*>(ws1);
  p.sync = sync;
  p.rows = rows; p.hidden = hidden; p.bf16 = dtype == kBF16; p.use_mc = use_multimem && ctx.world > 1;
  p.residual_in = static_cast<const uint32_t*>(residual_in);
  p.residual_out = static_cast<uint32_t*>(residual_out);
  p.gamma = static_cast<const uint32_t*>(gamma);
  p.normed_out = static_cast<uint32_t*>(normed_out);
  p.eps = eps;
  int grid = rows < sm_count() ? rows : sm_count();
  if (grid > kLLMaxCtas) grid = kLLMaxCtas;
  B200_CHECK_CUDA(launch_pdl(allreduce_ll_kernel, dim3(grid), dim3(kLLThreads), 0, static_cast<cudaStream_t>(stream), p, ctx));
  return kOk;
}
