// Small-message all-gather in four flavours plus the micro-kernels that exercise the device
// primitives one by one.
//
// All-gather (python/triton_dist/kernels/nvidia/low_latency_allgather.py:47-777, 964-994): the
// buffer is symmetric, [world][bytes_per_rank], and slot `rank` is pre-filled by the caller.
//   PULL          barrier, copy every peer's slot out of the peer's buffer, barrier
//   PUSH          barrier, write the local slot into every peer's buffer, barrier
//   PUSH_LL       8-byte {data, flag} packets into a double-buffered packet area; the receiver polls the
//                 payload itself, so there is no barrier at all (latency = one NVLink store + one poll)
//   PUSH_LL_MC    as PUSH_LL but one multimem.st per packet reaches all ranks through the switch
// On an NVSwitch node every peer is one hop away, so the reference's 2D / 3D / NUMA variants reduce to
// PUSH and PUSH_LL.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

namespace b200 {

constexpr int kAgMaxCtas = 64;
constexpr int kAgThreads = 512;
enum AgMode : int { kAgPull = 0, kAgPush = 1, kAgPushLL = 2, kAgPushLLMc = 3 };

struct AgParams {
  uint8_t* buf;        // symmetric [world][bytes]
  uint64_t bytes;      // per rank, multiple of 16 (4 for the LL modes)
  uint64_t* ll[2];     // symmetric packet areas [world][bytes / 4] u64, one per epoch parity (LL modes)
  uint32_t* flags;     // symmetric u32[2][kAgMaxCtas][kMaxRanks]
  uint32_t* sync;      // local u32[4]
  int mode;
};

__device__ __forceinline__ bool ag_cta_barrier(const SymmCtx& c, uint32_t* flags, int phase, uint32_t epoch) {
  uint32_t* mine = flags + (static_cast<size_t>(phase) * kAgMaxCtas + blockIdx.x) * kMaxRanks;
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < c.world) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(c, mine + c.rank, threadIdx.x), epoch);
    ok = wait_flag<WaitCmp::GE, true>(c, mine + threadIdx.x, epoch, threadIdx.x, __LINE__);
  }
  return __syncthreads_and(ok);
}

__global__ void __launch_bounds__(kAgThreads) allgather_kernel(const AgParams p, const SymmCtx ctx) {
  const uint32_t epoch = epoch_begin(p.sync);
  const int world = ctx.world, me = ctx.rank;
  const uint64_t tid = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
  if (p.mode == kAgPull) {
    const uint64_t nvec = p.bytes / 16;
    bool ok = ag_cta_barrier(ctx, p.flags, 0, epoch);
    if (ok) {
      for (int k = 1; k < world; ++k) {
        const int peer = (me + k) % world;
        uint4* dst = reinterpret_cast<uint4*>(p.buf + peer * p.bytes);
        const uint4* src = symm_at(ctx, dst, peer);
        for (uint64_t i = tid; i < nvec; i += nthreads) st_v4(dst + i, ld_v4_relaxed_sys(src + i));
      }
      ag_cta_barrier(ctx, p.flags, 1, epoch);
    }
  } else if (p.mode == kAgPush) {
    // entry barrier: a peer enters this call only after whatever consumed its buffer since the previous call has
    // finished (stream order), so only then may its slots be overwritten
    const uint64_t nvec = p.bytes / 16;
    uint4* mine = reinterpret_cast<uint4*>(p.buf + me * p.bytes);
    if (ag_cta_barrier(ctx, p.flags, 0, epoch)) {
      for (uint64_t i = tid; i < nvec; i += nthreads) {
        const uint4 v = mine[i];
        for (int k = 1; k < world; ++k) st_v4(symm_at(ctx, mine + i, (me + k) % world), v);
      }
      ag_cta_barrier(ctx, p.flags, 1, epoch);
    }
  } else {
    // LL: word i of rank s travels as packet ll[s][i] = {word, epoch}
    const uint64_t nwords = p.bytes / 4;
    uint64_t* ll = p.ll[epoch & 1];
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.buf + me * p.bytes);
    for (uint64_t i = tid; i < nwords; i += nthreads) {
      const uint32_t w = mine[i];
      uint64_t* pkt = ll + me * nwords + i;
      if (p.mode == kAgPushLLMc) {
        const uint64_t v = (static_cast<uint64_t>(epoch) << 32) | w;
        asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_ptr(ctx, pkt)), "l"(v) : "memory");
      } else {
        for (int k = 1; k < world; ++k) ll_store(symm_at(ctx, pkt, (me + k) % world), w, epoch);
      }
    }
    bool ok = true;
    for (int k = 1; k < world && ok; ++k) {
      const int src = (me + k) % world;
      uint32_t* dst = reinterpret_cast<uint32_t*>(p.buf + src * p.bytes);
      for (uint64_t i = tid; i < nwords && ok; i += nthreads) {
        uint32_t w;
        ok = ll_load(ctx, ll + src * nwords + i, epoch, &w);
        if (ok) dst[i] = w;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// primitive micro-kernels (tests and tutorials)
// ---------------------------------------------------------------------------------------------
// Ring put with signal: every rank writes `n` words of `src` into `dst` of rank+1 and signals it;
// then waits for its own signal. (python/triton_dist/test/nvidia/test_ring_put.py, test_notify.py)
__global__ void ring_put_kernel(const SymmCtx ctx, const uint32_t* src, uint32_t* dst, uint32_t* sig, uint32_t n,
                                uint32_t value, uint32_t* ok_out) {
  const int next = (ctx.rank + 1) % ctx.world;
  putmem_signal_block(ctx, dst, src, static_cast<size_t>(n) * 4, sig, value, SigOp::SET, next);
  bool ok = true;
  if (threadIdx.x < 32) ok = wait(ctx, sig, 1, value, true);
  ok = __syncthreads_and(ok);
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
}

// Pull `n` words of `src` from rank-1 (after a barrier) into `dst`.
__global__ void ring_get_kernel(const SymmCtx ctx, const uint32_t* src, uint32_t* dst, uint32_t n, uint32_t* flags,
                                uint32_t epoch, uint32_t* ok_out) {
  bool ok = barrier_all_block(ctx, flags, epoch);
  const int prev = (ctx.rank + ctx.world - 1) % ctx.world;
  if (ok) getmem_block(ctx, dst, src, static_cast<size_t>(n) * 4, prev);
  ok = barrier_all_block(ctx, flags, epoch + 1) && ok;
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
}

// Waits on flags that nobody sets; with a short budget this returns an error status instead of hanging.
__global__ void wait_probe_kernel(const SymmCtx ctx, const uint32_t* flags, int n, uint32_t value, uint32_t* ok_out) {
  bool ok = true;
  if (threadIdx.x < 32) ok = wait(ctx, flags, n, value, true);
  ok = __syncthreads_and(ok);
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
}

// notify(add) from every rank into rank `root`, which waits for the sum.
__global__ void notify_add_kernel(const SymmCtx ctx, uint32_t* counter, int root, uint32_t expected, uint32_t* ok_out) {
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    notify<SigOp::ADD>(ctx, counter, root, 1u);
    bool ok = true;
    if (ctx.rank == root) ok = wait_flag<WaitCmp::GE, true>(ctx, counter, expected, 0, __LINE__);
    *ok_out = ok ? 1u : 0u;
  }
}

// Grid barrier exercised `rounds` times; every CTA adds its id to acc[round] before each barrier and
// checks the total after it.
__global__ void grid_barrier_kernel(const SymmCtx ctx, uint32_t* counter, uint32_t* acc, int rounds, uint32_t base,
                                    uint32_t* bad) {
  for (int r = 0; r < rounds; ++r) {
    if (threadIdx.x == 0) atomicAdd(acc + r, blockIdx.x + 1);
    if (!grid_barrier(ctx, counter, base + r + 1, gridDim.x)) { if (threadIdx.x == 0) atomicAdd(bad, 1u); return; }
    if (threadIdx.x == 0) {
      const uint32_t want = gridDim.x * (gridDim.x + 1) / 2;
      if (ld_relaxed_gpu(acc + r) != want) atomicAdd(bad, 1u);
    }
  }
}

// multimem round trip: every rank adds its vector into the multicast address, then reads the sum.
__global__ void multimem_probe_kernel(const SymmCtx ctx, float* buf, uint32_t n4, uint32_t* flags, uint32_t epoch,
                                      float* out, uint32_t* ok_out) {
  bool ok = barrier_all_block(ctx, flags, epoch);
  if (ok) {
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) {
      float4 v = multimem_ld_reduce_f32x4(mc_ptr(ctx, buf + 4 * i));
      reinterpret_cast<float4*>(out)[i] = v;
    }
  }
  ok = barrier_all_block(ctx, flags, epoch + 1) && ok;
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
}

// Collective micro-test of the SHMEM-style API. One CTA per rank. `bcast` [n4 * 4 floats], `coll` [world][n4 * 4 floats],
// `ring` [n4 * 4 floats], `sig` u32[2], `word` int32[world] and `flags` u32[2][world] are symmetric; `src` is local.
//   1. broadcast_block from `root`           -> bcast holds root's src on every rank
//   2. fcollect_warp (warp 0)                -> coll[r] holds rank r's src
//   3. putmem_signal_warp to rank + 1        -> ring holds rank - 1's src once sig[0] == epoch
//   4. int_p of (epoch + rank) into word[rank] of every rank, then barrier_all_warp
__global__ void shmem_api_probe_kernel(const SymmCtx ctx, const float* src, float* bcast, float* coll, float* ring,
                                       uint32_t* sig, int32_t* word, uint32_t* flags, uint32_t n4, int root,
                                       uint32_t epoch, uint32_t* ok_out) {
  const size_t nbytes = static_cast<size_t>(n4) * 16;
  bool ok = team_my_pe(ctx) == my_pe(ctx) && team_n_pes(ctx) == n_pes(ctx) && team_translate_pe(ctx, root) == root &&
            remote_ptr(ctx, bcast, ctx.rank) == bcast;
  broadcast_block(ctx, bcast, src, nbytes, root);
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    fcollect_warp(ctx, coll, src, nbytes);
  } else if (warp == 1) {
    putmem_signal_warp(ctx, ring, src, nbytes, sig, epoch, SigOp::SET, (ctx.rank + 1) % ctx.world);
  } else if (warp == 2 && lane_id() < static_cast<uint32_t>(ctx.world)) {
    int_p(ctx, word + ctx.rank, static_cast<int32_t>(epoch) + ctx.rank, lane_id());
  }
  // every put of this CTA is released by the barrier's fence + flag store; after it all ranks' data has landed
  ok = barrier_all_block(ctx, flags, epoch) && ok;
  if (warp == 3) ok = barrier_all_warp(ctx, flags + kMaxRanks, epoch) && ok;
  if (warp == 1 && lane_id() == 0) ok = signal_wait_until(ctx, sig, WaitCmp::EQ, epoch) && ok;
  ok = __syncthreads_and(ok);
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
}

}  // namespace b200

using namespace b200;

#define LOAD_CTX(name)       \
  SymmCtx name;              \
  memcpy(&name, symm_ctx, sizeof(name))

B200_API int b200_allgather(const void* symm_ctx, void* buf, uint64_t bytes_per_rank, void* ll0, void* ll1,
                            uint32_t* flags, uint32_t* sync, int mode, int num_ctas, void* stream) {
  LOAD_CTX(ctx);
  B200_REQUIRE(mode >= kAgPull && mode <= kAgPushLLMc, "unknown all-gather mode %d", mode);
  const bool ll = mode == kAgPushLL || mode == kAgPushLLMc;
  B200_REQUIRE(bytes_per_rank % (ll ? 4 : 16) == 0, "bytes per rank (%llu) must be a multiple of %d",
               (unsigned long long)bytes_per_rank, ll ? 4 : 16);
  B200_REQUIRE(!ll || (ll0 && ll1), "LL modes need the packet areas");
  B200_REQUIRE(mode != kAgPushLLMc || ctx.mc_base != 0, "multimem mode needs an NVLS multicast mapping");
  AgParams p;
  memset(&p, 0, sizeof(p));
  p.buf = static_cast<uint8_t*>(buf);
  p.bytes = bytes_per_rank;
  p.ll[0] = static_cast<uint64_t*>(ll0);
  p.ll[1] = static_cast<uint64_t*>(ll1);
  p.flags = flags;
  p.sync = sync;
  p.mode = mode;
  int grid = num_ctas > 0 ? num_ctas : 4;
  if (grid > kAgMaxCtas) grid = kAgMaxCtas;
  allgather_kernel<<<grid, kAgThreads, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
B200_API int b200_allgather_max_ctas() { return kAgMaxCtas; }

B200_API int b200_test_ring_put(const void* symm_ctx, const void* src, void* dst, void* sig, uint32_t n, uint32_t value,
                                void* ok_out, void* stream) {
  LOAD_CTX(ctx);
  ring_put_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(ctx, static_cast<const uint32_t*>(src),
                                                                   static_cast<uint32_t*>(dst), static_cast<uint32_t*>(sig),
                                                                   n, value, static_cast<uint32_t*>(ok_out));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
B200_API int b200_test_ring_get(const void* symm_ctx, const void* src, void* dst, uint32_t n, void* flags, uint32_t epoch,
                                void* ok_out, void* stream) {
  LOAD_CTX(ctx);
  ring_get_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(ctx, static_cast<const uint32_t*>(src),
                                                                   static_cast<uint32_t*>(dst), n,
                                                                   static_cast<uint32_t*>(flags), epoch,
                                                                   static_cast<uint32_t*>(ok_out));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
B200_API int b200_test_wait(const void* symm_ctx, const void* flags, int n, uint32_t value, void* ok_out, void* stream) {
  LOAD_CTX(ctx);
  B200_REQUIRE(n >= 1 && n <= 32, "wait takes 1..32 flags");
  wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(ctx, static_cast<const uint32_t*>(flags), n, value,
                                                                    static_cast<uint32_t*>(ok_out));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
// 1 when this library was compiled with B200_DEBUG_CHECKS (the checking build), else 0.
B200_API int b200_debug_checks() {
#ifdef B200_DEBUG_CHECKS
  return 1;
#else
  return 0;
#endif
}

B200_API int b200_test_notify_add(const void* symm_ctx, void* counter, int root, uint32_t expected, void* ok_out,
                                  void* stream) {
  LOAD_CTX(ctx);
  notify_add_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx, static_cast<uint32_t*>(counter), root, expected,
                                                                    static_cast<uint32_t*>(ok_out));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
// `base_round` = rounds completed on `counter` by earlier launches (which must have used the same `ctas`).
B200_API int b200_test_grid_barrier(const void* symm_ctx, void* counter, void* acc, int rounds, int ctas,
                                    uint32_t base_round, void* bad, void* stream) {
  LOAD_CTX(ctx);
  B200_REQUIRE(ctas >= 1 && ctas <= sm_count(), "grid barrier needs a co-resident grid (<= %d CTAs)", sm_count());
  B200_CHECK_CUDA(launch_cooperative(grid_barrier_kernel, dim3(ctas), dim3(128), 0, static_cast<cudaStream_t>(stream), ctx,
                                     static_cast<uint32_t*>(counter), static_cast<uint32_t*>(acc), rounds, base_round,
                                     static_cast<uint32_t*>(bad)));
  return kOk;
}
B200_API int b200_test_multimem(const void* symm_ctx, void* buf, uint32_t n4, void* flags, uint32_t epoch, void* out,
                                void* ok_out, void* stream) {
  LOAD_CTX(ctx);
  B200_REQUIRE(ctx.mc_base != 0, "no NVLS multicast mapping");
  multimem_probe_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(ctx, static_cast<float*>(buf), n4,
                                                                         static_cast<uint32_t*>(flags), epoch,
                                                                         static_cast<float*>(out),
                                                                         static_cast<uint32_t*>(ok_out));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

B200_API int b200_test_shmem_api(const void* symm_ctx, const void* src, void* bcast, void* coll, void* ring, void* sig,
                                 void* word, void* flags, uint32_t n4, int root, uint32_t epoch, void* ok_out, void* stream) {
  LOAD_CTX(ctx);
  B200_REQUIRE(root >= 0 && root < ctx.world, "root (%d) out of range", root);
  shmem_api_probe_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ctx, static_cast<const float*>(src), static_cast<float*>(bcast), static_cast<float*>(coll), static_cast<float*>(ring),
      static_cast<uint32_t*>(sig), static_cast<int32_t*>(word), static_cast<uint32_t*>(flags), n4, root, epoch,
      static_cast<uint32_t*>(ok_out));
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

// ---------------------------------------------------------------------------------------------
// Stand-alone reduce-scatter: out[M / world, N] = rows of this rank of sum_r in_r[M, N].
// CTA b of every rank pushes its share of each owner's rows into the owner's slot [src][row], meets CTA b of
// the peers, then sums the slots of its own rows in fp32 (fixed order, so results are reproducible).
// (python/triton_dist/kernels/nvidia/reduce_scatter.py:597-882: scatter by copy engine + ring_reduce kernel.)
// ---------------------------------------------------------------------------------------------
namespace b200 {
struct RsParams {
  const uint4* in;     // [world * per_rank_vecs]
  uint4* out;          // [per_rank_vecs]
  uint4* ws[2];        // symmetric [world][per_rank_vecs]
  uint64_t per_rank_vecs;
  uint32_t* flags;     // symmetric u32[2][kAgMaxCtas][kMaxRanks]
  uint32_t* sync;
  int bf16;            // 1 bf16, 0 f16, 2 f32
};
__device__ __forceinline__ void rs_acc(float* acc, uint4 v, int kind) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if (kind == 2) {
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[q] += __uint_as_float(w[q]);
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = kind == 1 ? unpack_bf16x2(w[q]) : unpack_f16x2(w[q]);
      acc[2 * q] += f.x;
      acc[2 * q + 1] += f.y;
    }
  }
}
__global__ void __launch_bounds__(kAgThreads) reduce_scatter_kernel(const RsParams p, const SymmCtx ctx) {
  const uint32_t epoch = epoch_begin(p.sync);
  uint4* ws = p.ws[epoch & 1];
  const uint64_t tid = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x, nthreads = (uint64_t)gridDim.x * blockDim.x;
  for (int k = 0; k < ctx.world; ++k) {
    const int owner = (ctx.rank + 1 + k) % ctx.world;
    for (uint64_t i = tid; i < p.per_rank_vecs; i += nthreads)
      st_v4(symm_at(ctx, ws + ctx.rank * p.per_rank_vecs + i, owner), p.in[owner * p.per_rank_vecs + i]);
  }
  if (ag_cta_barrier(ctx, p.flags, 0, epoch)) {
    for (uint64_t i = tid; i < p.per_rank_vecs; i += nthreads) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int s = 0; s < ctx.world; ++s) rs_acc(acc, ld_v4_relaxed_sys(ws + s * p.per_rank_vecs + i), p.bf16);
      uint4 o;
      if (p.bf16 == 2) o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
      else if (p.bf16 == 1) o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      else o = make_uint4(pack_f16x2(acc[0], acc[1]), pack_f16x2(acc[2], acc[3]), pack_f16x2(acc[4], acc[5]), pack_f16x2(acc[6], acc[7]));
      p.out[i] = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) epoch_end(p.sync, p.sync + 1, epoch, gridDim.x);
}
}  // namespace b200

// in: [world * bytes_per_rank] (rows of owner r at r * bytes_per_rank); out: [bytes_per_rank]; ws0 / ws1: symmetric
// [world * bytes_per_rank]; dtype 0 bf16, 1 f16, 2 f32.
B200_API int b200_reduce_scatter(const void* symm_ctx, const void* in, void* out, uint64_t bytes_per_rank, int dtype, void* ws0,
                                 void* ws1, uint32_t* flags, uint32_t* sync, int num_ctas, void* stream) {
  LOAD_CTX(ctx);
  B200_REQUIRE(bytes_per_rank % 16 == 0, "bytes per rank (%llu) must be a multiple of 16", (unsigned long long)bytes_per_rank);
  B200_REQUIRE(dtype == kBF16 || dtype == kF16 || dtype == kF32, "reduce_scatter supports bf16/f16/f32");
  RsParams p;
  memset(&p, 0, sizeof(p));
  p.in = static_cast<const uint4*>(in); p.out = static_cast<uint4*>(out);
  p.ws[0] = static_cast<uint4*>(ws0); p.ws[1] = static_cast<uint4*>(ws1);
  p.per_rank_vecs = bytes_per_rank / 16; p.flags = flags; p.sync = sync;
  p.bf16 = dtype == kBF16 ? 1 : (dtype == kF16 ? 0 : 2);
  int grid = num_ctas > 0 ? num_ctas : 8;
  if (grid > kAgMaxCtas) grid = kAgMaxCtas;
  reduce_scatter_kernel<<<grid, kAgThreads, 0, static_cast<cudaStream_t>(stream)>>>(p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
