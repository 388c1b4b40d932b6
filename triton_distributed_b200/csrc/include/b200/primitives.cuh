// Device-side distributed primitives for sm_100a.
//
// These functions are the CUDA restatement of the reference's device language:
//   wait / notify / symm_at / rank / num_ranks
//     (python/triton_dist/language/distributed_ops.py:57-111, lowered in
//      lib/Conversion/TritonDistributedToLLVM/NVIDIA/DistributedOpToLLVM.cpp:146-423)
//   putmem / getmem / putmem_signal / signal_op / signal_wait_until / fence / quiet / barrier_all
//     (shmem/nvshmem_bind/runtime/nvshmem_wrapper.cu:26-695)
//   ld/st with scope+semantic, atomics, multimem ld_reduce/st/red
//     (backends/nvidia/language/cuda/language_extra.py:108-797)
//   grid barrier and intra-node barrier_all
//     (python/triton_dist/kernels/nvidia/common_ops.py:57-206)
//
// Differences by design:
//   * peers are reached through a per-rank base table of a CUDA VMM (or IPC) symmetric heap,
//     so symm_at is pointer arithmetic on a by-value context instead of a device-state load;
//   * every spin is bounded by a %globaltimer budget; on expiry the waiter records
//     {code, who, expected, seen} in the status block of the heap and returns false, so a
//     lost signal ends the kernel with an error that the host raises instead of a hung GPU;
//   * flags are monotone epochs (never reset), which removes the reset + double barrier
//     that the reference brackets its flag arrays with.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace b200 {

constexpr int kMaxRanks = 8;

// Error codes written to SymmCtx::status[0].
enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,     // a flag / signal wait ran out of budget
  kStatusBarrierTimeout = 2,  // a cross-rank or grid barrier ran out of budget
  kStatusPipeTimeout = 3,     // an intra-kernel mbarrier pipeline wait ran out of budget
  kStatusBadArgument = 4,
};

// By-value kernel argument describing the symmetric heap as seen from this rank.
struct SymmCtx {
  int32_t rank;
  int32_t world;
  uint64_t heap_base[kMaxRanks];  // VA (in this process) of rank k's heap
  uint64_t mc_base;               // NVLS multicast VA of the heap, 0 when unavailable
  uint64_t heap_bytes;
  uint32_t* status;               // 16 x u32, local: [0]=code [1]=who [2]=expected [3]=seen [4]=line
  uint64_t timeout_ns;            // budget of every bounded wait
};

// ----------------------------------------------------------------------------------------------
// rank / num_ranks / symm_at / mc_ptr
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ int rank(const SymmCtx& c) { return c.rank; }
__device__ __forceinline__ int num_ranks(const SymmCtx& c) { return c.world; }

// Checking build (`python -m triton_distributed_b200.build --debug` -> lib/libb200dist_debug.so, loaded when
// B200DIST_DEBUG_LIB=1): compiled with B200_DEBUG_CHECKS, every translation of a symmetric address verifies that the
// pointer lies inside this rank's heap and that the peer exists. A violation is recorded in the status block
// (bad argument: who = peer, expected = low word of the heap size, seen = low word of the offset) and the translation
// falls back to the local address, so the access stays inside this GPU's own memory instead of faulting a peer.
// notify / signal / wait / barrier entry points also sleep for a pseudo-random time of up to ~2 us first, which
// widens the windows in which a missing fence, an early flag or a reused buffer would show up in the multi-rank cases.
__device__ __forceinline__ void report_status(const SymmCtx& c, uint32_t code, uint32_t who, uint32_t expected,
                                              uint32_t seen, uint32_t line);
#ifdef B200_DEBUG_CHECKS
__device__ __forceinline__ bool debug_symm_ok(const SymmCtx& c, uint64_t off, int peer, uint32_t line) {
  if (off < c.heap_bytes && peer >= 0 && peer < c.world) return true;
  report_status(c, kStatusBadArgument, static_cast<uint32_t>(peer), static_cast<uint32_t>(c.heap_bytes),
                static_cast<uint32_t>(off), line);
  return false;
}
__device__ __forceinline__ void debug_jitter() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const uint32_t h = (static_cast<uint32_t>(t) ^ (threadIdx.x * 2654435761u) ^ (blockIdx.x * 40503u)) * 2246822519u;
  __nanosleep((h >> 21) & 2047u);
}
#else
__device__ __forceinline__ void debug_jitter() {}
#endif

// Translate a pointer into this rank's heap to the same offset of `peer`'s heap.
template <typename T>
__device__ __forceinline__ T* symm_at(const SymmCtx& c, T* local_ptr, int peer) {
  uint64_t off = reinterpret_cast<uint64_t>(local_ptr) - c.heap_base[c.rank];
#ifdef B200_DEBUG_CHECKS
  if (!debug_symm_ok(c, off, peer, __LINE__)) return local_ptr;
#endif
  return reinterpret_cast<T*>(c.heap_base[peer] + off);
}

// Multicast alias of a local symmetric pointer (stores reach every rank, ld_reduce sums over ranks).
template <typename T>
__device__ __forceinline__ T* mc_ptr(const SymmCtx& c, T* local_ptr) {
  uint64_t off = reinterpret_cast<uint64_t>(local_ptr) - c.heap_base[c.rank];
#ifdef B200_DEBUG_CHECKS
  if (c.mc_base == 0 || !debug_symm_ok(c, off, c.rank, __LINE__)) return local_ptr;
#endif
  return reinterpret_cast<T*>(c.mc_base + off);
}

// ----------------------------------------------------------------------------------------------
// thread / lane helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lane_id() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int flat_tid() {
  return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
}

// Programmatic dependent launch. griddep_launch_dependents(): the next kernel of the stream may be scheduled once
// every CTA of this grid has said so (or exited). griddep_wait(): block until the kernels this one depends on have
// completed and their memory operations are visible; call it before touching anything they produce or still read.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ----------------------------------------------------------------------------------------------
// scoped loads / stores / atomics on 32- and 64-bit words
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_release_sys(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.add.release.sys.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_add_acqrel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_cas_acqrel_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.cas.acq_rel.sys.global.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// Orders generic-proxy accesses with later async-proxy (TMA / tcgen05) accesses of the same memory.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// 16-byte vector accesses. The .relaxed.sys forms bypass L1 so data that a peer (or the switch)
// rewrote since the last call is never served from a stale line.
__device__ __forceinline__ uint4 ld_v4_relaxed_sys(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_v4_nc(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_v4_relaxed_sys(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w) : "memory");
}

// ----------------------------------------------------------------------------------------------
// NVLS multimem (pointers must come from mc_ptr)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st_u32(void* mc, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_add_u32(void* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_add_bf16x2(void* mc, uint32_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.bf16x2 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// ----------------------------------------------------------------------------------------------
// status block + bounded waits
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void report_status(const SymmCtx& c, uint32_t code, uint32_t who, uint32_t expected,
                                              uint32_t seen, uint32_t line) {
  if (c.status == nullptr) return;
  if (atomicCAS(c.status, 0u, code) == 0u) {
    c.status[1] = who;
    c.status[2] = expected;
    c.status[3] = seen;
    c.status[4] = line;
    __threadfence_system();
  }
}
__device__ __forceinline__ bool status_is_error(const SymmCtx& c) {
  return c.status != nullptr && ld_relaxed_gpu(c.status) != 0u;
}

enum class WaitCmp { EQ, GE };

// Spin on one flag until it compares true against `value` or the budget runs out. Returns false
// after recording a timeout, or as soon as another waiter of this rank has recorded one.
template <WaitCmp CMP = WaitCmp::GE, bool SYS = true>
__device__ __forceinline__ bool wait_flag(const SymmCtx& c, const uint32_t* flag, uint32_t value,
                                          uint32_t who = 0, uint32_t line = 0) {
  debug_jitter();
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t seen = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    bool ok = (CMP == WaitCmp::EQ) ? (seen == value) : (static_cast<int32_t>(seen - value) >= 0);
    if (ok) return true;
    // back off once the flag is clearly not about to flip: thousands of threads polling one line would otherwise
    // saturate its L2 slice and delay the very stores and atomics that the waiters are waiting for
    if (++spins > 8u) __nanosleep(spins > 64u ? 256u : 64u);
    if ((spins & 63u) == 0u) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > c.timeout_ns) {
        report_status(c, kStatusWaitTimeout, who, value, seen, line);
        return false;
      }
      if (status_is_error(c)) return false;
    }
  }
}

// `wait` of the reference: lane l < n spins on flags[l] until it equals `value` (acquire), then the
// warp reconverges. Every lane returns the warp-wide verdict. n <= 32.
__device__ __forceinline__ bool wait(const SymmCtx& c, const uint32_t* flags, int n, uint32_t value,
                                     bool sys_scope = true) {
  bool ok = true;
  int l = lane_id();
  if (l < n) {
    ok = sys_scope ? wait_flag<WaitCmp::EQ, true>(c, flags + l, value, l, __LINE__)
                   : wait_flag<WaitCmp::EQ, false>(c, flags + l, value, l, __LINE__);
  }
  return __all_sync(0xffffffffu, ok);
}
// The token of the reference only creates a data dependence; in CUDA program order after wait() is enough.
template <typename T>
__device__ __forceinline__ T consume_token(T v, bool /*token*/) { return v; }

enum class SigOp { SET, ADD };

// `notify` of the reference: called by ONE thread after the CTA's data stores were made visible to it
// (e.g. behind __syncthreads()); releases them at system scope and updates `peer`'s copy of the flag.
template <SigOp OP = SigOp::SET>
__device__ __forceinline__ void notify(const SymmCtx& c, uint32_t* local_flag, int peer, uint32_t value) {
  debug_jitter();
  uint32_t* dst = symm_at(c, local_flag, peer);
  if (OP == SigOp::SET) {
    st_release_sys(dst, value);
  } else {
    red_add_release_sys(dst, value);
  }
}
__device__ __forceinline__ void signal_op(const SymmCtx& c, uint32_t* local_flag, uint32_t value, SigOp op, int peer) {
  if (op == SigOp::SET) notify<SigOp::SET>(c, local_flag, peer, value);
  else notify<SigOp::ADD>(c, local_flag, peer, value);
}
__device__ __forceinline__ bool signal_wait_until(const SymmCtx& c, const uint32_t* flag, WaitCmp cmp, uint32_t value) {
  return cmp == WaitCmp::EQ ? wait_flag<WaitCmp::EQ, true>(c, flag, value, 0, __LINE__)
                            : wait_flag<WaitCmp::GE, true>(c, flag, value, 0, __LINE__);
}
__device__ __forceinline__ void fence() { fence_acq_rel_sys(); }
// All of this rank's earlier stores are performed by plain st/red instructions, so completion at
// system scope is what a fence provides; there is no separate NIC queue to drain.
__device__ __forceinline__ void quiet() { fence_acq_rel_sys(); }

// ----------------------------------------------------------------------------------------------
// putmem / getmem: 16-byte vectorised P2P copies. `nbytes`, `dst` and `src` must be 16-byte
// aligned for the vector path; a byte tail loop covers the rest.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void copy_bytes_strided(void* dst, const void* src, size_t nbytes, int tid, int nthreads) {
  size_t nvec = nbytes / 16;
  bool aligned = ((reinterpret_cast<uint64_t>(dst) | reinterpret_cast<uint64_t>(src)) & 15u) == 0;
  if (aligned) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    size_t i = tid;
    // four independent 16-byte loads in flight per thread
    for (; i + 3 * (size_t)nthreads < nvec; i += 4 * (size_t)nthreads) {
      uint4 a = ld_v4_relaxed_sys(s + i);
      uint4 b = ld_v4_relaxed_sys(s + i + nthreads);
      uint4 e = ld_v4_relaxed_sys(s + i + 2 * (size_t)nthreads);
      uint4 f = ld_v4_relaxed_sys(s + i + 3 * (size_t)nthreads);
      st_v4(d + i, a);
      st_v4(d + i + nthreads, b);
      st_v4(d + i + 2 * (size_t)nthreads, e);
      st_v4(d + i + 3 * (size_t)nthreads, f);
    }
    for (; i < nvec; i += nthreads) st_v4(d + i, ld_v4_relaxed_sys(s + i));
    for (size_t b = nvec * 16 + tid; b < nbytes; b += nthreads)
      reinterpret_cast<uint8_t*>(dst)[b] = reinterpret_cast<const volatile uint8_t*>(src)[b];
  } else {
    for (size_t b = tid; b < nbytes; b += nthreads)
      reinterpret_cast<uint8_t*>(dst)[b] = reinterpret_cast<const volatile uint8_t*>(src)[b];
  }
}
// dst is a LOCAL symmetric address; the data lands at the same offset on `peer`.
__device__ __forceinline__ void putmem_block(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int peer) {
  copy_bytes_strided(symm_at(c, reinterpret_cast<uint8_t*>(dst_local), peer), src, nbytes, flat_tid(),
                     blockDim.x * blockDim.y * blockDim.z);
}
__device__ __forceinline__ void putmem_warp(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int peer) {
  copy_bytes_strided(symm_at(c, reinterpret_cast<uint8_t*>(dst_local), peer), src, nbytes, lane_id(), 32);
}
__device__ __forceinline__ void putmem(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int peer) {
  copy_bytes_strided(symm_at(c, reinterpret_cast<uint8_t*>(dst_local), peer), src, nbytes, 0, 1);
}
// src is a LOCAL symmetric address whose counterpart on `peer` is read.
__device__ __forceinline__ void getmem_block(const SymmCtx& c, void* dst, const void* src_local, size_t nbytes, int peer) {
  copy_bytes_strided(dst, symm_at(c, reinterpret_cast<const uint8_t*>(src_local), peer), nbytes, flat_tid(),
                     blockDim.x * blockDim.y * blockDim.z);
}
__device__ __forceinline__ void getmem_warp(const SymmCtx& c, void* dst, const void* src_local, size_t nbytes, int peer) {
  copy_bytes_strided(dst, symm_at(c, reinterpret_cast<const uint8_t*>(src_local), peer), nbytes, lane_id(), 32);
}
// putmem_signal_block: copy by the whole CTA, then one thread releases the data and signals the peer.
__device__ __forceinline__ void putmem_signal_block(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes,
                                                    uint32_t* sig_local, uint32_t sig_value, SigOp op, int peer) {
  putmem_block(c, dst_local, src, nbytes, peer);
  __syncthreads();
  if (flat_tid() == 0) {
    fence_acq_rel_sys();
    signal_op(c, sig_local, sig_value, op, peer);
  }
}

// ----------------------------------------------------------------------------------------------
// barriers
// ----------------------------------------------------------------------------------------------
// Cross-rank barrier executed by ONE CTA per rank. `flags` is a symmetric u32[world] array and
// `epoch` the value of this round (strictly increasing from call to call, same on every rank).
// Thread k < world publishes epoch into flags[rank] on peer k, then waits for flags[k] locally.
__device__ __forceinline__ bool barrier_all_block(const SymmCtx& c, uint32_t* flags, uint32_t epoch) {
  debug_jitter();
  __syncthreads();
  int t = flat_tid();
  bool ok = true;
  if (t < c.world) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(c, flags + c.rank, t), epoch);
    ok = wait_flag<WaitCmp::GE, true>(c, flags + t, epoch, t, __LINE__);
    if (!ok) report_status(c, kStatusBarrierTimeout, t, epoch, 0, __LINE__);
  }
  return __syncthreads_and(ok);
}

// Grid-wide barrier for grids whose CTAs are all resident (persistent / cooperative launches).
// `counter` is a local u32 that only ever grows: round r completes when it reaches r * num_ctas.
__device__ __forceinline__ bool grid_barrier(const SymmCtx& c, uint32_t* counter, uint32_t round, uint32_t num_ctas) {
  __syncthreads();
  bool ok = true;
  if (flat_tid() == 0) {
    __threadfence();
    atom_add_acqrel_gpu(counter, 1u);
    ok = wait_flag<WaitCmp::GE, false>(c, counter, round * num_ctas, blockIdx.x, __LINE__);
    if (!ok) report_status(c, kStatusBarrierTimeout, blockIdx.x, round * num_ctas, 0, __LINE__);
  }
  return __syncthreads_and(ok);
}

// Device-resident epoch: every CTA reads `*epoch_ptr + 1` on entry; the last CTA to leave stores it
// back. Host code never passes a call counter, so a captured CUDA graph can be replayed.
__device__ __forceinline__ uint32_t epoch_begin(const uint32_t* epoch_ptr) { return ld_relaxed_gpu(epoch_ptr) + 1u; }
// Called by one thread per CTA after all of the CTA's work is done.
__device__ __forceinline__ void epoch_end(uint32_t* epoch_ptr, uint32_t* done_counter, uint32_t epoch, uint32_t num_ctas) {
  __threadfence();
  if (atomicAdd(done_counter, 1u) == num_ctas - 1u) {
    *done_counter = 0u;
    __threadfence();
    *epoch_ptr = epoch;
  }
}

// ----------------------------------------------------------------------------------------------
// Remainder of the SHMEM-style device API (shmem/nvshmem_bind/runtime/nvshmem_wrapper.cu:26-695,
// python/triton_dist/language/extra/libshmem_device.py:28-337). One NVSwitch node is one team.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ int my_pe(const SymmCtx& c) { return c.rank; }
__device__ __forceinline__ int n_pes(const SymmCtx& c) { return c.world; }
// Team queries: the only team is the node (TEAM_WORLD == TEAM_NODE), so team ranks are global ranks.
__device__ __forceinline__ int team_my_pe(const SymmCtx& c) { return c.rank; }
__device__ __forceinline__ int team_n_pes(const SymmCtx& c) { return c.world; }
__device__ __forceinline__ int team_translate_pe(const SymmCtx& c, int pe) { return pe >= 0 && pe < c.world ? pe : -1; }
// remote_ptr / remote_mc_ptr of the reference
template <typename T>
__device__ __forceinline__ T* remote_ptr(const SymmCtx& c, T* local_ptr, int pe) { return symm_at(c, local_ptr, pe); }
template <typename T>
__device__ __forceinline__ T* remote_mc_ptr(const SymmCtx& c, T* local_ptr) { return c.mc_base ? mc_ptr(c, local_ptr) : nullptr; }
// int_p: one 32-bit store into `pe`'s copy of a symmetric word
__device__ __forceinline__ void int_p(const SymmCtx& c, int32_t* dst_local, int32_t value, int pe) {
  st_relaxed_sys(reinterpret_cast<uint32_t*>(symm_at(c, dst_local, pe)), static_cast<uint32_t>(value));
}

// Non-blocking puts / gets. The copies above are already plain loads and stores that retire asynchronously, so the
// _nbi forms issue the same instructions; completion (and ordering against a later signal) is what quiet() / fence()
// give, exactly as for the blocking forms followed by a signal.
__device__ __forceinline__ void putmem_nbi_block(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int pe) {
  putmem_block(c, dst_local, src, nbytes, pe);
}
__device__ __forceinline__ void putmem_nbi_warp(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int pe) {
  putmem_warp(c, dst_local, src, nbytes, pe);
}
__device__ __forceinline__ void putmem_nbi(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int pe) {
  putmem(c, dst_local, src, nbytes, pe);
}
__device__ __forceinline__ void getmem_nbi_block(const SymmCtx& c, void* dst, const void* src_local, size_t nbytes, int pe) {
  getmem_block(c, dst, src_local, nbytes, pe);
}
__device__ __forceinline__ void getmem_nbi_warp(const SymmCtx& c, void* dst, const void* src_local, size_t nbytes, int pe) {
  getmem_warp(c, dst, src_local, nbytes, pe);
}
__device__ __forceinline__ void getmem(const SymmCtx& c, void* dst, const void* src_local, size_t nbytes, int pe) {
  copy_bytes_strided(dst, symm_at(c, reinterpret_cast<const uint8_t*>(src_local), pe), nbytes, 0, 1);
}
// putmem_signal for a warp and for one thread (the block form is above). The signal follows the data: the issuing
// lanes fence at system scope before the one signalling thread updates the peer's flag.
__device__ __forceinline__ void putmem_signal_warp(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes,
                                                   uint32_t* sig_local, uint32_t sig_value, SigOp op, int pe) {
  putmem_warp(c, dst_local, src, nbytes, pe);
  fence_acq_rel_sys();
  __syncwarp();
  if (lane_id() == 0) signal_op(c, sig_local, sig_value, op, pe);
}
__device__ __forceinline__ void putmem_signal(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes,
                                              uint32_t* sig_local, uint32_t sig_value, SigOp op, int pe) {
  putmem(c, dst_local, src, nbytes, pe);
  fence_acq_rel_sys();
  signal_op(c, sig_local, sig_value, op, pe);
}
__device__ __forceinline__ void putmem_signal_nbi_block(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes,
                                                        uint32_t* sig_local, uint32_t sig_value, SigOp op, int pe) {
  putmem_signal_block(c, dst_local, src, nbytes, sig_local, sig_value, op, pe);
}

// barrier_all executed by ONE warp per rank (lane k < world talks to peer k). Same flag protocol as
// barrier_all_block; `flags` must not be shared with a concurrent block-level barrier.
__device__ __forceinline__ bool barrier_all_warp(const SymmCtx& c, uint32_t* flags, uint32_t epoch) {
  __syncwarp();
  const int l = lane_id();
  bool ok = true;
  if (l < c.world) {
    fence_acq_rel_sys();
    st_release_sys(symm_at(c, flags + c.rank, l), epoch);
    ok = wait_flag<WaitCmp::GE, true>(c, flags + l, epoch, l, __LINE__);
    if (!ok) report_status(c, kStatusBarrierTimeout, l, epoch, 0, __LINE__);
  }
  return __all_sync(0xffffffffu, ok);
}
// sync_all: the barrier without the guarantee that earlier puts have completed (NVSHMEM's distinction). Stores here
// are ordinary memory operations that the release in the flag store already orders, so the two coincide.
__device__ __forceinline__ bool sync_all_block(const SymmCtx& c, uint32_t* flags, uint32_t epoch) { return barrier_all_block(c, flags, epoch); }
__device__ __forceinline__ bool sync_all_warp(const SymmCtx& c, uint32_t* flags, uint32_t epoch) { return barrier_all_warp(c, flags, epoch); }

// broadcast: `root` writes nbytes of `src` into `dst_local` of every rank (its own included). With an NVLS mapping
// one multimem.st per 16 bytes reaches all ranks through the switch; otherwise one store per peer. The caller
// synchronises before the data is read (barrier_all_block / a signal), as with NVSHMEM's collective.
// nbytes, dst and src 16-byte aligned.
__device__ __forceinline__ void broadcast_block(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int root) {
  if (c.rank != root) return;
  const int tid = flat_tid(), nth = blockDim.x * blockDim.y * blockDim.z;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst_local);
  for (size_t i = tid; i < nbytes / 16; i += nth) {
    const uint4 v = s[i];
    if (c.mc_base != 0) {
      multimem_st_v4(mc_ptr(c, d + i), v);
    } else {
      for (int k = 0; k < c.world; ++k) st_v4_relaxed_sys(symm_at(c, d + i, k), v);
    }
  }
}
__device__ __forceinline__ void broadcast_warp(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes, int root) {
  if (c.rank != root) return;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst_local);
  for (size_t i = lane_id(); i < nbytes / 16; i += 32) {
    const uint4 v = s[i];
    if (c.mc_base != 0) {
      multimem_st_v4(mc_ptr(c, d + i), v);
    } else {
      for (int k = 0; k < c.world; ++k) st_v4_relaxed_sys(symm_at(c, d + i, k), v);
    }
  }
}
// fcollect (all-gather): every rank writes its nbytes of `src` into slot `rank` of `dst_local` ([world][nbytes]) on
// every rank. Same synchronisation contract as broadcast.
__device__ __forceinline__ void fcollect_block(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes) {
  const int tid = flat_tid(), nth = blockDim.x * blockDim.y * blockDim.z;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst_local) + static_cast<size_t>(c.rank) * nbytes);
  for (size_t i = tid; i < nbytes / 16; i += nth) {
    const uint4 v = s[i];
    if (c.mc_base != 0) {
      multimem_st_v4(mc_ptr(c, d + i), v);
    } else {
      for (int k = 0; k < c.world; ++k) st_v4_relaxed_sys(symm_at(c, d + i, k), v);
    }
  }
}
__device__ __forceinline__ void fcollect_warp(const SymmCtx& c, void* dst_local, const void* src, size_t nbytes) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst_local) + static_cast<size_t>(c.rank) * nbytes);
  for (size_t i = lane_id(); i < nbytes / 16; i += 32) {
    const uint4 v = s[i];
    if (c.mc_base != 0) {
      multimem_st_v4(mc_ptr(c, d + i), v);
    } else {
      for (int k = 0; k < c.world; ++k) st_v4_relaxed_sys(symm_at(c, d + i, k), v);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// LL (low-latency) packets: 8 bytes = {data32, flag32}; the receiver polls the payload itself.
// (python/triton_dist/kernels/nvidia/low_latency_allgather.py:530-566)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void ll_store(uint64_t* dst, uint32_t data, uint32_t flag) {
  uint64_t v = (static_cast<uint64_t>(flag) << 32) | data;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(v) : "memory");
}
__device__ __forceinline__ bool ll_load(const SymmCtx& c, const uint64_t* src, uint32_t flag, uint32_t* data) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(src) : "memory");
    if (static_cast<uint32_t>(v >> 32) == flag) {
      *data = static_cast<uint32_t>(v);
      return true;
    }
    // back off once the packet is clearly not there yet: tens of thousands of threads re-reading their packet lines at
    // system scope otherwise compete in L2 with the very stores they are waiting for
    if (++spins > 4u) __nanosleep(spins > 32u ? 200u : 40u);
    if ((spins & 63u) == 0u) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > c.timeout_ns) {
        report_status(c, kStatusWaitTimeout, 0, flag, static_cast<uint32_t>(v >> 32), __LINE__);
        return false;
      }
      if (status_is_error(c)) return false;
    }
  }
}

// ----------------------------------------------------------------------------------------------
// small numeric helpers shared by kernels
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(h);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_f16x2(uint32_t v) {
  __half2 h = *reinterpret_cast<__half2*>(&v);
  return __half22float2(h);
}

}  // namespace b200
