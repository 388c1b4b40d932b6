// Tutorial 05 - an all-gather written twice with the device primitives.
//
// `out` is a symmetric buffer of world * n words; after the call slot r of every rank holds rank r's `src`.
//
//   push   every rank copies its shard into slot [rank] of every peer (putmem_signal_block: the CTA copies, one thread
//          fences and adds 1 to the peer's arrival counter), then waits until its own counter shows `world` arrivals.
//          One kernel, no barrier: the data of a peer is usable as soon as that peer's signal is seen.
//   fcollect   the same thing with the collective of the SHMEM-style API (fcollect_block stores through the NVLS
//          multicast address when the heap has one: one store reaches every rank) followed by barrier_all_block.
//
// The reference teaches the pattern with copy engines and one flag per source in tutorials/02-intra-node-allgather.py.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

using namespace b200;

__global__ void allgather_push_kernel(const SymmCtx ctx, const uint32_t* src, uint32_t* out, int n, uint32_t* arrived,
                                      uint32_t arrived_base, uint32_t* ok_out) {
  __shared__ uint32_t ok_s;
  uint32_t* my_slot = out + static_cast<size_t>(ctx.rank) * n;  // LOCAL address of slot [rank]; peers' copies by offset
  for (int k = 0; k < ctx.world; ++k) {
    const int peer = (ctx.rank + k) % ctx.world;  // start with myself, then walk the ring so that links load evenly
    putmem_signal_block(ctx, my_slot, src, static_cast<size_t>(n) * 4, arrived, 1u, SigOp::ADD, peer);
  }
  // the counter only grows: `world` more arrivals than before this call means every slot has landed here
  if (threadIdx.x == 0) ok_s = wait_flag<WaitCmp::GE, true>(ctx, arrived, arrived_base + ctx.world) ? 1u : 0u;
  __syncthreads();
  if (threadIdx.x == 0) *ok_out = ok_s;
}

__global__ void allgather_fcollect_kernel(const SymmCtx ctx, const uint32_t* src, uint32_t* out, int n, uint32_t* flags,
                                          uint32_t epoch, uint32_t* ok_out) {
  fcollect_block(ctx, out, src, static_cast<size_t>(n) * 4);
  const bool ok = barrier_all_block(ctx, flags, epoch);  // fences, tells every peer, waits for every peer
  if (threadIdx.x == 0) *ok_out = ok ? 1u : 0u;
}

extern "C" __attribute__((visibility("default"))) int tutorial_allgather(const void* symm_ctx, int variant, const void* src,
                                                                         void* out, int n, void* sync, unsigned round,
                                                                         void* ok_out, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  if (n % 4 != 0) return -1;  // the block copies move 16-byte vectors
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (variant == 0)  // sync[0]: arrival counter, `world` arrivals per earlier round
    allgather_push_kernel<<<1, 512, 0, s>>>(ctx, static_cast<const uint32_t*>(src), static_cast<uint32_t*>(out), n,
                                            static_cast<uint32_t*>(sync), round * ctx.world, static_cast<uint32_t*>(ok_out));
  else               // sync[8 .. 8 + world): barrier flags, epoch = round + 1
    allgather_fcollect_kernel<<<1, 512, 0, s>>>(ctx, static_cast<const uint32_t*>(src), static_cast<uint32_t*>(out), n,
                                                static_cast<uint32_t*>(sync) + 8, round + 1, static_cast<uint32_t*>(ok_out));
  return static_cast<int>(cudaGetLastError());
}
