// Tutorial 01 - a producer / consumer queue between two ranks, written with the device primitives.
//
// Rank r produces `chunks` chunks of `chunk_words` words and writes each one straight into the queue of rank r + 1
// (putmem_signal_block: the CTA copies, then one thread fences and adds 1 to the consumer's counter). At the same
// time it consumes the chunks that rank r - 1 produces for it: one thread waits until the counter has reached the
// chunk's number, then the CTA sums the chunk. Data and flag live in the symmetric heap, so `queue` and `counter` are
// LOCAL addresses; the primitives translate them to the peer's copy.
//
// The reference teaches the same pattern with dl.notify / dl.wait in tutorials/01-distributed-notify-wait.py.
#include "b200/host.h"
#include "b200/primitives.cuh"

#include <cstring>

using namespace b200;

__global__ void producer_consumer_kernel(const SymmCtx ctx, const uint32_t* produced, uint32_t* queue, uint32_t* counter,
                                         uint32_t counter_base, int chunks, int chunk_words, unsigned long long* sum_out,
                                         uint32_t* ok_out) {
  __shared__ unsigned long long partial[32];
  __shared__ uint32_t ok_s;
  const int next = (ctx.rank + 1) % ctx.world;
  unsigned long long acc = 0;
  bool ok = true;
  for (int c = 0; c < chunks && ok; ++c) {
    // produce chunk c for the next rank: data first, then the signal that releases it
    putmem_signal_block(ctx, queue + static_cast<size_t>(c) * chunk_words, produced + static_cast<size_t>(c) * chunk_words,
                        static_cast<size_t>(chunk_words) * 4, counter, 1u, SigOp::ADD, next);
    // consume chunk c of the previous rank: the counter only grows, so "at least base + c + 1" means chunk c landed
    if (threadIdx.x == 0) ok_s = wait_flag<WaitCmp::GE, true>(ctx, counter, counter_base + c + 1) ? 1u : 0u;
    __syncthreads();
    ok = ok_s != 0u;
    if (ok)
      for (int i = threadIdx.x; i < chunk_words; i += blockDim.x)
        acc += ld_relaxed_sys(queue + static_cast<size_t>(c) * chunk_words + i);  // bypass L1: a peer wrote this line
    __syncthreads();
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += partial[w];
    *sum_out = t;
    *ok_out = ok ? 1u : 0u;
  }
}

// symm_ctx: the bytes of SymmHeap.ctx. counter_base: the counter's value before this call (it is never reset).
extern "C" __attribute__((visibility("default"))) int tutorial_producer_consumer(
    const void* symm_ctx, const void* produced, void* queue, void* counter, unsigned counter_base, int chunks,
    int chunk_words, void* sum_out, void* ok_out, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  if (chunk_words % 4 != 0) return -1;  // putmem_block copies 16-byte vectors
  producer_consumer_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ctx, static_cast<const uint32_t*>(produced), static_cast<uint32_t*>(queue), static_cast<uint32_t*>(counter),
      counter_base, chunks, chunk_words, static_cast<unsigned long long*>(sum_out), static_cast<uint32_t*>(ok_out));
  return static_cast<int>(cudaGetLastError());
}
