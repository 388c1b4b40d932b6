// Persistent warp-specialised tcgen05 GEMM for sm_100a with three modes that share one mainloop:
//
//   PLAIN  C[M,N] = A[M,K] * B[N,K]^T                      (gemm_persistent of the reference,
//                                                           python/triton_dist/kernels/nvidia/allgather_gemm.py:660-744)
//   AG     C[M,N/r] = allgather(A)[M,K] * B[N/r,K]^T       (ag_gemm, allgather_gemm.py:145-251, 534-657)
//   RS     out[M/r,N] = reduce_scatter(A[M,K/r] * B[N,K/r]^T)   (gemm_rs with fuse_scatter,
//                                                           gemm_reduce_scatter.py:130-259, 515-590)
//
// One CTA per SM, 256 threads:
//   warp 0      TMA producer: 128x64 A tile + 256x64 B tile per stage, 128-byte swizzle, 4 stages
//   warp 1      one elected thread issues tcgen05.mma (M128 N256 K16, bf16/f16 -> f32) into TMEM;
//               two 256-column accumulators so the epilogue of tile i overlaps the mainloop of i+1
//   warps 2-3   AG mode: communication warps. Push gather (default): they store this rank's shard into every
//               peer's gather buffer, in the order in which the peers' tile schedules need it, and add the rows
//               to the destination's per-128-row-block counters. Pull gather: they copy the local shard,
//               publish it and pull the peers' shards with 16-byte loads. Either way the producer warp waits
//               (bounded) on a block's arrival before its first TMA load of the block, and TMA only ever
//               reads this GPU's own memory.
//               RS mode: warp 2 is the signalling warp. It waits for the epilogue warps of each tile, issues
//               the system-scope fence and bumps the owners' row counters, so the epilogue never waits for
//               its remote stores to be acknowledged.
//   warps 4-7   epilogue: tcgen05.ld -> convert -> swizzled smem staging -> 128-byte row segments.
//               RS mode stores each row into the owner rank's slot [src][row][col] through its peer
//               mapping; the signalling warp then bumps the owner's per-(src, block) row counter.
//   RS mode ends with a reduce phase in which all threads sum the `world` slots of this rank's
//   rows (fp32) as the blocks complete.
//
// All cross-rank and cross-CTA waits are bounded; on expiry the kernel records a status, unwinds
// every role through a CTA-wide abort flag, frees its TMEM and returns.
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/tcgen05.cuh"

#include <cstdlib>
#include <cstring>

namespace b200 {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;
constexpr int kBBytes = kBN * kBK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiBytes = 4 * 32 * 128;  // 4 warps x 32 rows x 64 bf16
constexpr int kGemmSmem = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr int kTmemCols = 512;
// CTA-pair variant: each CTA stages 128 rows of A and 128 of the 256 rows of B per k-block (32 KB), six stages deep.
constexpr int kPairBBytes = 128 * kBK * 2;
constexpr int kPairStageBytes = kABytes + kPairBBytes;
constexpr int kPairStages = 6;
static_assert(kPairStages * kPairStageBytes == kStages * kStageBytes, "both variants use the same shared-memory budget");
constexpr int kCommThreads = 64;
constexpr int kCommRows = 8;  // rows per communication chunk

enum GemmMode : int { kPlain = 0, kAG = 1, kRS = 2 };

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, group_m, m_rot;
  int bf16;          // 1 = bf16, 0 = f16 (inputs and output)
  void* C;           // PLAIN / AG: [M, ldc]
  int ldc;
  // ---- AG ----
  const void* a_local;   // this rank's shard [Mr, K]
  void* ag_buf[2];       // symmetric [world * Mr_cap, K], double-buffered by epoch parity
  uint32_t* ready;       // symmetric u32[world]: ready[s] == epoch once rank s published its shard
  uint32_t* blk_cnt;     // local u32[tiles_m cap]: rows of the block that have landed
  uint32_t* blk_flag;    // local u32[tiles_m cap]: == epoch once the block is complete
  uint32_t* sync;        // local u32[4]: [0] epoch, [1] done-CTA counter, [2] local-chunk counter
  int Mr;                // rows per rank (M / world)
  // push variant of the gather: every rank stores its shard into all peers' buffers and adds the rows it
  // delivered to the destination's per-block counters; a block is complete at base + rows_in_block
  int push;
  uint32_t* ag_cnt;      // symmetric u32[2][nblk_cap]: rows landed per 128-row block, by epoch parity (only ever grows)
  uint32_t* ag_base;     // local u32[2][nblk_cap]: counter values before this call
  int nblk_cap;
  // ---- RS ----
  void* slots[2];        // symmetric [world][Mr_cap][N], double-buffered by epoch parity
  uint32_t* rs_cnt;      // symmetric u32[world][rs_blocks]: rows received from src for block j
  uint32_t* rs_base;     // local u32[world][rs_blocks]: counter value before this call
  int Mr_cap;
  int rs_blocks;
  int rs_nvls;           // 1: partial tiles stay in this rank's own slots [owner][row][col]; the owner sums the
                         // `world` copies with one multimem.ld_reduce per vector (the switch does the additions)
  void* out;             // [Mr, N]
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int t, int& m_blk, int& n_blk) {
  const int per_group = p.group_m * p.tiles_n;
  const int group = t / per_group;
  const int first_m = group * p.group_m;
  const int gsize = min(p.group_m, p.tiles_m - first_m);
  const int in_group = t - group * per_group;
  const int mi = first_m + in_group % gsize;
  n_blk = in_group / gsize;
  m_blk = mi + p.m_rot;
  if (m_blk >= p.tiles_m) m_blk -= p.tiles_m;
}

__device__ __forceinline__ void comm_bar() { asm volatile("bar.sync 1, 64;" ::: "memory"); }

// Adds `nrows` landed rows [row0, row0 + nrows) to the arrival counters of the 128-row blocks they
// touch; whoever completes a block publishes its flag. Called by one thread after the chunk's
// stores were ordered before it (comm_bar) and fenced for the async proxy by their writers.
__device__ __forceinline__ void publish_rows(const GemmParams& p, int row0, int nrows, uint32_t epoch) {
  int r = row0;
  const int end = row0 + nrows;
  while (r < end) {
    const int b = r / kBM;
    const int bend = min(end, (b + 1) * kBM);
    const int n = bend - r;
    const int rows_in_block = min(kBM, p.M - b * kBM);
    const uint32_t old = atom_add_acqrel_gpu(p.blk_cnt + b, static_cast<uint32_t>(n));
    if (static_cast<int>(old) + n == rows_in_block) {
      p.blk_cnt[b] = 0;
      st_release_gpu(p.blk_flag + b, epoch);
    }
    r = bend;
  }
}

// Copy `nrows` rows of `row_bytes` from src to dst with the 64 communication threads, eight
// independent 16-byte loads in flight per thread.
__device__ __forceinline__ void comm_copy(uint8_t* dst, const uint8_t* src, size_t nbytes, int ct) {
  const size_t nvec = nbytes / 16;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  size_t i = ct;
  for (; i + 7 * kCommThreads < nvec; i += 8 * kCommThreads) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ld_v4_relaxed_sys(s + i + u * kCommThreads);
#pragma unroll
    for (int u = 0; u < 8; ++u) st_v4(d + i + u * kCommThreads, v[u]);
  }
  for (; i < nvec; i += kCommThreads) st_v4(d + i, ld_v4_relaxed_sys(s + i));
}

template <int kMode, int kCtas>
__global__ void __launch_bounds__(256, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                  const __grid_constant__ CUtensorMap tmB, const GemmParams p, const SymmCtx ctx) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr bool kPair = kCtas == 2;
  constexpr int kNS = kPair ? kPairStages : kStages;              // pipeline depth
  constexpr int kSB = kPair ? kPairStageBytes : kStageBytes;      // bytes per stage in this CTA
  uint8_t* epi_smem = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kEpiBytes);
  uint64_t* full_bar = bars;                        // [kNS] (pair: only the leader's copy is used)
  uint64_t* empty_bar = bars + kPairStages;         // [kNS]
  uint64_t* tfull_bar = bars + 2 * kPairStages;     // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* bcast = tmem_slot + 2;
  uint32_t* epi_done = tmem_slot + 3;  // RS: epilogue-warp completions, consumed by the signalling warp

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;  // pair: tiles are 256 rows high
  const int num_kb = (p.K + kBK - 1) / kBK;
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int unit = blockIdx.x / kCtas, num_units = gridDim.x / kCtas;  // a unit = one CTA or one CTA pair
  const int m_blocks = (p.M + kBM - 1) / kBM;
  const uint64_t pipe_timeout = ctx.timeout_ns;

  uint32_t epoch = 1;
  if (kMode != kPlain) epoch = epoch_begin(p.sync);
  const int par = epoch & 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kNS; ++i) {
      mbar_init(full_bar + i, 1);
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar + i, 1);
      mbar_init(tempty_bar + i, 4 * kCtas);  // pair: the epilogue warps of both CTAs release the leader's accumulator
    }
    *abort_flag = 0;
    *epi_done = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 2) {
    if (kPair) tmem_alloc_pair(tmem_slot, kTmemCols);
    else tmem_alloc(tmem_slot, kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kPair) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      const CUtensorMap* tmA = (kMode == kAG && par) ? &tmA1 : &tmA0;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += num_units) {
        int m_blk, n_blk;
        tile_coords(p, t, m_blk, n_blk);
        if (kPair) m_blk = 2 * m_blk + static_cast<int>(cta_rank);
        if (kMode == kAG && m_blk < m_blocks) {
          if (p.push) {
            const uint32_t rows = static_cast<uint32_t>(min(kBM, p.M - m_blk * kBM));
            const int idx = par * p.nblk_cap + m_blk;
            ok = wait_flag<WaitCmp::GE, true>(ctx, p.ag_cnt + idx, p.ag_base[idx] + rows, m_blk, __LINE__);
          } else {
            ok = wait_flag<WaitCmp::EQ, false>(ctx, p.blk_flag + m_blk, epoch, m_blk, __LINE__);
          }
          if (!ok) { *abort_flag = 1; break; }
          fence_proxy_async();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, pipe_timeout)) { ok = false; break; }
          uint8_t* sa = smem + stage * kSB;
          if (kPair) {
            // both CTAs' loads credit the leader's barrier; the leader announces the bytes of the whole pair
            if (leader) mbar_expect_tx(full_bar + stage, 2 * kSB);
            tma_load_2d_pair(sa, tmA, full_bar + stage, kb * kBK, m_blk * kBM);
            tma_load_2d_pair(sa + kABytes, &tmB, full_bar + stage, kb * kBK, n_blk * kBN + static_cast<int>(cta_rank) * 128);
          } else {
            mbar_expect_tx(full_bar + stage, kSB);
            tma_load_2d(sa, tmA, full_bar + stage, kb * kBK, m_blk * kBM);
            tma_load_2d(sa + kABytes, &tmB, full_bar + stage, kb * kBK, n_blk * kBN);
          }
          if (++stage == kNS) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (leader && elect_one()) {
      const uint32_t idesc = umma_idesc_f16(kBM * kCtas, kBN, p.bf16 != 0);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += num_units, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar + acc, acc_phase ^ 1, abort_flag, pipe_timeout)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar + stage, phase, abort_flag, pipe_timeout)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kSB);
          const uint64_t da = umma_desc_sw128_kmajor(sa);
          const uint64_t db = umma_desc_sw128_kmajor(sa + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            if (kPair) umma_f16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (kPair) {  // free the stage in both CTAs
            umma_commit_pair(mapa_u32(empty_bar + stage, 0));
            umma_commit_pair(mapa_u32(empty_bar + stage, 1));
          } else {
            umma_commit(empty_bar + stage);
          }
          if (++stage == kNS) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          if (kPair) {
            umma_commit_pair(mapa_u32(tfull_bar + acc, 0));
            umma_commit_pair(mapa_u32(tfull_bar + acc, 1));
          } else {
            umma_commit(tfull_bar + acc);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp < 4) {
    // ------------------------------------------------------------------ signalling warp (RS)
    if (kMode == kRS && warp == 2) {
      // For every tile of this CTA, in issue order: wait until the four epilogue warps have stored their rows into
      // the owners' slots, make those stores visible system-wide, and add the delivered rows to each owner's counter
      // for (this source, 128-row block). The fence can take microseconds on a loaded link; here it delays nobody.
      uint32_t it = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += num_units, ++it) {
        int m_blk, n_blk;
        tile_coords(p, t, m_blk, n_blk);
        if (kPair) m_blk = 2 * m_blk + static_cast<int>(cta_rank);
        const uint32_t want = 4u * (it + 1u);
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (true) {
          uint32_t seen;
          asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(seen) : "r"(smem_u32(epi_done)) : "memory");
          if (seen >= want) break;
          __nanosleep(64);
          if ((++spins & 63u) == 0u) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (*abort_flag != 0u || now - t0 > pipe_timeout) { ok = false; break; }
          }
        }
        if (!ok) break;
        const int r_lo = m_blk * kBM, r_hi = min(r_lo + kBM, p.M);
        if (r_lo < r_hi) {
          const int o_lo = r_lo / p.Mr, o_hi = (r_hi - 1) / p.Mr;
          for (int o = o_lo + lane; o <= o_hi; o += 32) {
            fence_acq_rel_sys();
            const int s0 = max(r_lo, o * p.Mr), s1 = min(r_hi, (o + 1) * p.Mr);
            const int j = m_blk - (o * p.Mr) / kBM;
            uint32_t* cnt = p.rs_cnt + ctx.rank * p.rs_blocks + j;
            red_add_release_sys(symm_at(ctx, cnt, o), static_cast<uint32_t>(s1 - s0));
          }
        }
      }
    }
    // ------------------------------------------------------------------ communication warps (AG)
    if (kMode == kAG) {
      const int ct = threadIdx.x - 64;
      const size_t row_bytes = static_cast<size_t>(p.K) * 2;
      uint8_t* buf = static_cast<uint8_t*>(p.ag_buf[par]);
      const int nch = (p.Mr + kCommRows - 1) / kCommRows;  // chunks per shard
      const int total_chunks = nch * ctx.world;            // local shard first, then peers in ring order
      if (p.push) {
        // Push: step s sends this rank's shard to rank - s, the peer whose tile schedule needs it s steps from now
        // (step 0 is the local copy). Stores are posted, so the gather runs at link speed however small M is.
        uint32_t* cnt = p.ag_cnt + par * p.nblk_cap;
        for (int g = blockIdx.x; g < total_chunks; g += gridDim.x) {
          const int step = g / nch;
          const int c = g - step * nch;
          int dst = ctx.rank - step;
          if (dst < 0) dst += ctx.world;
          const int r0 = c * kCommRows;
          const int nrows = min(kCommRows, p.Mr - r0);
          uint8_t* to = buf + (static_cast<size_t>(ctx.rank) * p.Mr + r0) * row_bytes;
          if (step != 0) to = symm_at(ctx, to, dst);
          comm_copy(to, static_cast<const uint8_t*>(p.a_local) + static_cast<size_t>(r0) * row_bytes, nrows * row_bytes, ct);
          if (step == 0) fence_proxy_async();
          comm_bar();
          if (ct == 0) {
            fence_acq_rel_sys();
            int r = ctx.rank * p.Mr + r0;
            const int end = r + nrows;
            while (r < end) {
              const int b = r / kBM;
              const int bend = min(end, (b + 1) * kBM);
              red_add_release_sys(symm_at(ctx, cnt + b, dst), static_cast<uint32_t>(bend - r));
              r = bend;
            }
          }
        }
      } else
      for (int g = blockIdx.x; g < total_chunks; g += gridDim.x) {
        const int step = g / nch;
        const int c = g - step * nch;
        int src = ctx.rank + step;
        if (src >= ctx.world) src -= ctx.world;
        const int r0 = c * kCommRows;
        const int nrows = min(kCommRows, p.Mr - r0);
        const size_t off = (static_cast<size_t>(src) * p.Mr + r0) * row_bytes;
        if (step == 0) {
          comm_copy(buf + off, static_cast<const uint8_t*>(p.a_local) + static_cast<size_t>(r0) * row_bytes,
                    nrows * row_bytes, ct);
        } else {
          if (ct == 0) {
            // at least this epoch: a peer that has finished this call may already have published the next one (its
            // buffer of this call's parity stays intact until the call after that, which needs this rank's next shard)
            bool ok = wait_flag<WaitCmp::GE, true>(ctx, p.ready + src, epoch, src, __LINE__);
            *bcast = ok ? 1u : 0u;
          }
          comm_bar();
          const bool ok = *bcast != 0u;
          comm_bar();
          if (!ok) break;
          comm_copy(buf + off, symm_at(ctx, buf + off, src), nrows * row_bytes, ct);
        }
        fence_proxy_async();
        comm_bar();
        if (ct == 0) {
          publish_rows(p, src * p.Mr + r0, nrows, epoch);
          if (step == 0 && ctx.world > 1) {
            // the CTA that lands the last local chunk tells every peer that this shard can be pulled
            const uint32_t old = atom_add_acqrel_gpu(p.sync + 2, 1u);
            if (old == static_cast<uint32_t>(nch - 1)) {
              p.sync[2] = 0;
              fence_acq_rel_sys();
              for (int k = 1; k < ctx.world; ++k) {
                int peer = ctx.rank + k;
                if (peer >= ctx.world) peer -= ctx.world;
                st_release_sys(symm_at(ctx, p.ready + ctx.rank, peer), epoch);
              }
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int w = warp - 4;  // == warp % 4: the TMEM lane quarter this warp may read
    uint8_t* stg = epi_smem + w * (32 * 128);
    uint32_t it = 0;
    for (int t = unit; t < total_tiles; t += num_units, ++it) {
      int m_blk, n_blk;
      tile_coords(p, t, m_blk, n_blk);
      if (kPair) m_blk = 2 * m_blk + static_cast<int>(cta_rank);
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      if (!mbar_wait(tfull_bar + acc, acc_phase, abort_flag, pipe_timeout)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(w * 32) << 16) + acc * kBN;
      const int row_base = m_blk * kBM + w * 32;
#pragma unroll 1
      for (int c = 0; c < kBN / 64; ++c) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr + c * 64, r0);
        tmem_ld_32x32(taddr + c * 64 + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t* r = j < 4 ? r0 + j * 8 : r1 + (j - 4) * 8;
          uint4 v;
          if (p.bf16) {
            v.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
            v.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
            v.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
            v.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
          } else {
            v.x = pack_f16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
            v.y = pack_f16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
            v.z = pack_f16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
            v.w = pack_f16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
          }
          *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) * 16)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3);
          const int ch = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) * 16));
          const int grow = row_base + rr;
          const int gcol = n_blk * kBN + c * 64 + ch * 8;
          if (grow < p.M && gcol < p.N) {
            if (kMode == kRS) {
              const int owner = grow / p.Mr;
              const int lrow = grow - owner * p.Mr;
              if (p.rs_nvls) {
                st_v4(static_cast<uint8_t*>(p.slots[par]) + ((static_cast<size_t>(owner) * p.Mr_cap + lrow) * p.N + gcol) * 2, v);
              } else {
                uint8_t* slot = static_cast<uint8_t*>(p.slots[par]) +
                                ((static_cast<size_t>(ctx.rank) * p.Mr_cap + lrow) * p.N + gcol) * 2;
                st_v4(symm_at(ctx, slot, owner), v);
              }
            } else {
              st_v4(static_cast<uint8_t*>(p.C) + (static_cast<size_t>(grow) * p.ldc + gcol) * 2, v);
            }
          }
        }
        __syncwarp();
      }
      // accumulator fully read: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (kPair && !leader) mbar_arrive_cluster(mapa_u32(tempty_bar + acc, 0));
        else mbar_arrive(tempty_bar + acc);
      }
      if (kMode == kRS && lane == 0) {
        // the stores above are ordered before this release by the __syncwarp; the signalling warp fences and tells
        // the owners, so that no epilogue warp ever waits for its remote stores to be acknowledged
        asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(epi_done)) : "memory");
      }
    }
  }
  // ---------------------------------------------------------------------- RS reduce phase
  __syncthreads();
  bool failed = *abort_flag != 0u;
  if (kMode == kRS && !failed) {
    const int seg0 = ctx.rank * p.Mr;
    const int first_blk = seg0 / kBM;
    const int vec_per_row = p.N / 8;
    const uint8_t* slots = static_cast<const uint8_t*>(p.slots[par]);
    // One work item = one row of this rank's segment; a thread owns up to four 16-byte vectors of the row and issues
    // all of their loads over all slots (4 x world) before it adds anything, so the phase runs at HBM speed instead
    // of one load latency per vector.
    // A CTA owns a contiguous run of rows, so it waits for one or two 128-row blocks in all.
    int ready_blk = -1;
    const int rows_per_cta = (p.Mr + gridDim.x - 1) / gridDim.x;
    const int row_begin = min(p.Mr, static_cast<int>(blockIdx.x) * rows_per_cta);
    const int row_end = min(p.Mr, row_begin + rows_per_cta);
    for (int lrow = row_begin; lrow < row_end && !failed; ++lrow) {
      const int j = (seg0 + lrow) / kBM - first_blk;
      if (j > ready_blk) {
        bool ok = true;
        if (threadIdx.x < ctx.world) {
          const int blk = first_blk + j;
          const int s0 = max(seg0, blk * kBM), s1 = min(seg0 + p.Mr, (blk + 1) * kBM);
          const uint32_t target = p.rs_base[threadIdx.x * p.rs_blocks + j] + static_cast<uint32_t>((s1 - s0) * p.tiles_n);
          ok = wait_flag<WaitCmp::GE, true>(ctx, p.rs_cnt + threadIdx.x * p.rs_blocks + j, target, threadIdx.x, __LINE__);
        }
        if (!__syncthreads_and(ok)) { failed = true; break; }
        ready_blk = j;
      }
      if (p.rs_nvls) {
        // in-switch reduction: every rank kept its partial rows for this owner at the same heap offset, so one
        // multimem load of that offset returns the sum over the ranks (fp32 accumulation inside the switch)
        const uint8_t* mine = slots + (static_cast<size_t>(ctx.rank) * p.Mr_cap + lrow) * p.N * 2;
        for (int v0 = threadIdx.x; v0 < vec_per_row; v0 += 4 * blockDim.x) {
          uint4 x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * blockDim.x;
            if (v < vec_per_row)
              x[u] = p.bf16 ? multimem_ld_reduce_bf16x8(mc_ptr(ctx, mine + v * 16)) : multimem_ld_reduce_f16x8(mc_ptr(ctx, mine + v * 16));
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * blockDim.x;
            if (v < vec_per_row) st_v4(static_cast<uint8_t*>(p.out) + (static_cast<size_t>(lrow) * p.N + v * 8) * 2, x[u]);
          }
        }
        continue;
      }
      for (int v0 = threadIdx.x; v0 < vec_per_row; v0 += 4 * blockDim.x) {
        uint4 x[4][kMaxRanks];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * blockDim.x;
          if (v < vec_per_row) {
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s)
              if (s < ctx.world)
                x[u][s] = ld_v4_relaxed_sys(slots + ((static_cast<size_t>(s) * p.Mr_cap + lrow) * p.N + v * 8) * 2);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * blockDim.x;
          if (v < vec_per_row) {
            float accv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s) {
              if (s < ctx.world) {
                const uint32_t xs[4] = {x[u][s].x, x[u][s].y, x[u][s].z, x[u][s].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float2 f = p.bf16 ? unpack_bf16x2(xs[q]) : unpack_f16x2(xs[q]);
                  accv[2 * q] += f.x;
                  accv[2 * q + 1] += f.y;
                }
              }
            }
            uint4 o;
            if (p.bf16) {
              o.x = pack_bf16x2(accv[0], accv[1]); o.y = pack_bf16x2(accv[2], accv[3]);
              o.z = pack_bf16x2(accv[4], accv[5]); o.w = pack_bf16x2(accv[6], accv[7]);
            } else {
              o.x = pack_f16x2(accv[0], accv[1]); o.y = pack_f16x2(accv[2], accv[3]);
              o.z = pack_f16x2(accv[4], accv[5]); o.w = pack_f16x2(accv[6], accv[7]);
            }
            st_v4(static_cast<uint8_t*>(p.out) + (static_cast<size_t>(lrow) * p.N + v * 8) * 2, o);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (kPair) cluster_sync_all();  // neither CTA's shared or tensor memory goes away while the pair may still use it
  if (warp == 2) {
    if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    if (*abort_flag != 0u) report_status(ctx, kStatusPipeTimeout, blockIdx.x, 0, 0, __LINE__);
    if (kMode != kPlain) {
      __threadfence();
      if (atomicAdd(p.sync + 1, 1u) == gridDim.x - 1) {
        p.sync[1] = 0;
        if (kMode == kAG && p.push) {
          for (int b = 0; b < m_blocks; ++b)
            p.ag_base[par * p.nblk_cap + b] += static_cast<uint32_t>(min(kBM, p.M - b * kBM));
        }
        if (kMode == kRS) {
          // every rank delivered its rows of this call: advance the counter bases
          const int seg0 = ctx.rank * p.Mr, first_blk = seg0 / kBM, last_blk = (seg0 + p.Mr - 1) / kBM;
          for (int j = 0; j <= last_blk - first_blk; ++j) {
            const int blk = first_blk + j;
            const int s0 = max(seg0, blk * kBM), s1 = min(seg0 + p.Mr, (blk + 1) * kBM);
            for (int s = 0; s < ctx.world; ++s)
              p.rs_base[s * p.rs_blocks + j] += static_cast<uint32_t>((s1 - s0) * p.tiles_n);
          }
        }
        __threadfence();
        p.sync[0] = epoch;
      }
    }
  }
}

// Whether the tiled GEMMs run as CTA pairs (256x256 tiles, cta_group::2). -1 = decide from B200DIST_GEMM_2CTA (default on).
static int g_two_cta = -1;
static bool two_cta_enabled() {
  if (g_two_cta < 0) {
    const char* e = getenv("B200DIST_GEMM_2CTA");
    g_two_cta = (e && e[0] == '0') ? 0 : 1;
  }
  return g_two_cta == 1;
}

template <int kMode, int kCtas>
static int launch_gemm_impl(const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b, const GemmParams& p,
                            const SymmCtx& ctx, int grid, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(gemm_sm100_kernel<kMode, kCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = kGemmSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kCtas > 1 ? 1 : 0;
  B200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemm_sm100_kernel<kMode, kCtas>, a0, a1, b, p, ctx));
  return kOk;
}

// B's TMA box is 256 rows for single CTAs and 128 rows for pairs, so the caller builds the map after this choice.
static bool use_pair(int M) { return two_cta_enabled() && M > kBM; }

template <int kMode>
static int launch_gemm(bool pair, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b, const GemmParams& p,
                       const SymmCtx& ctx, int grid, cudaStream_t stream) {
  if (pair) return launch_gemm_impl<kMode, 2>(a0, a1, b, p, ctx, grid & ~1, stream);
  return launch_gemm_impl<kMode, 1>(a0, a1, b, p, ctx, grid, stream);
}

// Tile geometry for the chosen variant: pairs tile M in 256-row steps (and rotate in those units).
static void set_tiles(GemmParams& p, bool pair, int first_row) {
  const int tm = pair ? 2 * kBM : kBM;
  p.tiles_m = (p.M + tm - 1) / tm;
  p.m_rot = first_row / tm;
  if (pair && p.group_m > 1) p.group_m = (p.group_m + 1) / 2;
}

static int fill_common(GemmParams& p, int M, int N, int K, int dtype, int group_m) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "gemm supports bf16 and f16, got dtype %d", dtype);
  B200_REQUIRE(M > 0 && N > 0 && K > 0, "empty problem %dx%dx%d", M, N, K);
  B200_REQUIRE(K % 8 == 0 && N % 8 == 0, "K (%d) and N (%d) must be multiples of 8", K, N);
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + kBM - 1) / kBM;
  p.tiles_n = (N + kBN - 1) / kBN;
  p.group_m = group_m > 0 ? group_m : 8;
  p.m_rot = 0;
  p.bf16 = dtype == kBF16;
  return kOk;
}

}  // namespace b200

using namespace b200;

// C[M,N] = A[M,K] * B[N,K]^T, all row-major with leading dimensions lda/ldb/ldc (elements).
B200_API int b200_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int dtype,
                       int max_ctas, void* stream) {
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int rc = fill_common(p, M, N, K, dtype, 16);
  if (rc != kOk) return rc;
  p.C = C;
  p.ldc = ldc;
  CUtensorMap ta, tb;
  rc = make_tma_2d(&ta, A, dtype, M, K, lda, kBM, kBK, true);
  if (rc != kOk) return rc;
  const bool pair = use_pair(M);
  set_tiles(p, pair, 0);
  rc = make_tma_2d(&tb, B, dtype, N, K, ldb, pair ? 128 : kBN, kBK, true);
  if (rc != kOk) return rc;
  SymmCtx ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.world = 1;
  ctx.timeout_ns = 4000000000ull;
  int grid = min(p.tiles_m * p.tiles_n * (pair ? 2 : 1), sm_count());
  if (max_ctas > 0) grid = min(grid, max_ctas);
  if (pair && grid < 2) grid = 2;
  return launch_gemm<kPlain>(pair, ta, ta, tb, p, ctx, grid, static_cast<cudaStream_t>(stream));
}

// AG-GEMM. a_local [Mr, K] is this rank's shard; ag_buf0/1 are the two symmetric gather buffers
// [world * Mr, K] (rows of rank s at s * Mr); B is [N, K]; C is [world * Mr, N].
// ready: symmetric u32[world]; blk_cnt/blk_flag: local u32[>= tiles_m]; sync: local u32[4]; all zero-initialised once.
// push != 0 selects the push gather: ag_cnt symmetric u32[2 * nblk_cap], ag_base local u32[2 * nblk_cap] (zero-initialised
// once); otherwise the communication warps pull and ag_cnt / ag_base are not touched.
B200_API int b200_ag_gemm(const void* symm_ctx, const void* a_local, void* ag_buf0, void* ag_buf1, const void* B, void* C,
                          int Mr, int N, int K, int ldb, int ldc, int dtype, uint32_t* ready, uint32_t* blk_cnt,
                          uint32_t* blk_flag, uint32_t* sync, int group_m, int max_ctas, int push, uint32_t* ag_cnt,
                          uint32_t* ag_base, int nblk_cap, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  const int M = Mr * ctx.world;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int rc = fill_common(p, M, N, K, dtype, group_m);
  if (rc != kOk) return rc;
  p.C = C;
  p.ldc = ldc;
  p.a_local = a_local;
  p.ag_buf[0] = ag_buf0;
  p.ag_buf[1] = ag_buf1;
  p.ready = ready;
  p.blk_cnt = blk_cnt;
  p.blk_flag = blk_flag;
  p.sync = sync;
  p.Mr = Mr;
  p.push = push;
  p.ag_cnt = ag_cnt;
  p.ag_base = ag_base;
  p.nblk_cap = nblk_cap;
  if (push) {
    B200_REQUIRE(ag_cnt != nullptr && ag_base != nullptr, "the push gather needs its block counters");
    B200_REQUIRE((M + kBM - 1) / kBM <= nblk_cap, "M (%d) needs more than %d block counters", M, nblk_cap);
  }
  const bool pair = use_pair(M);
  set_tiles(p, pair, ctx.rank * Mr);
  B200_REQUIRE((reinterpret_cast<uint64_t>(a_local) & 15u) == 0, "a_local must be 16-byte aligned");
  CUtensorMap ta0, ta1, tb;
  rc = make_tma_2d(&ta0, ag_buf0, dtype, M, K, K, kBM, kBK, true);
  if (rc != kOk) return rc;
  rc = make_tma_2d(&ta1, ag_buf1, dtype, M, K, K, kBM, kBK, true);
  if (rc != kOk) return rc;
  rc = make_tma_2d(&tb, B, dtype, N, K, ldb, pair ? 128 : kBN, kBK, true);
  if (rc != kOk) return rc;
  int grid = sm_count();
  if (max_ctas > 0) grid = min(grid, max_ctas);
  return launch_gemm<kAG>(pair, ta0, ta1, tb, p, ctx, grid, static_cast<cudaStream_t>(stream));
}

// GEMM-RS. A [M, K] (K is this rank's K shard), B [N, K], out [M / world, N].
// slots0/1: symmetric [world][Mr_cap][N]; rs_cnt: symmetric u32[world][rs_blocks]; rs_base: local
// u32[world][rs_blocks]; sync: local u32[4]; all zero-initialised once.
static int gemm_rs_impl(const void* symm_ctx, const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb,
                        int dtype, void* slots0, void* slots1, uint32_t* rs_cnt, uint32_t* rs_base, uint32_t* sync,
                        int Mr_cap, int rs_blocks, int group_m, int max_ctas, int nvls, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(M % ctx.world == 0, "M (%d) must be divisible by the world size (%d)", M, ctx.world);
  B200_REQUIRE(!nvls || ctx.mc_base != 0, "the in-switch reduction needs an NVLS multicast mapping");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int rc = fill_common(p, M, N, K, dtype, group_m);
  if (rc != kOk) return rc;
  p.Mr = M / ctx.world;
  B200_REQUIRE(p.Mr <= Mr_cap, "M / world (%d) exceeds the context capacity (%d)", p.Mr, Mr_cap);
  B200_REQUIRE((p.Mr + kBM - 1) / kBM + 1 <= rs_blocks, "rs_blocks (%d) too small for %d rows per rank", rs_blocks, p.Mr);
  p.slots[0] = slots0;
  p.slots[1] = slots1;
  p.rs_cnt = rs_cnt;
  p.rs_base = rs_base;
  p.sync = sync;
  p.Mr_cap = Mr_cap;
  p.rs_blocks = rs_blocks;
  p.rs_nvls = nvls ? 1 : 0;
  p.out = out;
  const bool pair = use_pair(M);
  set_tiles(p, pair, ((ctx.rank + 1) % ctx.world) * p.Mr);
  CUtensorMap ta, tb;
  rc = make_tma_2d(&ta, A, dtype, M, K, lda, kBM, kBK, true);
  if (rc != kOk) return rc;
  rc = make_tma_2d(&tb, B, dtype, N, K, ldb, pair ? 128 : kBN, kBK, true);
  if (rc != kOk) return rc;
  int grid = sm_count();
  if (max_ctas > 0) grid = min(grid, max_ctas);
  return launch_gemm<kRS>(pair, ta, ta, tb, p, ctx, grid, static_cast<cudaStream_t>(stream));
}

// nvls != 0: reduce in the switch (multimem.ld_reduce by the owner over every rank's local partial rows) instead of
// storing the rows into the owner's per-source slots and summing them there.
B200_API int b200_gemm_rs(const void* symm_ctx, const void* A, const void* B, void* out, int M, int N, int K, int lda,
                          int ldb, int dtype, void* slots0, void* slots1, uint32_t* rs_cnt, uint32_t* rs_base,
                          uint32_t* sync, int Mr_cap, int rs_blocks, int group_m, int max_ctas, int nvls, void* stream) {
  return gemm_rs_impl(symm_ctx, A, B, out, M, N, K, lda, ldb, dtype, slots0, slots1, rs_cnt, rs_base, sync, Mr_cap, rs_blocks,
                      group_m, max_ctas, nvls, stream);
}

// 1 = CTA pairs (256x256 tiles, cta_group::2), 0 = single CTAs (128x256), -1 = follow B200DIST_GEMM_2CTA.
B200_API int b200_set_gemm_two_cta(int mode) {
  b200::g_two_cta = mode;
  return kOk;
}
