// Grouped (MoE) tcgen05 GEMM for sm_100a: every 128-row tile of expert-sorted (token, k) pairs is multiplied by
// its expert's weight matrix W[e] [N, K]. Three modes share one mainloop:
//
//   PLAIN  out[pair, :] = A[pair / a_div, :] * W[e(pair)]^T (* row_scale[pair])
//   AG     the token rows come from all ranks: communication warps pull the peers' token shards over NVLink
//          into the local gather buffer while tiles whose source ranks have landed are already computed
//          (ag_group_gemm, python/triton_dist/kernels/nvidia/allgather_group_gemm.py:398-605)
//   RS     down-projection of tensor-parallel MoE: the epilogue applies the routing weight; after a grid barrier
//          the k copies of every token are summed, the sum is pushed into the owner rank's slot, and the owner
//          reduces the slots of all ranks (moe_reduce_rs_rowise, kernels/nvidia/moe_reduce_rs.py:379-601, 816-926)
//
// Rows of a tile are scattered tokens, so A cannot be one TMA box: four producer warps gather it with 16-byte
// cp.async copies (eight lanes per 128-byte row segment), writing the same 128-byte XOR swizzle that TMA would
// produce; cp.async.mbarrier.arrive makes each stage's barrier complete when the copies land, and the MMA thread
// issues fence.proxy.async before it reads the stage. W[e] arrives by TMA from a 3-D map [E, N, K], so a tile at
// the edge of N never reads the next expert. 384 threads:
//   warp 0 W producer | warp 1 MMA issuer | warps 2-3 communication (AG) | warps 4-7 epilogue | warps 8-11 A gather
// Tile metadata (sorted pair ids, expert per tile, source-rank range per tile, issue order, tile count) is read
// from device memory, so the grid is sized for the worst case and no host synchronisation is needed.
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/tcgen05.cuh"
#include "b200/moe_rs_phases.cuh"

#include <cstdlib>
#include <cstring>

namespace b200 {

constexpr int kGM = 128, kGK = 64;
constexpr int kGABytes = kGM * kGK * 2;
constexpr int kGEpiBytes = 4 * 32 * 128;
constexpr int kGThreads = 384;

// Tile width: 128 columns (6 stages of 32 KB) or 256 columns (4 stages of 48 KB). The wide tile gathers A once per
// 256 output columns and needs 96 instead of 128 bytes of shared-memory fill per tensor-core clock.
template <int kBN>
struct GTile {
  static constexpr int kStages = kBN == 256 ? 4 : 6;
  static constexpr int kWBytes = kBN * kGK * 2;
  static constexpr int kStageBytes = kGABytes + kWBytes;
  static constexpr int kSmem = kStages * kStageBytes + kGEpiBytes + 1024 + 512;
};

enum GroupedMode : int { kGPlain = 0, kGAG = 1, kGRS = 2 };

struct GroupedParams {
  int N, K, n_pairs, a_div, lda, ldo, tiles_n, bf16, max_tiles, bn;
  const void* A;
  const int32_t* sorted_ids;
  const int32_t* tile_expert;
  const int32_t* tile_order;  // nullable
  const int32_t* totals;      // [0] m_pad, [1] number of tiles
  void* out;                  // [n_pairs, ldo]
  const float* row_scale;     // [n_pairs] or null
  // ---- AG ----
  const void* a_local;        // this rank's tokens [Tr, K]
  void* ag_buf[2];            // symmetric [world * Tr, K], parity double buffer
  uint32_t* ready;            // symmetric u32[world]
  uint32_t* rank_cnt;         // local u32[world]: rows landed per source rank
  uint32_t* rank_flag;        // local u32[world]: == epoch once the shard of that rank is complete
  uint32_t* sync;             // local u32[4]: epoch, done counter, local chunk counter, grid barrier counter
  int Tr;                     // tokens per rank
  // ---- RS ----
  int topk, Tr_cap;
  void* slots[2];             // symmetric [world][Tr_cap][N]
  uint32_t* rs_cnt;           // symmetric u32[world]: rows received per source
  uint32_t* rs_base;          // local u32[world]
  void* rs_out;               // [Tr, N]
  int rs_nvls;                // RS: reduce in the switch (see b200/moe_rs_phases.cuh)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_g() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait_g() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void gcomm_bar() { asm volatile("bar.sync 1, 64;" ::: "memory"); }

__device__ __forceinline__ int work_tile(const GroupedParams& p, int w, int& n_blk) {
  const int slot = w / p.tiles_n;
  n_blk = w - slot * p.tiles_n;
  return p.tile_order ? p.tile_order[slot] : slot;
}

template <int kMode, int kGN>
__global__ void __launch_bounds__(kGThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const GroupedParams p, const SymmCtx ctx) {
  constexpr int kGStages = GTile<kGN>::kStages, kGWBytes = GTile<kGN>::kWBytes, kGStageBytes = GTile<kGN>::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + kGStages * kGStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kGEpiBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kGStages;
  uint64_t* tfull_bar = bars + 2 * kGStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* bcast = tmem_slot + 2;
  uint32_t* ready_cache = tmem_slot + 4;  // AG: [kMaxRanks] epoch of the last shard seen complete, per source rank

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = min(p.totals[1], p.max_tiles);
  const int total_work = num_tiles * p.tiles_n;
  const int num_kb = (p.K + kGK - 1) / kGK;
  const uint64_t pipe_timeout = ctx.timeout_ns;
  uint32_t epoch = 1;
  if (kMode != kGPlain) epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  const uint8_t* a_base = static_cast<const uint8_t*>(kMode == kGAG ? p.ag_buf[par] : p.A);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGStages; ++i) {
      mbar_init(full_bar + i, 128 + 1);
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar + i, 1);
      mbar_init(tempty_bar + i, 4);
    }
    *abort_flag = 0;
    for (int i = 0; i < kMaxRanks; ++i) ready_cache[i] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 2 * kGN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ W producer (TMA)
    const bool w_producer = elect_one();
    if (!w_producer && lane == 31 && kMode == kGAG) {
      // AG: ONE thread per CTA watches the per-source completion flags in global memory, in the order the shards are
      // pulled, and republishes them in shared memory for the 128 gather threads. (With every gather thread polling the
      // flags itself, ~19 K threads hammered one L2 line and starved the communication warps of this very GPU: the
      // local copy and the pull ran at a fifth of their speed.)
      for (int step = 1; step < ctx.world; ++step) {
        int src = ctx.rank + step;
        if (src >= ctx.world) src -= ctx.world;
        if (!wait_flag<WaitCmp::EQ, false>(ctx, p.rank_flag + src, epoch, src, __LINE__)) {
          *abort_flag = 1u;
          break;
        }
        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(ready_cache + src)), "r"(epoch) : "memory");
      }
    }
    if (w_producer) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int n_blk;
        const int tile = work_tile(p, w, n_blk);
        const int e = p.tile_expert[tile];
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, pipe_timeout)) { ok = false; break; }
          mbar_expect_tx(full_bar + stage, kGWBytes);
          tma_load_3d(smem + stage * kGStageBytes + kGABytes, &tmW, full_bar + stage, kb * kGK, n_blk * kGN, e);
          if (++stage == kGStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_f16(kGM, kGN, p.bf16 != 0);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar + acc, acc_phase ^ 1, abort_flag, pipe_timeout)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kGN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar + stage, phase, abort_flag, pipe_timeout)) { ok = false; break; }
          fence_view_async_shared();  // the gathered A rows were written through the generic proxy (cp.async)
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kGStageBytes);
          const uint64_t da = umma_desc_sw128_kmajor(sa);
          const uint64_t db = umma_desc_sw128_kmajor(sa + kGABytes);
#pragma unroll
          for (int k = 0; k < kGK / 16; ++k) umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty_bar + stage);
          if (++stage == kGStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(tfull_bar + acc);
      }
    }
    __syncwarp();
  } else if (warp < 4) {
    // ------------------------------------------------------------------ communication warps (AG)
    if (kMode == kGAG) {
      const int ct = threadIdx.x - 64;
      const size_t row_bytes = static_cast<size_t>(p.K) * 2;
      uint8_t* buf = static_cast<uint8_t*>(p.ag_buf[par]);
      constexpr int kRows = 8;
      constexpr int kInFlight = 16;  // 16-byte loads in flight per thread: 64 threads x 148 CTAs keep ~2.4 MB on the wire
      const int nch = (p.Tr + kRows - 1) / kRows;
      for (int g = blockIdx.x; g < nch * ctx.world; g += gridDim.x) {
        const int step = g / nch, c = g - step * nch;
        int src = ctx.rank + step;
        if (src >= ctx.world) src -= ctx.world;
        const int r0 = c * kRows, nrows = min(kRows, p.Tr - r0);
        const size_t off = (static_cast<size_t>(src) * p.Tr + r0) * row_bytes;
        const uint8_t* from;
        if (step == 0) {
          from = static_cast<const uint8_t*>(p.a_local) + static_cast<size_t>(r0) * row_bytes;
        } else {
          // at least this epoch: a peer that has finished this call may already have published the next one (its
          // buffer of this call's parity stays intact until the call after that, which needs this rank's next shard)
          if (ct == 0) *bcast = wait_flag<WaitCmp::GE, true>(ctx, p.ready + src, epoch, src, __LINE__) ? 1u : 0u;
          gcomm_bar();
          const bool ok = *bcast != 0u;
          gcomm_bar();
          if (!ok) break;
          from = symm_at(ctx, buf + off, src);
        }
        const size_t nvec = nrows * row_bytes / 16;
        for (size_t i = ct; i < nvec; i += 64 * kInFlight) {
          uint4 v[kInFlight];
#pragma unroll
          for (int u = 0; u < kInFlight; ++u)
            if (i + u * 64 < nvec) v[u] = ld_v4_relaxed_sys(reinterpret_cast<const uint4*>(from) + i + u * 64);
#pragma unroll
          for (int u = 0; u < kInFlight; ++u)
            if (i + u * 64 < nvec) st_v4(reinterpret_cast<uint4*>(buf + off) + i + u * 64, v[u]);
        }
        gcomm_bar();
        if (ct == 0) {
          const uint32_t old = atom_add_acqrel_gpu(p.rank_cnt + src, static_cast<uint32_t>(nrows));
          if (static_cast<int>(old) + nrows == p.Tr) {
            p.rank_cnt[src] = 0;
            st_release_gpu(p.rank_flag + src, epoch);
            if (step == 0) {  // this rank's shard is complete in the symmetric buffer: peers may pull it
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
  } else if (warp < 8) {
    // ------------------------------------------------------------------ epilogue warps
    const int w4 = warp - 4;
    uint8_t* stg = epi_smem + w4 * (32 * 128);
    uint32_t it = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++it) {
      int n_blk;
      const int tile = work_tile(p, w, n_blk);
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      const int my_pair = p.sorted_ids[tile * kGM + w4 * 32 + lane];
      const float my_scale = (p.row_scale && my_pair < p.n_pairs) ? p.row_scale[my_pair] : 1.f;
      if (!mbar_wait(tfull_bar + acc, acc_phase, abort_flag, pipe_timeout)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(w4 * 32) << 16) + acc * kGN;
#pragma unroll 1
      for (int c = 0; c < kGN / 64; ++c) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr + c * 64, r0);
        tmem_ld_32x32(taddr + c * 64 + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t* r = j < 4 ? r0 + j * 8 : r1 + (j - 4) * 8;
          float f[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) f[q] = __uint_as_float(r[q]) * my_scale;
          uint4 v;
          if (p.bf16) {
            v = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
          } else {
            v = make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
          }
          *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) * 16)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3), ch = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) * 16));
          const int pair = __shfl_sync(0xffffffffu, my_pair, rr);
          const int gcol = n_blk * kGN + c * 64 + ch * 8;
          if (pair < p.n_pairs && gcol < p.N)
            st_v4(static_cast<uint8_t*>(p.out) + (static_cast<size_t>(pair) * p.ldo + gcol) * 2, v);
        }
        __syncwarp();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar + acc);
    }
  } else {
    // ------------------------------------------------------------------ A gather producers
    // Eight consecutive lanes copy one 128-byte row segment (a whole line per row, four rows per warp instruction);
    // thread t owns 16-byte chunk t & 7 of rows (t >> 3) + 16 i, i = 0..7.
    const int t = threadIdx.x - 256;
    const int chunk = t & 7, rbase = t >> 3;
    const uint32_t sw_off = static_cast<uint32_t>(rbase * 128 + ((chunk ^ (rbase & 7)) * 16));
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      int n_blk;
      const int tile = work_tile(p, w, n_blk);
      const uint8_t* rp[8];
      int last_src = -1;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int pair = p.sorted_ids[tile * kGM + rbase + 16 * i];
        const bool valid = pair < p.n_pairs;
        const int src_row = valid ? pair / p.a_div : 0;
        bool local_row = false;
        if (kMode == kGAG && valid && ok) {
          const int src = src_row / p.Tr;
          // this rank's own tokens are read where the caller put them: no copy, no flag, so the tiles that need only
          // local rows start at once (the copy into the symmetric buffer is for the peers only)
          local_row = src == ctx.rank;
          if (!local_row && src != last_src) {
            // the shard's completion is republished in shared memory by the CTA's flag watcher (warp 0)
            uint32_t seen, spins = 0;
            while (true) {
              asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(seen) : "r"(smem_u32(ready_cache + src)) : "memory");
              if (seen == epoch) break;
              __nanosleep(100);
              if ((++spins & 63u) == 0u && *abort_flag != 0u) { ok = false; break; }
            }
            last_src = src;
          }
        }
        if (local_row)
          rp[i] = static_cast<const uint8_t*>(p.a_local) + (static_cast<size_t>(src_row - ctx.rank * p.Tr) * p.lda + chunk * 8) * 2;
        else
          rp[i] = valid ? a_base + (static_cast<size_t>(src_row) * p.lda + chunk * 8) * 2 : nullptr;
      }
      if (!ok) *abort_flag = 1;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, pipe_timeout)) { ok = false; break; }
        const uint32_t sa = smem_u32(smem + stage * kGStageBytes) + sw_off;
        const int col = kb * kGK + chunk * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool in = rp[i] != nullptr && col < p.K;
          cp_async16(sa + i * (16 * 128), in ? rp[i] + static_cast<size_t>(kb) * (kGK * 2) : a_base, in ? 16 : 0);
        }
        // the stage's barrier receives this thread's arrival when the copies above have landed: the producer never
        // blocks on its own copies, so every free stage has a gather in flight
        cp_async_arrive_noinc(full_bar + stage);
        if (++stage == kGStages) { stage = 0; phase ^= 1; }
      }
    }
    cp_async_wait_g<0>();  // nothing of this thread is in flight when the CTA's shared memory goes away
  }
  // (continues below: RS phases and teardown)

  // ---------------------------------------------------------------------- RS: topk-sum, scatter, owner reduce
  __syncthreads();
  bool failed = *abort_flag != 0u;
  if (kMode == kGRS && !failed) {
    // all tiles of this rank are in p.out ([n_pairs, N], routing weight applied)
    MoeRsArgs rs;
    rs.gemm_out = p.out; rs.ldo = p.ldo; rs.N = p.N; rs.topk = p.topk; rs.Tr = p.Tr; rs.Tr_cap = p.Tr_cap; rs.bf16 = p.bf16;
    rs.slots = p.slots[par]; rs.rs_cnt = p.rs_cnt; rs.rs_base = p.rs_base; rs.rs_out = p.rs_out; rs.barrier_ctr = p.sync + 3; rs.nvls = p.rs_nvls;
    failed = !moe_rs_phases(ctx, rs, epoch);
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, 2 * kGN);
  if (threadIdx.x == 0) {
    if (*abort_flag != 0u) report_status(ctx, kStatusPipeTimeout, blockIdx.x, 0, 0, __LINE__);
    if (kMode != kGPlain) {
      __threadfence();
      if (atomicAdd(p.sync + 1, 1u) == gridDim.x - 1) {
        p.sync[1] = 0;
        if (kMode == kGRS)
          for (int s = 0; s < ctx.world; ++s) p.rs_base[s] += static_cast<uint32_t>(p.Tr);
        __threadfence();
        p.sync[0] = epoch;
      }
    }
  }
}

template <int kMode, int kBN>
static int launch_grouped_bn(const CUtensorMap& tw, const GroupedParams& p, const SymmCtx& ctx, int grid, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<kMode, kBN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GTile<kBN>::kSmem));
    configured[dev & 63] = true;
  }
  if (kMode == kGRS) {
    // this mode crosses a grid-wide barrier between the GEMM and the reduce-scatter: launched cooperatively, so the
    // driver guarantees (or refuses) the co-residency the barrier needs
    B200_CHECK_CUDA(launch_cooperative(grouped_gemm_kernel<kMode, kBN>, dim3(grid), dim3(kGThreads), GTile<kBN>::kSmem, stream,
                                       tw, p, ctx));
    return kOk;
  }
  grouped_gemm_kernel<kMode, kBN><<<grid, kGThreads, GTile<kBN>::kSmem, stream>>>(tw, p, ctx);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
template <int kMode>
static int launch_grouped(const CUtensorMap& tw, const GroupedParams& p, const SymmCtx& ctx, int grid, cudaStream_t stream) {
  return p.bn == 256 ? launch_grouped_bn<kMode, 256>(tw, p, ctx, grid, stream)
                     : launch_grouped_bn<kMode, 128>(tw, p, ctx, grid, stream);
}

// Wide tiles when they waste no more columns than narrow ones would (N = 384 stays on 128-column tiles).
static int pick_bn(int N) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("B200DIST_GROUPED_BN");
    forced = e ? atoi(e) : 0;
  }
  if (forced == 128 || forced == 256) return forced;
  const int waste256 = (N + 255) / 256 * 256 - N, waste128 = (N + 127) / 128 * 128 - N;
  return (N >= 256 && waste256 <= waste128) ? 256 : 128;
}

static int fill_grouped(GroupedParams& p, CUtensorMap* tw, const void* W, int E, int N, int K, int n_pairs, int a_div,
                        const int32_t* sorted_ids, const int32_t* tile_expert, const int32_t* tile_order,
                        const int32_t* totals, int max_tiles, void* out, int ldo, const float* row_scale, int dtype) {
  B200_REQUIRE(dtype == kBF16 || dtype == kF16, "grouped gemm supports bf16/f16");
  B200_REQUIRE(K % 8 == 0 && N % 8 == 0, "K (%d) and N (%d) must be multiples of 8", K, N);
  memset(&p, 0, sizeof(p));
  p.N = N; p.K = K; p.n_pairs = n_pairs; p.a_div = a_div; p.ldo = ldo;
  p.bn = pick_bn(N);
  p.tiles_n = (N + p.bn - 1) / p.bn;
  p.bf16 = dtype == kBF16;
  p.max_tiles = max_tiles;
  p.sorted_ids = sorted_ids; p.tile_expert = tile_expert; p.tile_order = tile_order; p.totals = totals;
  p.out = out; p.row_scale = row_scale;
  return make_tma_3d(tw, W, dtype, K, N, E, K, static_cast<uint64_t>(N) * K, kGK, p.bn, 1, true);
}

}  // namespace b200

using namespace b200;

// out[pair, :] = A[pair / a_div, :] * W[e]^T (* row_scale[pair]) for the pairs listed in sorted_ids (tiles of 128 rows,
// one expert per tile, pad rows = n_pairs). W is [E, N, K]; A rows have pitch lda; out rows have pitch ldo.
B200_API int b200_grouped_gemm(const void* A, int lda, int a_div, const void* W, int E, int N, int K, int n_pairs,
                               const int32_t* sorted_ids, const int32_t* tile_expert, const int32_t* tile_order,
                               const int32_t* totals, int max_tiles, void* out, int ldo, const float* row_scale, int dtype,
                               void* stream) {
  GroupedParams p;
  CUtensorMap tw;
  int rc = fill_grouped(p, &tw, W, E, N, K, n_pairs, a_div, sorted_ids, tile_expert, tile_order, totals, max_tiles, out, ldo,
                        row_scale, dtype);
  if (rc != kOk) return rc;
  p.A = A; p.lda = lda;
  SymmCtx ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.world = 1;
  ctx.timeout_ns = 4000000000ull;
  int grid = sm_count();
  if (grid > max_tiles * p.tiles_n) grid = max_tiles * p.tiles_n;
  return launch_grouped<kGPlain>(tw, p, ctx, grid < 1 ? 1 : grid, static_cast<cudaStream_t>(stream));
}

// AG + grouped GEMM: a_local [Tr, K] are this rank's tokens; pairs index the gathered tokens (pair / topk = token).
static int ag_grouped_impl(const void* symm_ctx, const void* a_local, void* ag_buf0, void* ag_buf1, int Tr, int topk,
                           const void* W, int E, int N, int K, const int32_t* sorted_ids, const int32_t* tile_expert,
                           const int32_t* tile_order, const int32_t* totals, int max_tiles, void* out, int ldo,
                           uint32_t* ready, uint32_t* rank_cnt, uint32_t* rank_flag, uint32_t* sync, int dtype,
                           void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  GroupedParams p;
  CUtensorMap tw;
  const int n_pairs = Tr * ctx.world * topk;
  int rc = fill_grouped(p, &tw, W, E, N, K, n_pairs, topk, sorted_ids, tile_expert, tile_order, totals, max_tiles, out, ldo,
                        nullptr, dtype);
  if (rc != kOk) return rc;
  p.lda = K; p.a_local = a_local; p.ag_buf[0] = ag_buf0; p.ag_buf[1] = ag_buf1; p.ready = ready;
  p.rank_cnt = rank_cnt; p.rank_flag = rank_flag; p.sync = sync; p.Tr = Tr;
  return launch_grouped<kGAG>(tw, p, ctx, sm_count(), static_cast<cudaStream_t>(stream));
}

B200_API int b200_ag_grouped_gemm(const void* symm_ctx, const void* a_local, void* ag_buf0, void* ag_buf1, int Tr, int topk,
                                  const void* W, int E, int N, int K, const int32_t* sorted_ids, const int32_t* tile_expert,
                                  const int32_t* tile_order, const int32_t* totals, int max_tiles, void* out, int ldo,
                                  uint32_t* ready, uint32_t* rank_cnt, uint32_t* rank_flag, uint32_t* sync, int dtype,
                                  void* stream) {
  return ag_grouped_impl(symm_ctx, a_local, ag_buf0, ag_buf1, Tr, topk, W, E, N, K, sorted_ids, tile_expert, tile_order, totals,
                         max_tiles, out, ldo, ready, rank_cnt, rank_flag, sync, dtype, stream);
}

// Grouped GEMM + topk-reduce + reduce-scatter: A [n_pairs, K_local] (row per pair), W [E, N, K_local],
// row_scale [n_pairs] routing weights, gemm_out [n_pairs, N] local scratch, rs_out [Tr, N]. nvls != 0: the final sum over
// the ranks runs inside the switch (multimem.ld_reduce) instead of over per-source slots at the owner.
B200_API int b200_grouped_gemm_rs(const void* symm_ctx, const void* A, int lda, const void* W, int E, int N, int K, int Tr,
                                  int topk, const int32_t* sorted_ids, const int32_t* tile_expert, const int32_t* tile_order,
                                  const int32_t* totals, int max_tiles, const float* row_scale, void* gemm_out, void* slots0,
                                  void* slots1, int Tr_cap, uint32_t* rs_cnt, uint32_t* rs_base, uint32_t* sync, void* rs_out,
                                  int dtype, int nvls, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(Tr <= Tr_cap, "tokens per rank (%d) exceed the context capacity (%d)", Tr, Tr_cap);
  B200_REQUIRE(!nvls || ctx.mc_base != 0, "the in-switch reduction needs an NVLS multicast mapping");
  GroupedParams p;
  CUtensorMap tw;
  const int n_pairs = Tr * ctx.world * topk;
  int rc = fill_grouped(p, &tw, W, E, N, K, n_pairs, 1, sorted_ids, tile_expert, tile_order, totals, max_tiles, gemm_out, N,
                        row_scale, dtype);
  if (rc != kOk) return rc;
  p.A = A; p.lda = lda; p.sync = sync; p.Tr = Tr; p.topk = topk; p.Tr_cap = Tr_cap;
  p.slots[0] = slots0; p.slots[1] = slots1; p.rs_cnt = rs_cnt; p.rs_base = rs_base; p.rs_out = rs_out;
  p.rs_nvls = nvls ? 1 : 0;
  return launch_grouped<kGRS>(tw, p, ctx, sm_count(), static_cast<cudaStream_t>(stream));
}
