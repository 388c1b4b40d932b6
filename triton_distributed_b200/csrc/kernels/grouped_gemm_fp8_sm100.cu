// Grouped (MoE) fp8 GEMM for sm_100a with block scales, DeepSeek-style:
//
//   out[pair, n] = row_scale[pair] * sum over k-blocks kb of
//                  sa[row(pair), kb] * sw[e(pair), n / 128, kb] * (A8[row(pair), kb] . W8[e(pair), n, kb])
//
// A8 is e4m3 [rows, K] with one fp32 scale per row and 128 channels (what the expert-parallel dispatch kernel
// produces), W8 is e4m3 [E, N, K] with one fp32 scale per 128 x 128 block. One k-block (128 channels = one scale
// block) is one pipeline stage: the MMA thread issues four tcgen05.mma kind::f8f6f4 (K = 32 each) into one of two
// 128-column TMEM partial buffers, and the epilogue warps promote every partial into fp32 register accumulators
// with the product of the two scales while the next k-block is being multiplied. Rows of a tile are scattered, so
// A is gathered by cp.async (eight lanes per 128-byte row segment, completion through cp.async.mbarrier.arrive);
// W[e] arrives by TMA from a 3-D map. 384 threads, registers rebalanced with setmaxnreg:
//   warp 0 W producer | warp 1 MMA issuer | warps 2-3 idle | warps 4-7 promotion + epilogue (232 registers) |
//   warps 8-11 A gather
//
// Three modes share the mainloop (the AG and RS machinery is that of grouped_gemm_sm100.cu):
//   PLAIN  rows and scales are local
//   AG     rows come from all ranks. A row travels together with its scales ([K bytes of e4m3 | K / 128 fp32 scales],
//          pitch lda): warps 2-3 pull the peers' shards into the local gather buffer while tiles whose source ranks
//          have landed are computed; this rank's own rows are read in place
//   RS     down-projection of tensor-parallel MoE: the epilogue applies the routing weight, then the shared top-k
//          reduction + reduce-scatter phases run (b200/moe_rs_phases.cuh)
//
// Role in the reference: the fp8 path of the expert-parallel MoE inference test
// (python/triton_dist/test/nvidia/test_ep_moe_inference.py:169-327) and the grouped GEMM mainloops
// (kernels/nvidia/allgather_group_gemm.py:531-605), which run block-scaled fp8 through Triton's dot.
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/tcgen05.cuh"
#include "b200/moe_rs_phases.cuh"

#include <cstring>

namespace b200 {

constexpr int kFM = 128, kFN = 128, kFK = 128;  // tile rows, tile columns, channels (= bytes) per k-block
constexpr int kFStages = 6;
constexpr int kFABytes = kFM * kFK, kFWBytes = kFN * kFK, kFStageBytes = kFABytes + kFWBytes;
constexpr int kFEpiBytes = 4 * 32 * 128;
constexpr int kFSmem = kFStages * kFStageBytes + kFEpiBytes + 1024 + 512;
constexpr int kFThreads = 384;

struct Fp8GroupedParams {
  int N, K, n_pairs, a_div, lda, ldo, tiles_n, max_tiles, num_kb, sa_ld, bf16;
  const uint8_t* A;           // e4m3 rows, pitch lda bytes
  const float* sa;            // [rows, sa_ld] activation scales, one per 128 channels
  const float* sw;            // [E, tiles_n, num_kb] weight scales, one per 128 x 128 block
  const int32_t* sorted_ids;  // [tiles * 128] pair per sorted row, pad = n_pairs
  const int32_t* tile_expert;
  const int32_t* totals;      // [1] number of tiles
  void* out;                  // [n_pairs, ldo] bf16 / f16
  const float* row_scale;     // [n_pairs] or null
  const int32_t* tile_order;  // nullable: issue order of the tiles
  uint32_t* sync;             // AG / RS: local u32[4]: epoch, done counter, unused, grid barrier counter
  // ---- AG ---- (rows are [K e4m3 | K / 128 fp32], pitch lda; sa is unused)
  const uint8_t* a_local;     // this rank's rows [Tr, lda]
  uint8_t* ag_buf[2];         // symmetric [world * Tr, lda], parity double buffer
  uint32_t* ready;            // symmetric u32[world]
  uint32_t* rank_cnt;         // local u32[world]: rows landed per source rank
  uint32_t* rank_flag;        // local u32[world]: == epoch once the shard of that rank is complete
  int Tr;                     // tokens per rank
  // ---- RS ----
  int topk, Tr_cap;
  void* slots[2];             // symmetric [world][Tr_cap][N]
  uint32_t* rs_cnt;           // symmetric u32[world]
  uint32_t* rs_base;          // local u32[world]
  void* rs_out;               // [Tr, N]
  int rs_nvls;                // RS: reduce in the switch (see b200/moe_rs_phases.cuh)
};

enum Fp8GroupedMode : int { kFPlain = 0, kFAG = 1, kFRS = 2 };
__device__ __forceinline__ void f8_comm_bar() { asm volatile("bar.sync 1, 64;" ::: "memory"); }

__device__ __forceinline__ void f8_cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void f8_cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void f8_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int kMode>
__global__ void __launch_bounds__(kFThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const Fp8GroupedParams p, const SymmCtx ctx,
                        uint32_t* status) {
  const uint64_t timeout_ns = ctx.timeout_ns;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + kFStages * kFStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kFEpiBytes);
  uint64_t* full_bar = bars;                  // [stages] 128 gather arrivals + the W producer's expect_tx arrival
  uint64_t* empty_bar = bars + kFStages;      // [stages] tcgen05.commit
  uint64_t* pfull_bar = bars + 2 * kFStages;  // [2] partial buffer written (tcgen05.commit)
  uint64_t* pempty_bar = pfull_bar + 2;       // [2] partial buffer promoted (four epilogue warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* bcast = tmem_slot + 2;
  uint32_t* ready_cache = tmem_slot + 4;  // AG: [kMaxRanks] epoch of the last shard seen complete, per source rank

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = min(p.totals[1], p.max_tiles);
  const int total_work = num_tiles * p.tiles_n;
  uint32_t epoch = 1;
  if (kMode != kFPlain) epoch = epoch_begin(p.sync);
  const int par = epoch & 1;
  const uint8_t* a_base = kMode == kFAG ? p.ag_buf[par] : p.A;
  auto work_tile = [&](int w, int& n_blk) {
    const int slot = w / p.tiles_n;
    n_blk = w - slot * p.tiles_n;
    return p.tile_order ? p.tile_order[slot] : slot;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kFStages; ++i) {
      mbar_init(full_bar + i, 128 + 1);
      mbar_init(empty_bar + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(pfull_bar + i, 1);
      mbar_init(pempty_bar + i, 4);
    }
    *abort_flag = 0;
    for (int i = 0; i < kMaxRanks; ++i) ready_cache[i] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
  }
  if (warp == 2) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Roles by warpgroup, each starting with its register budget: the promotion warps hold 128 fp32 accumulators per
  // thread, everybody else gives registers back.
  if (warp < 4) {
    if (kMode == kFAG) asm volatile("setmaxnreg.dec.sync.aligned.u32 120;");  // the communication warps keep 16 vectors in flight
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ------------------------------------------------------------------ W producer (TMA)
    const bool w_producer = elect_one();
    if (!w_producer && lane == 31 && kMode == kFAG) {
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
        const int tile = work_tile(w, n_blk);
        const int e = p.tile_expert[tile];
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, timeout_ns)) { ok = false; break; }
          mbar_expect_tx(full_bar + stage, kFWBytes);
          tma_load_3d(smem + stage * kFStageBytes + kFABytes, &tmW, full_bar + stage, kb * kFK, n_blk * kFN, e);
          if (++stage == kFStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_e4m3(kFM, kFN);
      uint32_t stage = 0, phase = 0, pcount = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        for (int kb = 0; kb < p.num_kb; ++kb, ++pcount) {
          const uint32_t pb = pcount & 1, pphase = (pcount >> 1) & 1;
          if (!mbar_wait(pempty_bar + pb, pphase ^ 1, abort_flag, timeout_ns)) { ok = false; break; }
          if (!mbar_wait(full_bar + stage, phase, abort_flag, timeout_ns)) { ok = false; break; }
          fence_view_async_shared();  // the gathered A rows were written through the generic proxy (cp.async)
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kFStageBytes);
          const uint64_t da = umma_desc_sw128_kmajor(sa);
          const uint64_t db = umma_desc_sw128_kmajor(sa + kFABytes);
          const uint32_t d_tmem = tmem_base + pb * kFN;
#pragma unroll
          for (int k = 0; k < kFK / 32; ++k) umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, k != 0 ? 1u : 0u);
          umma_commit(empty_bar + stage);
          umma_commit(pfull_bar + pb);
          if (++stage == kFStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (kMode == kFAG) {
    // ------------------------------------------------------------------ communication warps (AG), warps 2-3
    const int ct = threadIdx.x - 64;
    const size_t row_bytes = static_cast<size_t>(p.lda);
    uint8_t* buf = p.ag_buf[par];
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
        from = p.a_local + static_cast<size_t>(r0) * row_bytes;
      } else {
        // at least this epoch: a peer that has finished this call may already have published the next one
        if (ct == 0) *bcast = wait_flag<WaitCmp::GE, true>(ctx, p.ready + src, epoch, src, __LINE__) ? 1u : 0u;
        f8_comm_bar();
        const bool ok = *bcast != 0u;
        f8_comm_bar();
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
      f8_comm_bar();
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
    // ------------------------------------------------------------------ promotion + epilogue warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int w4 = warp - 4;  // == warp % 4: the TMEM lane quarter this warp may read
    uint8_t* stg = epi_smem + w4 * (32 * 128);
    uint32_t pcount = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      int n_blk;
      const int tile = work_tile(w, n_blk);
      const int e = p.tile_expert[tile];
      const int my_pair = p.sorted_ids[tile * kFM + w4 * 32 + lane];
      const bool valid = my_pair < p.n_pairs;
      const float my_rs = (p.row_scale && valid) ? p.row_scale[my_pair] : 1.f;
      const float* sa_row;
      if (kMode == kFAG) {
        // the scales travel behind the row's K bytes; this rank's own rows are read where the caller put them
        const int src_row = valid ? my_pair / p.a_div : ctx.rank * p.Tr;
        const bool local_row = src_row / p.Tr == ctx.rank;
        const uint8_t* row = local_row ? p.a_local + static_cast<size_t>(src_row - ctx.rank * p.Tr) * p.lda
                                       : a_base + static_cast<size_t>(src_row) * p.lda;
        sa_row = reinterpret_cast<const float*>(row + p.K);
      } else {
        sa_row = p.sa + static_cast<size_t>(valid ? my_pair / p.a_div : 0) * p.sa_ld;
      }
      const float* sw_row = p.sw + (static_cast<size_t>(e) * p.tiles_n + n_blk) * p.num_kb;
      float acc[kFN];
#pragma unroll
      for (int j = 0; j < kFN; ++j) acc[j] = 0.f;
      // The scale of k-block kb is sa[row, kb] * sw[e, n, kb]: two global loads per k-block. They are requested four
      // k-blocks ahead and kept as raw values (no arithmetic on them until their k-block), so their latency never sits
      // between two promotions; with a look-ahead of one the loop ran at one L2 round trip per k-block, about six times
      // the time of the k-block's MMAs. AG: a gathered row's scales may be read only after the tile's first partial is
      // complete (by then the gather warps have seen the row's shard land); they are read past L1.
      auto ld_sa = [&](int kb) -> float { return valid ? (kMode == kFAG ? __ldcg(sa_row + kb) : sa_row[kb]) : 0.f; };
      float sa_r[4], sw_r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sw_r[j] = j < p.num_kb ? sw_row[j] : 0.f;
        sa_r[j] = (kMode != kFAG && j < p.num_kb) ? ld_sa(j) : 0.f;
      }
      for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = kb0 + j;
          if (kb >= p.num_kb || !ok) break;  // uniform over the CTA's promotion warps
          const uint32_t pb = pcount & 1, pphase = (pcount >> 1) & 1;
          ++pcount;
          if (!mbar_wait(pfull_bar + pb, pphase, abort_flag, timeout_ns)) { ok = false; break; }
          if (kMode == kFAG && kb == 0) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) sa_r[jj] = jj < p.num_kb ? ld_sa(jj) : 0.f;
          }
          const float s = sa_r[j] * sw_r[j];
          if (kb + 4 < p.num_kb) {  // refill this slot for the k-block four ahead
            sa_r[j] = ld_sa(kb + 4);
            sw_r[j] = sw_row[kb + 4];
          }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(w4 * 32) << 16) + pb * kFN;
          // 16 columns in registers while the next 16 are on their way from TMEM (two small buffers in turn: the 128
          // accumulators leave no room for more)
          uint32_t r0[16], r1[16];
          tmem_ld_32x16(taddr, r0);
#pragma unroll
          for (int h = 0; h < 8; ++h) {
            tmem_ld_wait();
            if (h + 1 < 8) tmem_ld_32x16(taddr + (h + 1) * 16, (h & 1) ? r0 : r1);
            uint32_t* r = (h & 1) ? r1 : r0;
#pragma unroll
            for (int q = 0; q < 16; ++q) acc[h * 16 + q] = fmaf(s, __uint_as_float(r[q]), acc[h * 16 + q]);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(pempty_bar + pb);
        }
      }
      if (!ok) break;
      // ---- write the tile: convert, stage through swizzled shared memory, store 128-byte row segments
#pragma unroll
      for (int c = 0; c < kFN / 64; ++c) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float f[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) f[q] = acc[c * 64 + j * 8 + q] * my_rs;
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
          const int gcol = n_blk * kFN + c * 64 + ch * 8;
          if (pair < p.n_pairs && gcol < p.N)
            st_v4(static_cast<uint8_t*>(p.out) + (static_cast<size_t>(pair) * p.ldo + gcol) * 2, v);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ A gather producers
    // thread t owns 16-byte chunk t & 7 of rows (t >> 3) + 16 i, i = 0..7: eight lanes copy one 128-byte row segment
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    const int t = threadIdx.x - 256;
    const int chunk = t & 7, rbase = t >> 3;
    const uint32_t sw_off = static_cast<uint32_t>(rbase * 128 + ((chunk ^ (rbase & 7)) * 16));
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      int n_blk_unused;
      const int tile = work_tile(w, n_blk_unused);
      const uint8_t* rp[8];
      int last_src = -1;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int pair = p.sorted_ids[tile * kFM + rbase + 16 * i];
        const bool valid = pair < p.n_pairs;
        const int src_row = valid ? pair / p.a_div : 0;
        bool local_row = false;
        if (kMode == kFAG && valid && ok) {
          const int src = src_row / p.Tr;
          local_row = src == ctx.rank;  // read in place: no copy, no flag
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
        if (local_row) rp[i] = p.a_local + static_cast<size_t>(src_row - ctx.rank * p.Tr) * p.lda + chunk * 16;
        else rp[i] = valid ? a_base + static_cast<size_t>(src_row) * p.lda + chunk * 16 : nullptr;
      }
      if (!ok) *abort_flag = 1;
      for (int kb = 0; kb < p.num_kb && ok; ++kb) {
        if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, timeout_ns)) { ok = false; break; }
        const uint32_t sa = smem_u32(smem + stage * kFStageBytes) + sw_off;
        const bool in_k = kb * kFK + chunk * 16 < p.K;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool in = rp[i] != nullptr && in_k;
          f8_cp_async16(sa + i * (16 * 128), in ? rp[i] + static_cast<size_t>(kb) * kFK : a_base, in ? 16 : 0);
        }
        f8_cp_async_arrive_noinc(full_bar + stage);
        if (++stage == kFStages) { stage = 0; phase ^= 1; }
      }
    }
    f8_cp_async_wait_all();
  }

  // ---------------------------------------------------------------------- RS: topk-sum, scatter, owner reduce
  if (kMode == kFRS) {
    // every warp runs the reduce phases: bring all warpgroups to the same register allocation first (the promotion
    // warps give back what the others take)
    if (warp >= 4 && warp < 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 168;");
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
  }
  __syncthreads();
  bool failed = *abort_flag != 0u;
  if (kMode == kFRS && !failed) {
    MoeRsArgs rs;
    rs.gemm_out = p.out; rs.ldo = p.ldo; rs.N = p.N; rs.topk = p.topk; rs.Tr = p.Tr; rs.Tr_cap = p.Tr_cap; rs.bf16 = p.bf16;
    rs.slots = p.slots[par]; rs.rs_cnt = p.rs_cnt; rs.rs_base = p.rs_base; rs.rs_out = p.rs_out; rs.barrier_ctr = p.sync + 3; rs.nvls = p.rs_nvls;
    failed = !moe_rs_phases(ctx, rs, epoch);
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, 256);
  if (threadIdx.x == 0) {
    if (*abort_flag != 0u) {
      if (status != nullptr) atomicMax(status, static_cast<uint32_t>(kStatusPipeTimeout));
      if (kMode != kFPlain) report_status(ctx, kStatusPipeTimeout, blockIdx.x, 0, 0, __LINE__);
    }
    if (kMode != kFPlain) {
      __threadfence();
      if (atomicAdd(p.sync + 1, 1u) == gridDim.x - 1) {
        p.sync[1] = 0;
        if (kMode == kFRS)
          for (int s = 0; s < ctx.world; ++s) p.rs_base[s] += static_cast<uint32_t>(p.Tr);
        __threadfence();
        p.sync[0] = epoch;
      }
    }
  }
}

static int fp8_fill(Fp8GroupedParams& p, CUtensorMap* tw, const void* A8, int lda, const float* sa, int sa_ld, int a_div,
                    const void* W8, const float* sw, int E, int N, int K, int n_pairs, const int32_t* sorted_ids,
                    const int32_t* tile_expert, const int32_t* tile_order, const int32_t* totals, int max_tiles, void* out,
                    int ldo, const float* row_scale, int out_dtype) {
  B200_REQUIRE(out_dtype == kBF16 || out_dtype == kF16, "the fp8 grouped gemm writes bf16 or f16");
  B200_REQUIRE(K % kFK == 0 && K > 0, "K (%d) must be a positive multiple of 128 (one scale per 128 channels)", K);
  B200_REQUIRE(N % 8 == 0 && N > 0, "N (%d) must be a positive multiple of 8", N);
  B200_REQUIRE(lda % 16 == 0 && (reinterpret_cast<uintptr_t>(A8) & 15u) == 0, "A rows must be 16-byte aligned");
  B200_REQUIRE(a_div >= 1 && max_tiles >= 1, "bad a_div / max_tiles");
  memset(&p, 0, sizeof(p));
  p.N = N; p.K = K; p.n_pairs = n_pairs; p.a_div = a_div; p.lda = lda; p.ldo = ldo;
  p.tiles_n = (N + kFN - 1) / kFN;
  p.max_tiles = max_tiles;
  p.num_kb = K / kFK;
  p.sa_ld = sa_ld;
  p.bf16 = out_dtype == kBF16;
  p.A = static_cast<const uint8_t*>(A8); p.sa = sa; p.sw = sw;
  p.sorted_ids = sorted_ids; p.tile_expert = tile_expert; p.tile_order = tile_order; p.totals = totals;
  p.out = out; p.row_scale = row_scale;
  return make_tma_3d(tw, W8, kE4M3, K, N, E, K, static_cast<uint64_t>(N) * K, kFK, kFN, 1, true);
}

template <int kMode>
static int fp8_launch(const CUtensorMap& tw, const Fp8GroupedParams& p, const SymmCtx& ctx, int grid, uint32_t* status,
                      cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(grouped_gemm_fp8_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem));
    configured[dev & 63] = true;
  }
  if (kMode == kFRS) {  // grid barrier inside: cooperative launch
    B200_CHECK_CUDA(launch_cooperative(grouped_gemm_fp8_kernel<kMode>, dim3(grid), dim3(kFThreads), kFSmem, stream, tw, p, ctx,
                                       status));
    return kOk;
  }
  grouped_gemm_fp8_kernel<kMode><<<grid, kFThreads, kFSmem, stream>>>(tw, p, ctx, status);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace b200

using namespace b200;

// out[pair, :] = row_scale[pair] * sum_kb sa[pair / a_div, kb] * sw[e, n / 128, kb] * (A8[pair / a_div, kb] . W8[e, :, kb]^T)
// for the pairs listed in sorted_ids (tiles of 128 rows, one expert per tile, pad rows = n_pairs).
// A8 e4m3 rows with pitch lda bytes; sa fp32 [rows, sa_ld]; W8 e4m3 [E, N, K]; sw fp32 [E, ceil(N / 128), K / 128];
// out bf16 (dtype 0) or f16 (1) with pitch ldo elements. status (nullable) receives a non-zero code if a pipeline
// wait expired. K must be a multiple of 128 and N a multiple of 8.
B200_API int b200_grouped_gemm_fp8(const void* A8, int lda, const float* sa, int sa_ld, int a_div, const void* W8,
                                   const float* sw, int E, int N, int K, int n_pairs, const int32_t* sorted_ids,
                                   const int32_t* tile_expert, const int32_t* totals, int max_tiles, void* out, int ldo,
                                   const float* row_scale, int out_dtype, uint32_t* status, void* stream) {
  Fp8GroupedParams p;
  CUtensorMap tw;
  int rc = fp8_fill(p, &tw, A8, lda, sa, sa_ld, a_div, W8, sw, E, N, K, n_pairs, sorted_ids, tile_expert, nullptr, totals,
                    max_tiles, out, ldo, row_scale, out_dtype);
  if (rc != kOk) return rc;
  SymmCtx ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.world = 1;
  ctx.timeout_ns = 4000000000ull;
  int grid = sm_count();
  if (grid > max_tiles * p.tiles_n) grid = max_tiles * p.tiles_n;
  return fp8_launch<kFPlain>(tw, p, ctx, grid < 1 ? 1 : grid, status, static_cast<cudaStream_t>(stream));
}

// AG + fp8 grouped GEMM. a_local [Tr, lda bytes]: this rank's rows, each K e4m3 bytes followed by K / 128 fp32 scales
// (lda >= K + K / 32, a multiple of 16); ag_buf0 / ag_buf1: symmetric [world * Tr, lda] parity buffers; pairs index the
// gathered tokens (pair / topk = token). ready: symmetric u32[world]; rank_cnt, rank_flag: local u32[world]; sync:
// local u32[4]; all zero-initialised once.
B200_API int b200_ag_grouped_gemm_fp8(const void* symm_ctx, const void* a_local, int lda, void* ag_buf0, void* ag_buf1, int Tr,
                                      int topk, const void* W8, const float* sw, int E, int N, int K,
                                      const int32_t* sorted_ids, const int32_t* tile_expert, const int32_t* tile_order,
                                      const int32_t* totals, int max_tiles, void* out, int ldo, uint32_t* ready,
                                      uint32_t* rank_cnt, uint32_t* rank_flag, uint32_t* sync, int out_dtype, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(lda >= K + K / 32, "row pitch (%d) must hold K (%d) bytes and K / 128 fp32 scales", lda, K);
  Fp8GroupedParams p;
  CUtensorMap tw;
  const int n_pairs = Tr * ctx.world * topk;
  int rc = fp8_fill(p, &tw, a_local, lda, nullptr, 0, topk, W8, sw, E, N, K, n_pairs, sorted_ids, tile_expert, tile_order,
                    totals, max_tiles, out, ldo, nullptr, out_dtype);
  if (rc != kOk) return rc;
  p.a_local = static_cast<const uint8_t*>(a_local);
  p.ag_buf[0] = static_cast<uint8_t*>(ag_buf0); p.ag_buf[1] = static_cast<uint8_t*>(ag_buf1);
  p.ready = ready; p.rank_cnt = rank_cnt; p.rank_flag = rank_flag; p.sync = sync; p.Tr = Tr;
  return fp8_launch<kFAG>(tw, p, ctx, sm_count(), nullptr, static_cast<cudaStream_t>(stream));
}

// fp8 grouped GEMM + topk-reduce + reduce-scatter: A8 [n_pairs, lda] (row per pair) with scales sa [n_pairs, sa_ld],
// W8 [E, N, K_local] with block scales sw, row_scale [n_pairs] routing weights, gemm_out [n_pairs, N] local scratch,
// rs_out [Tr, N]. Buffers as in b200_grouped_gemm_rs.
B200_API int b200_grouped_gemm_fp8_rs(const void* symm_ctx, const void* A8, int lda, const float* sa, int sa_ld,
                                      const void* W8, const float* sw, int E, int N, int K, int Tr, int topk,
                                      const int32_t* sorted_ids, const int32_t* tile_expert, const int32_t* tile_order,
                                      const int32_t* totals, int max_tiles, const float* row_scale, void* gemm_out,
                                      void* slots0, void* slots1, int Tr_cap, uint32_t* rs_cnt, uint32_t* rs_base,
                                      uint32_t* sync, void* rs_out, int out_dtype, int nvls, void* stream) {
  SymmCtx ctx;
  memcpy(&ctx, symm_ctx, sizeof(ctx));
  B200_REQUIRE(Tr <= Tr_cap, "tokens per rank (%d) exceed the context capacity (%d)", Tr, Tr_cap);
  B200_REQUIRE(!nvls || ctx.mc_base != 0, "the in-switch reduction needs an NVLS multicast mapping");
  Fp8GroupedParams p;
  CUtensorMap tw;
  const int n_pairs = Tr * ctx.world * topk;
  int rc = fp8_fill(p, &tw, A8, lda, sa, sa_ld, 1, W8, sw, E, N, K, n_pairs, sorted_ids, tile_expert, tile_order, totals,
                    max_tiles, gemm_out, N, row_scale, out_dtype);
  if (rc != kOk) return rc;
  p.sync = sync; p.Tr = Tr; p.topk = topk; p.Tr_cap = Tr_cap;
  p.slots[0] = slots0; p.slots[1] = slots1; p.rs_cnt = rs_cnt; p.rs_base = rs_base; p.rs_out = rs_out;
  p.rs_nvls = nvls ? 1 : 0;
  return fp8_launch<kFRS>(tw, p, ctx, sm_count(), nullptr, static_cast<cudaStream_t>(stream));
}
