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
// Role in the reference: the fp8 path of the expert-parallel MoE inference test
// (python/triton_dist/test/nvidia/test_ep_moe_inference.py:169-327) and the grouped GEMM mainloops
// (kernels/nvidia/allgather_group_gemm.py:531-605), which run block-scaled fp8 through Triton's dot.
#include "b200/host.h"
#include "b200/primitives.cuh"
#include "b200/tcgen05.cuh"

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
};

__device__ __forceinline__ void f8_cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void f8_cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void f8_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__global__ void __launch_bounds__(kFThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const Fp8GroupedParams p, const uint64_t timeout_ns,
                        uint32_t* status) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = min(p.totals[1], p.max_tiles);
  const int total_work = num_tiles * p.tiles_n;

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
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ------------------------------------------------------------------ W producer (TMA)
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int tile = w / p.tiles_n, n_blk = w - tile * p.tiles_n;
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
  }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ promotion + epilogue warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int w4 = warp - 4;  // == warp % 4: the TMEM lane quarter this warp may read
    uint8_t* stg = epi_smem + w4 * (32 * 128);
    uint32_t pcount = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const int tile = w / p.tiles_n, n_blk = w - tile * p.tiles_n;
      const int e = p.tile_expert[tile];
      const int my_pair = p.sorted_ids[tile * kFM + w4 * 32 + lane];
      const bool valid = my_pair < p.n_pairs;
      const float my_rs = (p.row_scale && valid) ? p.row_scale[my_pair] : 1.f;
      const float* sa_row = p.sa + static_cast<size_t>(valid ? my_pair / p.a_div : 0) * p.sa_ld;
      const float* sw_row = p.sw + (static_cast<size_t>(e) * p.tiles_n + n_blk) * p.num_kb;
      float acc[kFN];
#pragma unroll
      for (int j = 0; j < kFN; ++j) acc[j] = 0.f;
      float s_next = valid ? sa_row[0] * sw_row[0] : 0.f;
      for (int kb = 0; kb < p.num_kb; ++kb, ++pcount) {
        const uint32_t pb = pcount & 1, pphase = (pcount >> 1) & 1;
        const float s = s_next;
        if (kb + 1 < p.num_kb) s_next = valid ? sa_row[kb + 1] * sw_row[kb + 1] : 0.f;  // in flight during the wait
        if (!mbar_wait(pfull_bar + pb, pphase, abort_flag, timeout_ns)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(w4 * 32) << 16) + pb * kFN;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + h * 64, r0);
          tmem_ld_32x32(taddr + h * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            acc[h * 64 + j] = fmaf(s, __uint_as_float(r0[j]), acc[h * 64 + j]);
            acc[h * 64 + 32 + j] = fmaf(s, __uint_as_float(r1[j]), acc[h * 64 + 32 + j]);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(pempty_bar + pb);
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
      const int tile = w / p.tiles_n;
      const uint8_t* rp[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int pair = p.sorted_ids[tile * kFM + rbase + 16 * i];
        rp[i] = pair < p.n_pairs ? p.A + static_cast<size_t>(pair / p.a_div) * p.lda + chunk * 16 : nullptr;
      }
      for (int kb = 0; kb < p.num_kb && ok; ++kb) {
        if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, timeout_ns)) { ok = false; break; }
        const uint32_t sa = smem_u32(smem + stage * kFStageBytes) + sw_off;
        const bool in_k = kb * kFK + chunk * 16 < p.K;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool in = rp[i] != nullptr && in_k;
          f8_cp_async16(sa + i * (16 * 128), in ? rp[i] + static_cast<size_t>(kb) * kFK : p.A, in ? 16 : 0);
        }
        f8_cp_async_arrive_noinc(full_bar + stage);
        if (++stage == kFStages) { stage = 0; phase ^= 1; }
      }
    }
    f8_cp_async_wait_all();
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, 256);
  if (threadIdx.x == 0 && *abort_flag != 0u && status != nullptr) atomicMax(status, static_cast<uint32_t>(kStatusPipeTimeout));
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
  B200_REQUIRE(out_dtype == kBF16 || out_dtype == kF16, "the fp8 grouped gemm writes bf16 or f16");
  B200_REQUIRE(K % kFK == 0 && K > 0, "K (%d) must be a positive multiple of 128 (one scale per 128 channels)", K);
  B200_REQUIRE(N % 8 == 0 && N > 0, "N (%d) must be a positive multiple of 8", N);
  B200_REQUIRE(lda % 16 == 0 && (reinterpret_cast<uintptr_t>(A8) & 15u) == 0, "A rows must be 16-byte aligned");
  B200_REQUIRE(a_div >= 1 && max_tiles >= 1, "bad a_div / max_tiles");
  Fp8GroupedParams p;
  memset(&p, 0, sizeof(p));
  p.N = N; p.K = K; p.n_pairs = n_pairs; p.a_div = a_div; p.lda = lda; p.ldo = ldo;
  p.tiles_n = (N + kFN - 1) / kFN;
  p.max_tiles = max_tiles;
  p.num_kb = K / kFK;
  p.sa_ld = sa_ld;
  p.bf16 = out_dtype == kBF16;
  p.A = static_cast<const uint8_t*>(A8); p.sa = sa; p.sw = sw;
  p.sorted_ids = sorted_ids; p.tile_expert = tile_expert; p.totals = totals;
  p.out = out; p.row_scale = row_scale;
  CUtensorMap tw;
  int rc = make_tma_3d(&tw, W8, kE4M3, K, N, E, K, static_cast<uint64_t>(N) * K, kFK, kFN, 1, true);
  if (rc != kOk) return rc;
  static bool configured[64] = {false};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(grouped_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem));
    configured[dev & 63] = true;
  }
  int grid = sm_count();
  if (grid > max_tiles * p.tiles_n) grid = max_tiles * p.tiles_n;
  grouped_gemm_fp8_kernel<<<grid < 1 ? 1 : grid, kFThreads, kFSmem, static_cast<cudaStream_t>(stream)>>>(
      tw, p, 4000000000ull, status);
  B200_CHECK_CUDA(cudaGetLastError());
  return kOk;
}
