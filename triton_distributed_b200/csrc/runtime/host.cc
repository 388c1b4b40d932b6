// Error reporting, driver entry-point resolution and TMA descriptor construction.
#include "b200/host.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b200 {

static thread_local char g_err[1024] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

template <typename F>
static bool resolve(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

const DriverApi* driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
#define R(name) ok = resolve(api.name, #name) && ok
    R(cuMemCreate);
    R(cuMemRelease);
    R(cuMemAddressReserve);
    R(cuMemAddressFree);
    R(cuMemMap);
    R(cuMemUnmap);
    R(cuMemSetAccess);
    R(cuMemGetAllocationGranularity);
    R(cuMemExportToShareableHandle);
    R(cuMemImportFromShareableHandle);
    R(cuMulticastCreate);
    R(cuMulticastAddDevice);
    R(cuMulticastBindMem);
    R(cuMulticastUnbind);
    R(cuMulticastGetGranularity);
    R(cuDeviceGet);
    R(cuDeviceGetAttribute);
    R(cuTensorMapEncodeTiled);
    R(cuStreamWriteValue32);
    R(cuStreamWaitValue32);
#undef R
    api.ok = ok;
  });
  if (!api.ok) {
    set_error(kErrDriverUnavailable, "CUDA driver entry points could not be resolved (no driver on this machine?)");
    return nullptr;
  }
  return &api;
}

static CUtensorMapDataType tma_dtype(int dt) {
  switch (dt) {
    case kBF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case kF16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case kF32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case kI32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

int make_tma_2d(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld,
                uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  const uint64_t es = dtype_size(dtype);
  B200_REQUIRE((reinterpret_cast<uint64_t>(base) & 15u) == 0, "TMA base address %p is not 16-byte aligned", base);
  B200_REQUIRE((ld * es) % 16 == 0, "TMA row pitch %llu bytes is not a multiple of 16",
               static_cast<unsigned long long>(ld * es));
  B200_REQUIRE(box_rows <= 256 && box_cols <= 256, "TMA box %ux%u exceeds 256", box_rows, box_cols);
  B200_REQUIRE(!swizzle128 || box_cols * es == 128, "128-byte swizzle needs a 128-byte inner box, got %llu",
               static_cast<unsigned long long>(box_cols * es));
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * es};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  B200_CHECK_CU(d->cuTensorMapEncodeTiled(map, tma_dtype(dtype), 2, const_cast<void*>(base), dims, strides, box, estr,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return kOk;
}

int make_tma_3d(CUtensorMap* map, const void* base, int dtype, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128) {
  const DriverApi* d = driver();
  if (!d) return kErrDriverUnavailable;
  const uint64_t es = dtype_size(dtype);
  B200_REQUIRE((reinterpret_cast<uint64_t>(base) & 15u) == 0, "TMA base address %p is not 16-byte aligned", base);
  B200_REQUIRE((s1 * es) % 16 == 0 && (s2 * es) % 16 == 0, "TMA strides must be multiples of 16 bytes");
  B200_REQUIRE(!swizzle128 || b0 * es == 128, "128-byte swizzle needs a 128-byte inner box");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * es, s2 * es};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  B200_CHECK_CU(d->cuTensorMapEncodeTiled(map, tma_dtype(dtype), 3, const_cast<void*>(base), dims, strides, box, estr,
                                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return kOk;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool pdl_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("B200DIST_PDL");
    cached = (e && e[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

}  // namespace b200

B200_API const char* b200_last_error() { return b200::g_err; }
B200_API int b200_sm_count() { return b200::sm_count(); }
B200_API int b200_driver_available() { return b200::driver() != nullptr ? 1 : 0; }
