// Host-side helpers shared by every launcher in this library: error reporting, lazily resolved
// driver entry points (the library never links libcuda, so it also loads on a machine without a
// driver), TMA descriptor construction and per-device one-time kernel attribute set-up.
//
// Role in the reference: the generated C launchers and the AOT runtime
// (python/triton_dist/tools/runtime/triton_aot_runtime.cc:24-314, backends/nvidia/backend/driver.py:260-339).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace b200 {

// Negative return codes of the C API. Positive values are cudaError_t / CUresult codes.
enum ApiError : int {
  kOk = 0,
  kErrBadArgument = -1,
  kErrDriverUnavailable = -2,
  kErrUnsupported = -3,
  kErrOutOfHeap = -4,
  kErrSocket = -5,
  kErrTimeout = -6,
};

// printf-style; stores the message for b200_last_error() (thread local) and returns `code`.
int set_error(int code, const char* fmt, ...);

#define B200_CHECK_CUDA(expr)                                                                       \
  do {                                                                                              \
    cudaError_t _e = (expr);                                                                        \
    if (_e != cudaSuccess)                                                                          \
      return ::b200::set_error(static_cast<int>(_e), "%s failed: %s (%s:%d)", #expr,                \
                               cudaGetErrorString(_e), __FILE__, __LINE__);                         \
  } while (0)

#define B200_CHECK_CU(expr)                                                                         \
  do {                                                                                              \
    CUresult _r = (expr);                                                                           \
    if (_r != CUDA_SUCCESS)                                                                         \
      return ::b200::set_error(static_cast<int>(_r), "%s failed: CUresult %d (%s:%d)", #expr,       \
                               static_cast<int>(_r), __FILE__, __LINE__);                           \
  } while (0)

#define B200_REQUIRE(cond, ...)                                                                     \
  do {                                                                                              \
    if (!(cond)) return ::b200::set_error(::b200::kErrBadArgument, __VA_ARGS__);                    \
  } while (0)

// Driver entry points resolved through cudaGetDriverEntryPoint on first use.
struct DriverApi {
  bool ok = false;
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                           unsigned long long);
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long);
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*cuDeviceGet)(CUdevice*, int);
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  CUresult (*cuStreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  CUresult (*cuStreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
};
// Returns nullptr (after set_error) when no driver is present.
const DriverApi* driver();

// Element kinds understood by the launchers (values are part of the C ABI).
enum DType : int { kBF16 = 0, kF16 = 1, kF32 = 2, kE4M3 = 3, kU8 = 4, kI32 = 5 };
inline int dtype_size(int dt) {
  switch (dt) {
    case kBF16: case kF16: return 2;
    case kF32: case kI32: return 4;
    default: return 1;
  }
}

// 2-D row-major tensor [rows, cols] with `ld` elements between rows, tiled into boxes of
// [box_rows, box_cols] with the 128-byte swizzle (box_cols * elem_size must equal 128 bytes) or
// without swizzle (swizzle128 = false). Out-of-range elements read as zero.
int make_tma_2d(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld,
                uint32_t box_rows, uint32_t box_cols, bool swizzle128);
// 3-D tensor [d2, d1, d0] (d0 innermost) with element strides s2, s1 (s0 = 1).
int make_tma_3d(CUtensorMap* map, const void* base, int dtype, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128);

// Number of SMs of the current device (cached per device).
int sm_count();

// Whether kernels of the decode path are launched with programmatic stream serialization (on unless
// B200DIST_PDL=0): the next kernel's CTAs may start their prologue while this one drains.
bool pdl_enabled();

// Launch with the programmatic-dependent-launch attribute. The kernel must execute griddep_wait() before it reads
// anything an earlier kernel wrote or writes anything an earlier kernel may still read.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Cooperative launch: the driver refuses the launch unless every CTA of the grid can be resident at once, which is
// what a kernel that contains a grid-wide barrier relies on (a plain launch would only assume it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cooperative(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
  cudaLaunchConfig_t cfg;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200
