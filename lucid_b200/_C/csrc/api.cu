// Library-level entry points and the host helpers shared by all kernels files.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace lc {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int32_t check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(LC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return LC_OK;
}

// Read-only after its first fill per device, so concurrent callers are safe.
int sm_count() {
  constexpr int kMaxDevices = 64;
  static int counts[kMaxDevices] = {0};
  static std::once_flag flags[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::call_once(flags[dev], [dev]() {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    counts[dev] = n;
  });
  return counts[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      cudaGetLastError();
  });
  return fn;
}

int32_t encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                             uint64_t rows, uint64_t stride_bytes, uint32_t box_inner, uint32_t box_rows,
                             CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(LC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LC_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LC_OK;
}

}  // namespace lc

extern "C" int32_t lc_version(void) { return 100; }

extern "C" int32_t lc_last_error(char* host_buf, int32_t n) {
  if (!host_buf || n <= 0) return LC_ERR_INVALID_ARG;
  strncpy(host_buf, lc::g_error, static_cast<size_t>(n));
  host_buf[n - 1] = '\0';
  return LC_OK;
}

extern "C" int32_t lc_device_info(int32_t device, int32_t* host_sm, int32_t* host_sm_count) {
  int major = 0, minor = 0, sms = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    cudaGetLastError();
    return lc::fail(LC_ERR_CUDA, "device %d is not usable", device);
  }
  if (host_sm) *host_sm = major * 10 + minor;
  if (host_sm_count) *host_sm_count = sms;
  return LC_OK;
}

extern "C" int32_t lc_stream_capture_id(void* stream, uint64_t* host_id) {
  if (!host_id) return lc::fail(LC_ERR_INVALID_ARG, "stream_capture_id: null pointer");
  cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
  unsigned long long id = 0;
  if (cudaStreamGetCaptureInfo(reinterpret_cast<cudaStream_t>(stream), &status, &id) != cudaSuccess)
    return lc::fail(LC_ERR_CUDA, "stream_capture_id: %s", cudaGetErrorString(cudaGetLastError()));
  *host_id = status == cudaStreamCaptureStatusActive ? static_cast<uint64_t>(id) : 0;
  return LC_OK;
}
