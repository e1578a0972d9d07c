// Shared host/device helpers for liblucid_cuda (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lucid_cuda.h"

namespace lc {

// ---- host side: error text and launch checking ---------------------------
void set_error(const char* fmt, ...);
int32_t fail(int32_t code, const char* fmt, ...);
int32_t check_launch(const char* what);
int sm_count();  // SM count of the current device (cached per device)

// 2-D tiled TMA descriptor: `inner` x `rows` elements of `dtype`, rows `stride_bytes` apart, box
// `box_inner` x `box_rows`, out-of-bounds elements read as zero.  The driver entry point is
// looked up through the runtime, so the library does not link against libcuda.
int32_t encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                             uint64_t rows, uint64_t stride_bytes, uint32_t box_inner, uint32_t box_rows,
                             CUtensorMapSwizzle swizzle);

// GEMV-shaped int8 x int8 product for up to 32 rows against a weight of 4 MB and more (qgemv_kernels.cu): same
// arguments and bit-identical results as the tensor-core GEMM behind lc_qlinear_i8
bool qgemv_i8_applies(int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, const void* a, const void* b,
                      int32_t out_dtype);
int32_t launch_qgemv_i8(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b, int64_t ldb, int64_t M,
                        int64_t N, int64_t K, const float* sx, int32_t sx_per_row, const float* zx, const int32_t* wsum,
                        const float* sw, const float* bias, void* out, int32_t out_dtype, int64_t ldo, int32_t* status,
                        cudaStream_t st);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- programmatic dependent launch ----------------------------------------------------
// A kernel launched with launch_overlapped() may be scheduled while the kernel before it on the
// stream is still running; it must execute pdl_wait() before it reads anything that kernel
// wrote or writes anything that kernel reads (the wait returns when that grid has completed
// and its memory is visible).  What precedes the wait may only touch the kernel's own shared
// memory, TMEM and registers.  pdl_launch_dependents() in the earlier kernel lets the next
// grid take SM resources as they free up instead of after this grid has drained; it is a
// no-op when nothing overlapped is queued.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename Kernel, typename... Args>
inline cudaError_t launch_overlapped(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// ---- device side: the quantization grid, one IEEE fp32 step at a time ------
// The reference evaluates round(x * (1/s)) + z as separate eager fp32 ops
// (lucid/quantization/_functional.py:59-69); the explicit _rn intrinsics stop
// the compiler from contracting the multiply and the add into an FMA.
__device__ __forceinline__ float grid_code(float x, float inv, float z) {
  return __fadd_rn(rintf(__fmul_rn(x, inv)), z);
}

// clip(code, qmin, qmax) followed by the reference's saturating float->int
// cast, which maps NaN to 0 (lucid/_C/backend/cpu/methods/Factory.cpp:103-135).
__device__ __forceinline__ int code_to_int(float c, float qmin, float qmax) {
  float cl = fminf(fmaxf(c, qmin), qmax);
  return (c != c) ? 0 : __float2int_rn(cl);
}

// fake_quantize of one value onto a per-tensor grid: (clip(round(x * inv) + z) - z) * s, NaN
// passing through (lucid/quantization/_functional.py:326-333); inv = 1 / s by IEEE division.
__device__ __forceinline__ float fake_quant_value(float x, float s, float inv, float z, float qmin, float qmax) {
  const float pre = grid_code(x, inv, z);
  const float q = (pre != pre) ? pre : fminf(fmaxf(pre, qmin), qmax);
  return __fmul_rn(__fsub_rn(q, z), s);
}

// Fast path for grids that coincide with the storage type's own range (qint8 [-128,127] in
// int8, [0,255] in uint8): the float->int conversion rounds to nearest even and the packing
// instruction saturates, so clip + cast cost nothing extra; NaN converts to 0 as the
// reference's cast does.  `t` values are x * inv; with a zero-point the code is rint(t) + z
// (rounded first, then shifted, as the reference does), which is integral, so converting it
// again changes nothing.  cvt.pack: d = (c << 16) | (sat(a) << 8) | sat(b).
template <bool UNSIGNED>
__device__ __forceinline__ uint32_t pack4_sat(float t0, float t1, float t2, float t3, float z, bool has_z) {
  if (has_z) {
    t0 = __fadd_rn(rintf(t0), z);
    t1 = __fadd_rn(rintf(t1), z);
    t2 = __fadd_rn(rintf(t2), z);
    t3 = __fadd_rn(rintf(t3), z);
  }
  const int a = __float2int_rn(t0), b = __float2int_rn(t1), c = __float2int_rn(t2), d = __float2int_rn(t3);
  uint32_t hi, r;
  if (UNSIGNED) {
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
  } else {
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
  }
  return r;
}

// calculate_qparams for one (min, max) pair (lucid/quantization/_qparams.py:186-205).
// The host fills the constants exactly as the reference's Python does:
// half = (qmax-qmin)/2.0 and range = qmax-qmin rounded once to fp32,
// sym_zp = 0 for a signed grid else (qmax+qmin+1)//2.
struct QParamSpec {
  int symmetric;
  float half;
  float sym_zp;
  float range;
  float qmin;
  float qmax;
  float eps;
};

inline QParamSpec make_qparam_spec(int symmetric, int quant_min, int quant_max, int is_signed,
                                   float eps) {
  QParamSpec sp;
  sp.symmetric = symmetric;
  sp.half = static_cast<float>((static_cast<double>(quant_max) - static_cast<double>(quant_min)) / 2.0);
  long long mid = (static_cast<long long>(quant_max) + static_cast<long long>(quant_min) + 1);
  mid = (mid >= 0) ? mid / 2 : -((-mid + 1) / 2);  // floor division
  sp.sym_zp = is_signed ? 0.0f : static_cast<float>(mid);
  sp.range = static_cast<float>(static_cast<double>(quant_max) - static_cast<double>(quant_min));
  sp.qmin = static_cast<float>(quant_min);
  sp.qmax = static_cast<float>(quant_max);
  sp.eps = eps;
  return sp;
}

__device__ __forceinline__ void qparams_from_range(float mn, float mx, const QParamSpec& sp,
                                                   float& scale, float& zp) {
  mn = fminf(mn, 0.0f);
  mx = fmaxf(mx, 0.0f);
  if (sp.symmetric) {
    float max_abs = fmaxf(fabsf(mn), fabsf(mx));
    scale = fmaxf(__fdiv_rn(max_abs, sp.half), sp.eps);
    zp = sp.sym_zp;
  } else {
    scale = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), sp.range), sp.eps);
    float r = rintf(__fdiv_rn(mn, scale));
    zp = fminf(fmaxf(__fsub_rn(sp.qmin, r), sp.qmin), sp.qmax);
  }
}

// ---- warp / block reductions ----------------------------------------------
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide min and max; every thread returns the result.  `red` is 2*32 floats.
__device__ __forceinline__ void block_minmax(float& mn, float& mx, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  mn = warp_min(mn);
  mx = warp_max(mx);
  __syncthreads();  // protects `red` against a previous use
  if (lane == 0) {
    red[warp] = mn;
    red[32 + warp] = mx;
  }
  __syncthreads();
  float a = (lane < nwarps) ? red[lane] : INFINITY;
  float b = (lane < nwarps) ? red[32 + lane] : -INFINITY;
  mn = warp_min(a);
  mx = warp_max(b);
}

// float atomic min/max through integer atomics on the float's bit pattern
// (ordering of IEEE bit patterns: as signed int for >= 0, reversed as unsigned
// for < 0).  -0.0 is canonicalised to +0.0 first.
__device__ __forceinline__ void atomic_min_float(float* addr, float v) {
  v = v + 0.0f;
  if (v >= 0.0f)
    atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
  else
    atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  v = v + 0.0f;
  if (v >= 0.0f)
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else
    atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// ---- vector store of four codes -------------------------------------------
template <typename T>
struct Vec4;
template <>
struct Vec4<int8_t> {
  using type = char4;
};
template <>
struct Vec4<uint8_t> {
  using type = uchar4;
};
template <>
struct Vec4<int16_t> {
  using type = short4;
};
template <>
struct Vec4<int32_t> {
  using type = int4;
};

template <typename T>
__device__ __forceinline__ void store4(T* p, int a, int b, int c, int d) {
  typename Vec4<T>::type v;
  v.x = static_cast<decltype(v.x)>(a);
  v.y = static_cast<decltype(v.y)>(b);
  v.z = static_cast<decltype(v.z)>(c);
  v.w = static_cast<decltype(v.w)>(d);
  *reinterpret_cast<typename Vec4<T>::type*>(p) = v;
}
template <typename T>
__device__ __forceinline__ void load4(const T* p, int& a, int& b, int& c, int& d) {
  typename Vec4<T>::type v = *reinterpret_cast<const typename Vec4<T>::type*>(p);
  a = v.x;
  b = v.y;
  c = v.z;
  d = v.w;
}

}  // namespace lc
