// Operand preparation for the tensor-core weight-only Linear (lc_wo_gemm_16): int8 codes widened
// to a 16-bit float type once per weight, and fp32 activations split into three bf16 terms whose
// sum is the fp32 value.  Both are plain HBM-bound passes.
#include "common.cuh"

namespace lc {
namespace {

constexpr int kPrepThreads = 256;

template <typename T>
__device__ __forceinline__ T int_to_16(int v);
template <>
__device__ __forceinline__ __nv_bfloat16 int_to_16<__nv_bfloat16>(int v) {
  return __float2bfloat16_rn(static_cast<float>(v));  // |v| <= 128: exact
}
template <>
__device__ __forceinline__ __half int_to_16<__half>(int v) {
  return __float2half_rn(static_cast<float>(v));
}

// one thread per 16 output elements (16 bytes in, 32 bytes out); the padding columns are zeros
template <typename T, bool VEC>
__global__ void __launch_bounds__(kPrepThreads)
widen_s8_kernel(const int8_t* __restrict__ q, int64_t rows, int64_t cols, int64_t ld_in, T* __restrict__ out,
                int64_t ld_out) {
  const int64_t per_row = (ld_out + 15) / 16;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * kPrepThreads + threadIdx.x;
  if (item >= rows * per_row) return;
  const int64_t r = item / per_row, c0 = (item % per_row) * 16;
  T v[16];
  if (VEC && c0 + 16 <= cols) {
    const int4 raw = __ldg(reinterpret_cast<const int4*>(q + r * ld_in + c0));
    const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = int_to_16<T>(b[e]);
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = int_to_16<T>(c0 + e < cols ? q[r * ld_in + c0 + e] : 0);
  }
  T* o = out + r * ld_out + c0;
  if (VEC && c0 + 16 <= ld_out) {
    reinterpret_cast<uint4*>(o)[0] = reinterpret_cast<const uint4*>(v)[0];
    reinterpret_cast<uint4*>(o)[1] = reinterpret_cast<const uint4*>(v)[1];
  } else {
    for (int e = 0; e < 16; ++e)
      if (c0 + e < ld_out) o[e] = v[e];
  }
}

__device__ __forceinline__ void split3(float x, __nv_bfloat16& a, __nv_bfloat16& b, __nv_bfloat16& c) {
  a = __float2bfloat16_rn(x);
  const float r1 = __fsub_rn(x, __bfloat162float(a));   // exact: the low bits of x
  b = __float2bfloat16_rn(r1);
  const float r2 = __fsub_rn(r1, __bfloat162float(b));  // exact
  c = __float2bfloat16_rn(r2);
}

// one CTA per row: 4 elements per thread and step, the three terms written as 8-byte stores
template <bool VEC>
__global__ void __launch_bounds__(kPrepThreads)
split_f32_bf16x3_kernel(const float* __restrict__ x, int64_t cols, int64_t ldx, __nv_bfloat16* __restrict__ terms,
                        int64_t kp, float* __restrict__ rowsum) {
  __shared__ float red[kPrepThreads / 32];
  const int64_t r = blockIdx.x;
  const float* xr = x + r * ldx;
  __nv_bfloat16* t0 = terms + r * 3 * kp;
  float sum = 0.0f;
  for (int64_t k = static_cast<int64_t>(threadIdx.x) * 4; k < kp; k += kPrepThreads * 4) {
    float v[4];
    if (VEC && k + 4 <= cols) {
      const float4 f = __ldcs(reinterpret_cast<const float4*>(xr + k));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = k + e < cols ? xr[k + e] : 0.0f;
    }
    __nv_bfloat16 a[4], b[4], c[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      split3(v[e], a[e], b[e], c[e]);
      sum += v[e];
    }
    *reinterpret_cast<uint2*>(t0 + k) = *reinterpret_cast<const uint2*>(a);
    *reinterpret_cast<uint2*>(t0 + kp + k) = *reinterpret_cast<const uint2*>(b);
    *reinterpret_cast<uint2*>(t0 + 2 * kp + k) = *reinterpret_cast<const uint2*>(c);
  }
  if (rowsum) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f;
      for (int w = 0; w < kPrepThreads / 32; ++w) s += red[w];
      rowsum[r] = s;
    }
  }
}

// fp32 row -> four signed base-256 digit planes of round(x * 2^e), 2^e the power of two that puts the
// row's largest magnitude into [2^29, 2^30).  One team of threads per row: pass 1 finds the maximum,
// pass 2 re-reads the row (from L1/L2) and writes the digits of 4 elements as one 4-byte store per plane.
// Plane d of row m = 32t + r lives in row 128t + 32d + r of `digits`: the digit planes of 32 rows
// make up one 128-row GEMM tile, plane d in accumulator lanes 32d .. 32d+31.
template <bool VEC, int TEAM>
__global__ void __launch_bounds__(kPrepThreads)
split_f32_digits_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, int64_t ldx,
                        int8_t* __restrict__ digits, int64_t ldd, float* __restrict__ row_scale,
                        float* __restrict__ rowsum) {
  // TEAM threads share a row: a whole CTA for long rows, one warp (8 rows per CTA) for short ones
  static_assert(TEAM == 32 || TEAM == kPrepThreads, "a warp or the whole CTA per row");
  constexpr int kTeams = kPrepThreads / TEAM;
  __shared__ float red[2 * (kPrepThreads / 32)];
  __shared__ float s_mul;
  const int team = threadIdx.x / TEAM, tid = threadIdx.x % TEAM;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kTeams + team;
  const bool row_ok = r < rows;
  const float* xr = x + (row_ok ? r : 0) * ldx;
  float mx = 0.0f, sum = 0.0f;
  bool bad = false;
  if (row_ok) {
    for (int64_t k = static_cast<int64_t>(tid) * 4; k < cols; k += TEAM * 4) {
      float v[4];
      if (VEC && k + 4 <= cols) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(xr + k));
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = k + e < cols ? xr[k + e] : 0.0f;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mx = fmaxf(mx, fabsf(v[e]));
        bad |= !(fabsf(v[e]) <= 3.402823466e38f);  // NaN or infinity
        sum += v[e];
      }
    }
  }
  if (bad) mx = INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
  }
  if (TEAM != 32) {
    if ((threadIdx.x & 31) == 0) {
      red[threadIdx.x >> 5] = mx;
      red[kPrepThreads / 32 + (threadIdx.x >> 5)] = sum;
    }
    __syncthreads();
    mx = 0.0f;
    sum = 0.0f;
    for (int w = 0; w < kPrepThreads / 32; ++w) {
      mx = fmaxf(mx, red[w]);
      sum += red[kPrepThreads / 32 + w];
    }
  }
  // mx = f * 2^ex with f in [0.5, 1): x * 2^(30 - ex) has magnitude below 2^30.  A non-finite row gets
  // a NaN scale (its outputs become NaN); an all-zero row any scale.  e is capped so that 2^e and
  // 2^-e stay normal numbers.
  float mul = 1.0f, inv = 1.0f;
  if (mx > 3.402823466e38f) {
    mul = 0.0f;
    inv = __int_as_float(0x7fc00000);
  } else if (mx > 0.0f) {
    int ex = 0;
    frexpf(mx, &ex);
    int e = 30 - ex;
    e = e > 126 ? 126 : e;
    mul = __int_as_float((127 + e) << 23);
    inv = __int_as_float((127 - e) << 23);
  }
  (void)s_mul;
  if (!row_ok) return;
  if (tid == 0) {
    row_scale[r] = inv;
    if (rowsum) rowsum[r] = sum;
  }
  int8_t* base = digits + ((r >> 5) * 128 + (r & 31)) * ldd;
  for (int64_t k = static_cast<int64_t>(tid) * 4; k < ldd; k += TEAM * 4) {
    float v[4];
    if (VEC && k + 4 <= cols) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(xr + k));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = k + e < cols ? xr[k + e] : 0.0f;
    }
    uint32_t plane[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int X = __float2int_rn(__fmul_rn(v[e], mul));  // the product is exact: mul is a power of two
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        const int digit = ((X + 128) & 255) - 128;  // signed digit in [-128, 127]
        plane[d] |= static_cast<uint32_t>(digit & 255) << (8 * e);
        X = (X - digit) >> 8;                        // exact: X - digit is a multiple of 256
      }
    }
#pragma unroll
    for (int d = 0; d < 4; ++d) *reinterpret_cast<uint32_t*>(base + static_cast<int64_t>(d) * 32 * ldd + k) = plane[d];
  }
}

}  // namespace
}  // namespace lc

using namespace lc;

extern "C" int32_t lc_widen_s8(const int8_t* q, int64_t rows, int64_t cols, int64_t ld_in, void* out,
                               int32_t out_dtype, int64_t ld_out, void* stream) {
  if (rows < 0 || cols <= 0 || ld_in < cols || ld_out < cols) return fail(LC_ERR_INVALID_ARG, "widen_s8: bad shape");
  if (rows == 0) return LC_OK;
  if (!q || !out) return fail(LC_ERR_INVALID_ARG, "widen_s8: null pointer");
  if (out_dtype != LC_BF16 && out_dtype != LC_F16)
    return fail(LC_ERR_UNSUPPORTED, "widen_s8: out_dtype must be bf16 or f16, got %d", out_dtype);
  const bool vec = ld_in % 16 == 0 && ld_out % 8 == 0 && aligned(q, 16) && aligned(out, 16);
  const int64_t items = rows * ((ld_out + 15) / 16);
  const unsigned grid = static_cast<unsigned>((items + kPrepThreads - 1) / kPrepThreads);
  cudaStream_t st = as_stream(stream);
#define LC_WIDEN(T)                                                                                             \
  (vec ? widen_s8_kernel<T, true><<<grid, kPrepThreads, 0, st>>>(q, rows, cols, ld_in, static_cast<T*>(out), ld_out) \
       : widen_s8_kernel<T, false><<<grid, kPrepThreads, 0, st>>>(q, rows, cols, ld_in, static_cast<T*>(out), ld_out))
  if (out_dtype == LC_BF16)
    LC_WIDEN(__nv_bfloat16);
  else
    LC_WIDEN(__half);
#undef LC_WIDEN
  return check_launch("widen_s8");
}

extern "C" int32_t lc_split_f32_bf16x3(const float* x, int64_t rows, int64_t cols, int64_t ldx, void* terms,
                                       int64_t kp, float* rowsum, void* stream) {
  if (rows < 0 || cols <= 0 || ldx < cols || kp < cols || kp % 64)
    return fail(LC_ERR_INVALID_ARG, "split_f32_bf16x3: bad shape (kp must be a multiple of 64 and >= cols)");
  if (rows == 0) return LC_OK;
  if (!x || !terms) return fail(LC_ERR_INVALID_ARG, "split_f32_bf16x3: null pointer");
  if (rows > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "split_f32_bf16x3: too many rows");
  if (!aligned(terms, 8)) return fail(LC_ERR_UNSUPPORTED, "split_f32_bf16x3: terms must be 8-byte aligned");
  const bool vec = ldx % 4 == 0 && aligned(x, 16);
  cudaStream_t st = as_stream(stream);
  __nv_bfloat16* t = static_cast<__nv_bfloat16*>(terms);
  if (vec)
    split_f32_bf16x3_kernel<true><<<static_cast<unsigned>(rows), kPrepThreads, 0, st>>>(x, cols, ldx, t, kp, rowsum);
  else
    split_f32_bf16x3_kernel<false><<<static_cast<unsigned>(rows), kPrepThreads, 0, st>>>(x, cols, ldx, t, kp, rowsum);
  return check_launch("split_f32_bf16x3");
}

extern "C" int64_t lc_wo_digit_rows(int64_t rows) { return rows <= 0 ? 0 : (rows + 31) / 32 * 128; }

extern "C" int32_t lc_split_f32_digits(const float* x, int64_t rows, int64_t cols, int64_t ldx, int8_t* digits,
                                       int64_t ldd, float* row_scale, float* rowsum, void* stream) {
  if (rows < 0 || cols <= 0 || ldx < cols || ldd < cols || ldd % 16)
    return fail(LC_ERR_INVALID_ARG, "split_f32_digits: bad shape (ldd must be a multiple of 16 and >= cols)");
  if (rows == 0) return LC_OK;
  if (!x || !digits || !row_scale) return fail(LC_ERR_INVALID_ARG, "split_f32_digits: null pointer");
  if (rows > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "split_f32_digits: too many rows");
  if (!aligned(digits, 4)) return fail(LC_ERR_UNSUPPORTED, "split_f32_digits: digits must be 4-byte aligned");
  const bool vec = ldx % 4 == 0 && aligned(x, 16);
  cudaStream_t st = as_stream(stream);
  // a warp per row while a row is at most 16 elements per lane and step (2048 columns), else a CTA per row
  const bool warp_rows = cols <= 2048;
  const unsigned grid = static_cast<unsigned>(warp_rows ? (rows + kPrepThreads / 32 - 1) / (kPrepThreads / 32) : rows);
#define LC_SPLIT(V, T) \
  split_f32_digits_kernel<V, T><<<grid, kPrepThreads, 0, st>>>(x, rows, cols, ldx, digits, ldd, row_scale, rowsum)
  if (vec) {
    if (warp_rows) LC_SPLIT(true, 32); else LC_SPLIT(true, kPrepThreads);
  } else {
    if (warp_rows) LC_SPLIT(false, 32); else LC_SPLIT(false, kPrepThreads);
  }
#undef LC_SPLIT
  return check_launch("split_f32_digits");
}
