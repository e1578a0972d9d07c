// HBM-bound kernels of the quantization path: range observers, calculate_qparams,
// quantize / dequantize / fake_quantize and the fused dynamic activation
// quantizers.  All arithmetic is IEEE fp32, one rounding per reference op.
//
// Work decomposition.  A tensor is seen as (outer, channels, inner).  When the
// contiguous run `inner` is long ("segment mode") one CTA handles one chunk of
// one segment, reads it with 128-bit loads, and takes its scale / zero-point
// once per CTA.  When `inner` is short ("strided mode", e.g. ch_axis = last)
// threads walk the flat tensor and derive the channel per element.
#include <mutex>

#include "common.cuh"

namespace lc {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;                           // float4 loads in flight per thread
constexpr int kChunk = kThreads * 4 * kUnroll;       // 4096 elements per CTA
constexpr int64_t kSegModeMinInner = 128;
constexpr int kMaxObserveCtas = 148 * 8;

// =========================================================================
// observers
// =========================================================================
struct TensorObserveScratch {
  unsigned int ticket;
  unsigned int pad[3];
  float part_min[kMaxObserveCtas];
  float part_max[kMaxObserveCtas];
};

// Global min/max.  Phase 1: grid-stride partial reduction per CTA.  Phase 2: the
// CTA that draws the last ticket folds the partials; nobody spins.  atomicInc
// wraps the ticket back to 0, so the scratch is reusable without a memset.
__global__ void __launch_bounds__(kThreads)
observe_tensor_kernel(const float* __restrict__ x, int64_t n, int vec_ok, float* min_out,
                      float* max_out, int accumulate, int with_qparams, QParamSpec spec,
                      float* scale_out, float* zp_out, TensorObserveScratch* ws) {
  pdl_launch_dependents();
  __shared__ float red[64];
  __shared__ int is_last;
  float mn = INFINITY, mx = -INFINITY;
  if (vec_ok) {
    const int64_t nvec = n >> 2;
    const float4* xv = reinterpret_cast<const float4*>(x);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
      float4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[u] = __ldg(xv + i + u * stride);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        mn = fminf(fminf(mn, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
        mx = fmaxf(fmaxf(mx, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
      }
    }
    for (; i < nvec; i += stride) {
      float4 v = __ldg(xv + i);
      mn = fminf(fminf(mn, fminf(v.x, v.y)), fminf(v.z, v.w));
      mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
    // scalar tail (n not a multiple of 4)
    for (int64_t t = (nvec << 2) + static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; t < n;
         t += stride) {
      float v = __ldg(x + t);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  } else {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; t < n; t += stride) {
      float v = __ldg(x + t);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
  }
  block_minmax(mn, mx, red);
  if (threadIdx.x == 0) {
    ws->part_min[blockIdx.x] = mn;
    ws->part_max[blockIdx.x] = mx;
    __threadfence();
    unsigned int t = atomicInc(&ws->ticket, gridDim.x - 1);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  mn = INFINITY;
  mx = -INFINITY;
  for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += kThreads) {
    mn = fminf(mn, __ldcg(&ws->part_min[i]));
    mx = fmaxf(mx, __ldcg(&ws->part_max[i]));
  }
  block_minmax(mn, mx, red);
  if (threadIdx.x == 0) {
    if (accumulate) {
      mn = fminf(mn, *min_out);
      mx = fmaxf(mx, *max_out);
    }
    *min_out = mn;
    *max_out = mx;
    if (with_qparams) {
      float s, z;
      qparams_from_range(mn, mx, spec, s, z);
      *scale_out = s;
      *zp_out = z;
    }
  }
}

__global__ void fill_minmax_kernel(float* mn, float* mx, int64_t n) {
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    mn[i] = INFINITY;
    mx[i] = -INFINITY;
  }
}

// segment mode: CTA = one chunk of one (outer, channel) segment
template <bool VEC>
__global__ void __launch_bounds__(kThreads)
observe_channel_seg_kernel(const float* __restrict__ x, int64_t channels, int64_t inner,
                           int chunks_per_seg, float* min_out, float* max_out) {
  __shared__ float red[64];
  const int64_t seg = blockIdx.x / chunks_per_seg;
  const int chunk = blockIdx.x % chunks_per_seg;
  const int64_t c = seg % channels;
  const float* xs = x + seg * inner;
  const int64_t base = static_cast<int64_t>(chunk) * kChunk;
  float mn = INFINITY, mx = -INFINITY;
  if (VEC) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      v[u] = (i < inner) ? __ldg(reinterpret_cast<const float4*>(xs + i))
                         : make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) {
        mn = fminf(fminf(mn, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
        mx = fmaxf(fmaxf(mx, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
      }
    }
  } else {
#pragma unroll 4
    for (int u = 0; u < 4 * kUnroll; ++u) {
      int64_t i = base + static_cast<int64_t>(u) * kThreads + threadIdx.x;
      if (i < inner) {
        float v = __ldg(xs + i);
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
    }
  }
  block_minmax(mn, mx, red);
  if (threadIdx.x == 0) {
    atomic_min_float(min_out + c, mn);
    atomic_max_float(max_out + c, mx);
  }
}

// strided mode: the tensor is [outer, width] with width = channels*inner small;
// a thread owns one column of a row band, so loads stay coalesced.
__global__ void __launch_bounds__(kThreads)
observe_channel_strided_kernel(const float* __restrict__ x, int64_t outer, int64_t width,
                               int64_t inner, int rows_per_cta, float* min_out, float* max_out) {
  const int64_t col = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (col >= width) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_cta;
  int64_t r1 = r0 + rows_per_cta;
  if (r1 > outer) r1 = outer;
  float mn = INFINITY, mx = -INFINITY;
  for (int64_t r = r0; r < r1; ++r) {
    float v = __ldg(x + r * width + col);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  const int64_t c = col / inner;
  atomic_min_float(min_out + c, mn);
  atomic_max_float(max_out + c, mx);
}

__global__ void calculate_qparams_kernel(const float* mn, const float* mx, int64_t n,
                                         QParamSpec spec, float* scale, float* zp) {
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    float s, z;
    qparams_from_range(mn[i], mx[i], spec, s, z);
    scale[i] = s;
    zp[i] = z;
  }
}

// =========================================================================
// elementwise: quantize / dequantize / fake_quantize
// =========================================================================
struct ChannelParams {
  const float* scale;  // device, or nullptr -> host values
  const float* zp;
  int64_t n_scale;
  int64_t n_zp;
  float host_inv;
  float host_scale;
  float host_zp;
};

__device__ __forceinline__ void load_params(const ChannelParams& p, int64_t c, float& s, float& inv,
                                            float& z) {
  if (p.scale) {
    s = __ldg(p.scale + (p.n_scale == 1 ? 0 : c));
    inv = __fdiv_rn(1.0f, s);  // the reference's `1.0 / s` on a tensor scale
  } else {
    s = p.host_scale;
    inv = p.host_inv;
  }
  z = p.zp ? __ldg(p.zp + (p.n_zp == 1 ? 0 : c)) : p.host_zp;
}

// segment mode.  `in_stride` / `out_stride` are the distances between segment
// starts (== inner for dense tensors; a padded leading dimension otherwise).
// `reverse` walks the CTAs from the end of the tensor: after a full-tensor
// reduction the tail is what is still resident in L2.
template <typename OutT, bool VEC>
__global__ void __launch_bounds__(kThreads)
quantize_seg_kernel(const float* __restrict__ x, OutT* __restrict__ out, int64_t channels,
                    int64_t inner, int64_t in_stride, int64_t out_stride, int chunks_per_seg,
                    ChannelParams p, float qmin, float qmax, int reverse) {
  pdl_launch_dependents();
  const int64_t bid = reverse ? (static_cast<int64_t>(gridDim.x) - 1 - blockIdx.x) : blockIdx.x;
  const int64_t seg = bid / chunks_per_seg;
  const int chunk = static_cast<int>(bid % chunks_per_seg);
  float s, inv, z;
  load_params(p, seg % channels, s, inv, z);
  const float* xs = x + seg * in_stride;
  OutT* os = out + seg * out_stride;
  const int64_t base = static_cast<int64_t>(chunk) * kChunk;
  if (VEC) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) v[u] = __ldcs(reinterpret_cast<const float4*>(xs + i));
    }
    constexpr bool kByte = sizeof(OutT) == 1;
    constexpr bool kUnsigned = static_cast<OutT>(-1) > static_cast<OutT>(0);
    const bool natural = kByte && (kUnsigned ? (qmin == 0.0f && qmax == 255.0f) : (qmin == -128.0f && qmax == 127.0f));
    const bool has_z = z != 0.0f;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) {
        if (natural) {
          *reinterpret_cast<uint32_t*>(os + i) =
              pack4_sat<kUnsigned>(__fmul_rn(v[u].x, inv), __fmul_rn(v[u].y, inv), __fmul_rn(v[u].z, inv),
                                   __fmul_rn(v[u].w, inv), z, has_z);
        } else {
          store4<OutT>(os + i, code_to_int(grid_code(v[u].x, inv, z), qmin, qmax),
                       code_to_int(grid_code(v[u].y, inv, z), qmin, qmax),
                       code_to_int(grid_code(v[u].z, inv, z), qmin, qmax),
                       code_to_int(grid_code(v[u].w, inv, z), qmin, qmax));
        }
      }
    }
  } else {
#pragma unroll 4
    for (int u = 0; u < 4 * kUnroll; ++u) {
      int64_t i = base + static_cast<int64_t>(u) * kThreads + threadIdx.x;
      if (i < inner) os[i] = static_cast<OutT>(code_to_int(grid_code(__ldg(xs + i), inv, z), qmin, qmax));
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads)
quantize_strided_kernel(const float* __restrict__ x, OutT* __restrict__ out, int64_t total,
                        int64_t channels, int64_t inner, ChannelParams p, float qmin, float qmax) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < total; e += stride) {
    float s, inv, z;
    load_params(p, (e / inner) % channels, s, inv, z);
    out[e] = static_cast<OutT>(code_to_int(grid_code(__ldg(x + e), inv, z), qmin, qmax));
  }
}

template <typename OutT>
__device__ __forceinline__ OutT float_to_out(float v);
template <>
__device__ __forceinline__ float float_to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 float_to_out<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// (f32(q) - z) * s  (lucid/quantization/_functional.py:293)
__device__ __forceinline__ float dequant_one(int q, float s, float z) {
  return __fmul_rn(__fsub_rn(static_cast<float>(q), z), s);
}

template <typename InT, typename OutT, bool VEC>
__global__ void __launch_bounds__(kThreads)
dequantize_seg_kernel(const InT* __restrict__ q, OutT* __restrict__ out, int64_t channels,
                      int64_t inner, int chunks_per_seg, ChannelParams p) {
  const int64_t seg = blockIdx.x / chunks_per_seg;
  const int chunk = blockIdx.x % chunks_per_seg;
  float s, inv, z;
  load_params(p, seg % channels, s, inv, z);
  const InT* qs = q + seg * inner;
  OutT* os = out + seg * inner;
  const int64_t base = static_cast<int64_t>(chunk) * kChunk;
  if (VEC) {
    int a[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) load4<InT>(qs + i, a[u][0], a[u][1], a[u][2], a[u][3]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) {
        float r0 = dequant_one(a[u][0], s, z), r1 = dequant_one(a[u][1], s, z);
        float r2 = dequant_one(a[u][2], s, z), r3 = dequant_one(a[u][3], s, z);
        if (sizeof(OutT) == 4) {
          __stcs(reinterpret_cast<float4*>(os + i), make_float4(r0, r1, r2, r3));
        } else {
          __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
          uint2 w;
          w.x = *reinterpret_cast<unsigned int*>(&lo);
          w.y = *reinterpret_cast<unsigned int*>(&hi);
          *reinterpret_cast<uint2*>(os + i) = w;
        }
      }
    }
  } else {
#pragma unroll 4
    for (int u = 0; u < 4 * kUnroll; ++u) {
      int64_t i = base + static_cast<int64_t>(u) * kThreads + threadIdx.x;
      if (i < inner) os[i] = float_to_out<OutT>(dequant_one(static_cast<int>(qs[i]), s, z));
    }
  }
}

template <typename InT, typename OutT>
__global__ void __launch_bounds__(kThreads)
dequantize_strided_kernel(const InT* __restrict__ q, OutT* __restrict__ out, int64_t total,
                          int64_t channels, int64_t inner, ChannelParams p) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < total; e += stride) {
    float s, inv, z;
    load_params(p, (e / inner) % channels, s, inv, z);
    out[e] = float_to_out<OutT>(dequant_one(static_cast<int>(q[e]), s, z));
  }
}

// ---- short inner extents (channel axis last, or a few elements per channel) --------------
// The tensor is [outer][L = channels * inner]: column j belongs to channel j / inner.  A thread owns
// four adjacent columns, loads their parameters once and walks down kColsRows rows; a warp reads 512
// contiguous bytes per row and nothing is divided per element (the element-wise kernels below spend
// their time on a 64-bit divide and modulo per element: 1.3 TB/s on an [8192, 8192] tensor with the
// channel axis last).
constexpr int kColsRows = 16;  // rows per CTA

struct ColumnWalk {
  int64_t j, r0, r1;
  bool live;
};
__device__ __forceinline__ ColumnWalk column_walk(int64_t outer, int64_t L) {
  ColumnWalk w;
  w.j = (static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x) * 4;
  w.r0 = static_cast<int64_t>(blockIdx.x) * kColsRows;
  w.r1 = w.r0 + kColsRows < outer ? w.r0 + kColsRows : outer;
  w.live = w.j < L;
  return w;
}
__device__ __forceinline__ void load_params4(const ChannelParams& p, int64_t j, int64_t inner, float (&s)[4],
                                             float (&inv)[4], float (&z)[4]) {
  const int64_t c = j / inner;
#pragma unroll
  for (int i = 0; i < 4; ++i) load_params(p, inner == 1 ? c + i : (j + i) / inner, s[i], inv[i], z[i]);
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads)
quantize_cols_kernel(const float* __restrict__ x, OutT* __restrict__ out, int64_t outer, int64_t L,
                     int64_t inner, ChannelParams p, float qmin, float qmax) {
  const ColumnWalk w = column_walk(outer, L);
  if (!w.live) return;
  float s[4], inv[4], z[4];
  load_params4(p, w.j, inner, s, inv, z);
  for (int64_t r = w.r0; r < w.r1; r += kUnroll) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (r + u < w.r1) v[u] = __ldcs(reinterpret_cast<const float4*>(x + (r + u) * L + w.j));
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (r + u < w.r1)
        store4<OutT>(out + (r + u) * L + w.j, code_to_int(grid_code(v[u].x, inv[0], z[0]), qmin, qmax),
                     code_to_int(grid_code(v[u].y, inv[1], z[1]), qmin, qmax),
                     code_to_int(grid_code(v[u].z, inv[2], z[2]), qmin, qmax),
                     code_to_int(grid_code(v[u].w, inv[3], z[3]), qmin, qmax));
  }
}

template <typename InT, typename OutT>
__global__ void __launch_bounds__(kThreads)
dequantize_cols_kernel(const InT* __restrict__ q, OutT* __restrict__ out, int64_t outer, int64_t L,
                       int64_t inner, ChannelParams p) {
  const ColumnWalk w = column_walk(outer, L);
  if (!w.live) return;
  float s[4], inv[4], z[4];
  load_params4(p, w.j, inner, s, inv, z);
  for (int64_t r = w.r0; r < w.r1; r += kUnroll) {
    int a[kUnroll][4];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (r + u < w.r1) load4<InT>(q + (r + u) * L + w.j, a[u][0], a[u][1], a[u][2], a[u][3]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (r + u < w.r1) {
        OutT* o = out + (r + u) * L + w.j;
        const float r0 = dequant_one(a[u][0], s[0], z[0]), r1 = dequant_one(a[u][1], s[1], z[1]);
        const float r2 = dequant_one(a[u][2], s[2], z[2]), r3 = dequant_one(a[u][3], s[3], z[3]);
        if (sizeof(OutT) == 4) {
          __stcs(reinterpret_cast<float4*>(o), make_float4(r0, r1, r2, r3));
        } else {
          __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
          uint2 pk;
          pk.x = *reinterpret_cast<unsigned int*>(&lo);
          pk.y = *reinterpret_cast<unsigned int*>(&hi);
          *reinterpret_cast<uint2*>(o) = pk;
        }
      }
  }
}

// per-channel range over [outer][channels * inner] for 128..2047 elements per channel (a multiple of 128): a warp's
// 128 adjacent columns lie in one channel, every lane walks its four columns down kColsRows rows, the warp
// reduces with shuffles and one lane merges into the channel's running values (a segment kernel's CTA holds one
// such short segment: [32, 4096, 1024] ran at 2.8 TB/s)
__global__ void __launch_bounds__(kThreads)
observe_channel_cols_kernel(const float* __restrict__ x, int64_t outer, int64_t L, int64_t inner,
                            float* min_out, float* max_out) {
  const ColumnWalk w = column_walk(outer, L);
  float mn = INFINITY, mx = -INFINITY;
  if (w.live) {
    for (int64_t r = w.r0; r < w.r1; r += kUnroll) {
      float4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        v[u] = (r + u < w.r1) ? __ldg(reinterpret_cast<const float4*>(x + (r + u) * L + w.j))
                              : make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (r + u < w.r1) {
          mn = fminf(fminf(mn, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
          mx = fmaxf(fmaxf(mx, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
        }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0 && w.live) {  // (L is a multiple of 128: a warp is live or not as a whole)
    const int64_t c = w.j / inner;
    atomic_min_float(min_out + c, mn);
    atomic_max_float(max_out + c, mx);
  }
}

// whether the column kernels apply, and their grid: rows in x (no 65535 limit), column blocks in y.
// Below kSegModeMinInner elements per channel they replace the element-wise kernels; up to 2048 they replace
// the segment kernels too when there are rows to walk down (a segment kernel's CTA of 4096 slots holds one
// segment: [32, 4096, 1024] ran at 3.0 TB/s).
static bool columns_ok(int64_t outer, int64_t channels, int64_t inner, dim3* grid) {
  const int64_t L = channels * inner;
  const int64_t col_blocks = (L / 4 + kThreads - 1) / kThreads, row_blocks = (outer + kColsRows - 1) / kColsRows;
  if (channels == 1) return false;  // one set of parameters: the segment kernels
  if (L % 4 != 0 || col_blocks > 65535 || row_blocks > 0x7fffffffLL) return false;
  if (inner < kSegModeMinInner ? outer < 4 : (inner >= 2048 || outer < 8)) return false;
  *grid = dim3(static_cast<unsigned>(row_blocks), static_cast<unsigned>(col_blocks));
  return true;
}

// (clip(code) - z) * s and the straight-through mask
// (lucid/quantization/_functional.py:326-333)
__device__ __forceinline__ float fake_one(float x, float s, float inv, float z, float qmin,
                                          float qmax, float& mask) {
  float pre = grid_code(x, inv, z);
  float q = (pre != pre) ? pre : fminf(fmaxf(pre, qmin), qmax);
  mask = (pre >= qmin && pre <= qmax) ? 1.0f : 0.0f;
  return __fmul_rn(__fsub_rn(q, z), s);
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
fake_quantize_seg_kernel(const float* __restrict__ x, float* __restrict__ out,
                         float* __restrict__ mask_out, int64_t channels, int64_t inner,
                         int chunks_per_seg, ChannelParams p, float qmin, float qmax) {
  const int64_t seg = blockIdx.x / chunks_per_seg;
  const int chunk = blockIdx.x % chunks_per_seg;
  float s, inv, z;
  load_params(p, seg % channels, s, inv, z);
  const float* xs = x + seg * inner;
  float* os = out + seg * inner;
  float* ms = mask_out ? mask_out + seg * inner : nullptr;
  const int64_t base = static_cast<int64_t>(chunk) * kChunk;
  if (VEC) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) v[u] = __ldcs(reinterpret_cast<const float4*>(xs + i));
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < inner) {
        float4 m, r;
        r.x = fake_one(v[u].x, s, inv, z, qmin, qmax, m.x);
        r.y = fake_one(v[u].y, s, inv, z, qmin, qmax, m.y);
        r.z = fake_one(v[u].z, s, inv, z, qmin, qmax, m.z);
        r.w = fake_one(v[u].w, s, inv, z, qmin, qmax, m.w);
        __stcs(reinterpret_cast<float4*>(os + i), r);
        if (ms) __stcs(reinterpret_cast<float4*>(ms + i), m);
      }
    }
  } else {
#pragma unroll 4
    for (int u = 0; u < 4 * kUnroll; ++u) {
      int64_t i = base + static_cast<int64_t>(u) * kThreads + threadIdx.x;
      if (i < inner) {
        float m;
        os[i] = fake_one(__ldg(xs + i), s, inv, z, qmin, qmax, m);
        if (ms) ms[i] = m;
      }
    }
  }
}

// fake_quantize of an element-wise merge, the converted form of a residual add
// (lucid/nn/quantized/functional_module.py QFunctional.add / mul / add_relu and the scalar
// variants): t = a (+|*) b in fp32, optional ReLU that lets NaN through, then the per-tensor
// grid.  One pass over two inputs and one output (12 B/elem) instead of the eager
// merge (12 B) followed by the eager fake-quantize chain.
enum : int { kMergeAdd = 0, kMergeMul = 1, kMergeAddRelu = 2 };

template <int OP>
__device__ __forceinline__ float merge_one(float a, float b) {
  float t = OP == kMergeMul ? __fmul_rn(a, b) : __fadd_rn(a, b);
  if (OP == kMergeAddRelu) t = (t < 0.0f) ? 0.0f : t;  // NaN compares false and stays
  return t;
}

template <int OP, bool VEC>
__global__ void __launch_bounds__(kThreads)
fake_quantize_merge_kernel(const float* __restrict__ a, const float* __restrict__ b, float scalar,
                           float* __restrict__ out, int64_t n, ChannelParams p, float qmin, float qmax) {
  float s, inv, z, m;
  load_params(p, 0, s, inv, z);
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kChunk;
  if (VEC) {
    float4 va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < n) {
        va[u] = __ldcs(reinterpret_cast<const float4*>(a + i));
        vb[u] = b ? __ldcs(reinterpret_cast<const float4*>(b + i)) : make_float4(scalar, scalar, scalar, scalar);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + (static_cast<int64_t>(u) * kThreads + threadIdx.x) * 4;
      if (i < n) {
        float4 r;
        r.x = fake_one(merge_one<OP>(va[u].x, vb[u].x), s, inv, z, qmin, qmax, m);
        r.y = fake_one(merge_one<OP>(va[u].y, vb[u].y), s, inv, z, qmin, qmax, m);
        r.z = fake_one(merge_one<OP>(va[u].z, vb[u].z), s, inv, z, qmin, qmax, m);
        r.w = fake_one(merge_one<OP>(va[u].w, vb[u].w), s, inv, z, qmin, qmax, m);
        __stcs(reinterpret_cast<float4*>(out + i), r);
      }
    }
  } else {
#pragma unroll 4
    for (int u = 0; u < 4 * kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * kThreads + threadIdx.x;
      if (i < n) out[i] = fake_one(merge_one<OP>(__ldg(a + i), b ? __ldg(b + i) : scalar), s, inv, z, qmin, qmax, m);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
fake_quantize_strided_kernel(const float* __restrict__ x, float* __restrict__ out,
                             float* __restrict__ mask_out, int64_t total, int64_t channels,
                             int64_t inner, ChannelParams p, float qmin, float qmax) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < total; e += stride) {
    float s, inv, z, m;
    load_params(p, (e / inner) % channels, s, inv, z);
    out[e] = fake_one(__ldg(x + e), s, inv, z, qmin, qmax, m);
    if (mask_out) mask_out[e] = m;
  }
}

__global__ void __launch_bounds__(kThreads)
fake_quantize_cols_kernel(const float* __restrict__ x, float* __restrict__ out, float* __restrict__ mask_out,
                          int64_t outer, int64_t L, int64_t inner, ChannelParams p, float qmin, float qmax) {
  const ColumnWalk w = column_walk(outer, L);
  if (!w.live) return;
  float s[4], inv[4], z[4];
  load_params4(p, w.j, inner, s, inv, z);
  for (int64_t r = w.r0; r < w.r1; r += kUnroll) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (r + u < w.r1) v[u] = __ldcs(reinterpret_cast<const float4*>(x + (r + u) * L + w.j));
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (r + u < w.r1) {
        float4 m, o;
        o.x = fake_one(v[u].x, s[0], inv[0], z[0], qmin, qmax, m.x);
        o.y = fake_one(v[u].y, s[1], inv[1], z[1], qmin, qmax, m.y);
        o.z = fake_one(v[u].z, s[2], inv[2], z[2], qmin, qmax, m.z);
        o.w = fake_one(v[u].w, s[3], inv[3], z[3], qmin, qmax, m.w);
        __stcs(reinterpret_cast<float4*>(out + (r + u) * L + w.j), o);
        if (mask_out) __stcs(reinterpret_cast<float4*>(mask_out + (r + u) * L + w.j), m);
      }
  }
}

// =========================================================================
// fused per-row dynamic quantization: observer + qparams + quantize, one read
// =========================================================================
// The whole row lives in registers (ITEMS float4 per thread), so HBM sees each
// element once: 4 bytes in, 1 byte out.
template <typename OutT, int BLOCK, int ITEMS>
__global__ void __launch_bounds__(BLOCK)
dynamic_quantize_rows_kernel(const float* __restrict__ x, int64_t cols, int64_t ldx,
                             QParamSpec spec, OutT* __restrict__ q, int64_t ldq,
                             float* __restrict__ scale_out, float* __restrict__ zp_out) {
  pdl_launch_dependents();
  __shared__ float red[64];
  const int64_t row = blockIdx.x;
  const float* xr = x + row * ldx;
  OutT* qr = q + row * ldq;
  float4 v[ITEMS];
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    int64_t i = (static_cast<int64_t>(u) * BLOCK + threadIdx.x) * 4;
    if (i < cols) v[u] = __ldcs(reinterpret_cast<const float4*>(xr + i));
  }
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    int64_t i = (static_cast<int64_t>(u) * BLOCK + threadIdx.x) * 4;
    if (i < cols) {
      mn = fminf(fminf(mn, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
      mx = fmaxf(fmaxf(mx, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
    }
  }
  block_minmax(mn, mx, red);
  float s, z;
  qparams_from_range(mn, mx, spec, s, z);
  const float inv = __fdiv_rn(1.0f, s);
  if (threadIdx.x == 0) {
    scale_out[row] = s;
    if (zp_out) zp_out[row] = z;
  }
  constexpr bool kByte = sizeof(OutT) == 1;
  constexpr bool kUnsigned = static_cast<OutT>(-1) > static_cast<OutT>(0);
  const bool natural = kByte && (kUnsigned ? (spec.qmin == 0.0f && spec.qmax == 255.0f)
                                           : (spec.qmin == -128.0f && spec.qmax == 127.0f));
  const bool has_z = z != 0.0f;
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    int64_t i = (static_cast<int64_t>(u) * BLOCK + threadIdx.x) * 4;
    if (i < cols) {
      if (natural) {
        *reinterpret_cast<uint32_t*>(qr + i) =
            pack4_sat<kUnsigned>(__fmul_rn(v[u].x, inv), __fmul_rn(v[u].y, inv), __fmul_rn(v[u].z, inv),
                                 __fmul_rn(v[u].w, inv), z, has_z);
      } else {
        store4<OutT>(qr + i, code_to_int(grid_code(v[u].x, inv, z), spec.qmin, spec.qmax),
                     code_to_int(grid_code(v[u].y, inv, z), spec.qmin, spec.qmax),
                     code_to_int(grid_code(v[u].z, inv, z), spec.qmin, spec.qmax),
                     code_to_int(grid_code(v[u].w, inv, z), spec.qmin, spec.qmax));
      }
    }
  }
}

// Rows of up to 2048 elements: one WARP per row, eight rows per CTA.  A CTA per row leaves a short row with one
// 16-byte load per thread in flight and a block-wide reduction behind two barriers ([131072, 512]: 2.4 TB/s,
// [1048576, 64]: 0.3 TB/s); a warp keeps the row in ITEMS float4 per lane and reduces with shuffles.
constexpr int kRowsPerCta = 8;
template <typename OutT, int ITEMS>
__global__ void __launch_bounds__(kRowsPerCta * 32)
dynamic_quantize_rows_warp_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, int64_t ldx,
                                  QParamSpec spec, OutT* __restrict__ q, int64_t ldq,
                                  float* __restrict__ scale_out, float* __restrict__ zp_out) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;  // (whole warps leave together)
  const float* xr = x + row * ldx;
  OutT* qr = q + row * ldq;
  float4 v[ITEMS];
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    const int64_t i = (static_cast<int64_t>(u) * 32 + lane) * 4;
    if (i < cols) v[u] = __ldcs(reinterpret_cast<const float4*>(xr + i));
  }
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    const int64_t i = (static_cast<int64_t>(u) * 32 + lane) * 4;
    if (i < cols) {
      mn = fminf(fminf(mn, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
      mx = fmaxf(fmaxf(mx, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  float s, z;
  qparams_from_range(mn, mx, spec, s, z);
  const float inv = __fdiv_rn(1.0f, s);
  if (lane == 0) {
    scale_out[row] = s;
    if (zp_out) zp_out[row] = z;
  }
  constexpr bool kByte = sizeof(OutT) == 1;
  constexpr bool kUnsigned = static_cast<OutT>(-1) > static_cast<OutT>(0);
  const bool natural = kByte && (kUnsigned ? (spec.qmin == 0.0f && spec.qmax == 255.0f)
                                           : (spec.qmin == -128.0f && spec.qmax == 127.0f));
  const bool has_z = z != 0.0f;
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    const int64_t i = (static_cast<int64_t>(u) * 32 + lane) * 4;
    if (i < cols) {
      if (natural) {
        *reinterpret_cast<uint32_t*>(qr + i) =
            pack4_sat<kUnsigned>(__fmul_rn(v[u].x, inv), __fmul_rn(v[u].y, inv), __fmul_rn(v[u].z, inv),
                                 __fmul_rn(v[u].w, inv), z, has_z);
      } else {
        store4<OutT>(qr + i, code_to_int(grid_code(v[u].x, inv, z), spec.qmin, spec.qmax),
                     code_to_int(grid_code(v[u].y, inv, z), spec.qmin, spec.qmax),
                     code_to_int(grid_code(v[u].z, inv, z), spec.qmin, spec.qmax),
                     code_to_int(grid_code(v[u].w, inv, z), spec.qmin, spec.qmax));
      }
    }
  }
}

// Per-tensor dynamic quantization of a small tensor in ONE launch: the activations of a
// single Linear on a small batch (64 x 1024 at C1) are too few for the two-kernel form
// (global range, then quantize) to be anything but two launch latencies.  A cluster of up
// to 8 CTAs keeps the whole tensor in registers, exchanges the eight partial ranges through
// distributed shared memory behind a hardware cluster barrier, and every CTA then derives the
// same qparams and quantizes its share.  x is dense [rows, cols], cols % 4 == 0; the codes go
// to a matrix with leading dimension ldq.
constexpr int kSmallThreads = 512;
constexpr int kSmallItems = 8;                                      // float4 per thread
constexpr int kSmallMaxCluster = 8;
constexpr int64_t kSmallPerCta = int64_t{kSmallThreads} * kSmallItems * 4;  // 16384 elements
constexpr int64_t kSmallMaxElems = kSmallPerCta * kSmallMaxCluster;          // 131072

template <typename OutT>
__global__ void __launch_bounds__(kSmallThreads)
dynamic_quantize_tensor_small_kernel(const float* __restrict__ x, int64_t n, int64_t cols, QParamSpec spec,
                                     OutT* __restrict__ q, int64_t ldq, float* __restrict__ scale_out,
                                     float* __restrict__ zp_out, float* __restrict__ minmax_out) {
  pdl_launch_dependents();
  __shared__ float red[64];
  __shared__ float part[2];
  uint32_t rank, nctas;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nctas));
  const int64_t base = static_cast<int64_t>(rank) * kSmallPerCta;
  float4 v[kSmallItems];
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < kSmallItems; ++u) {
    const int64_t i = base + (static_cast<int64_t>(u) * kSmallThreads + threadIdx.x) * 4;
    if (i < n) v[u] = __ldg(reinterpret_cast<const float4*>(x + i));
  }
#pragma unroll
  for (int u = 0; u < kSmallItems; ++u) {
    const int64_t i = base + (static_cast<int64_t>(u) * kSmallThreads + threadIdx.x) * 4;
    if (i < n) {
      mn = fminf(fminf(mn, fminf(v[u].x, v[u].y)), fminf(v[u].z, v[u].w));
      mx = fmaxf(fmaxf(mx, fmaxf(v[u].x, v[u].y)), fmaxf(v[u].z, v[u].w));
    }
  }
  block_minmax(mn, mx, red);
  if (threadIdx.x == 0) {
    part[0] = mn;
    part[1] = mx;
  }
  // all CTAs of the cluster have published their range (release / acquire at cluster scope)
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  mn = INFINITY;
  mx = -INFINITY;
  const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(part));
  for (uint32_t r = 0; r < nctas; ++r) {
    uint32_t remote;
    float a, b;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(r));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(a) : "r"(remote));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(b) : "r"(remote + 4));
    mn = fminf(mn, a);
    mx = fmaxf(mx, b);
  }
  // nobody leaves (and frees its shared memory) while a peer may still be reading it
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  float s, z;
  qparams_from_range(mn, mx, spec, s, z);
  const float inv = __fdiv_rn(1.0f, s);
  if (rank == 0 && threadIdx.x == 0) {
    scale_out[0] = s;
    zp_out[0] = z;
    minmax_out[0] = mn;
    minmax_out[1] = mx;
  }
#pragma unroll
  for (int u = 0; u < kSmallItems; ++u) {
    const int64_t i = base + (static_cast<int64_t>(u) * kSmallThreads + threadIdx.x) * 4;
    if (i < n) {
      const int64_t row = i / cols, col = i - row * cols;  // cols % 4 == 0: the four stay in one row
      store4<OutT>(q + row * ldq + col, code_to_int(grid_code(v[u].x, inv, z), spec.qmin, spec.qmax),
                   code_to_int(grid_code(v[u].y, inv, z), spec.qmin, spec.qmax),
                   code_to_int(grid_code(v[u].z, inv, z), spec.qmin, spec.qmax),
                   code_to_int(grid_code(v[u].w, inv, z), spec.qmin, spec.qmax));
    }
  }
}

template <typename OutT>
static int32_t launch_dynamic_quantize_small(const float* x, int64_t rows, int64_t cols, const QParamSpec& spec,
                                             OutT* q, int64_t ldq, float* scale_out, float* zp_out,
                                             float* minmax_out, cudaStream_t st) {
  const int64_t n = rows * cols;
  const unsigned ctas = static_cast<unsigned>((n + kSmallPerCta - 1) / kSmallPerCta);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kSmallThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ctas;  // the whole grid is one cluster (<= 8 CTAs)
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, dynamic_quantize_tensor_small_kernel<OutT>, x, n, cols, spec, q, ldq,
                                             scale_out, zp_out, minmax_out);
  if (err != cudaSuccess) return fail(LC_ERR_CUDA, "dynamic_quantize_tensor (small): %s", cudaGetErrorString(err));
  return check_launch("dynamic_quantize_tensor (small)");
}

// any row length / alignment: two passes over the row (the second one is
// served by L1/L2 for rows of ordinary size)
template <typename OutT>
__global__ void __launch_bounds__(kThreads)
dynamic_quantize_rows_generic_kernel(const float* __restrict__ x, int64_t cols, int64_t ldx,
                                     QParamSpec spec, OutT* __restrict__ q, int64_t ldq,
                                     float* __restrict__ scale_out, float* __restrict__ zp_out) {
  __shared__ float red[64];
  const int64_t row = blockIdx.x;
  const float* xr = x + row * ldx;
  OutT* qr = q + row * ldq;
  float mn = INFINITY, mx = -INFINITY;
  for (int64_t i = threadIdx.x; i < cols; i += kThreads) {
    float v = __ldg(xr + i);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  block_minmax(mn, mx, red);
  float s, z;
  qparams_from_range(mn, mx, spec, s, z);
  const float inv = __fdiv_rn(1.0f, s);
  if (threadIdx.x == 0) {
    scale_out[row] = s;
    if (zp_out) zp_out[row] = z;
  }
  for (int64_t i = threadIdx.x; i < cols; i += kThreads)
    qr[i] = static_cast<OutT>(code_to_int(grid_code(__ldg(xr + i), inv, z), spec.qmin, spec.qmax));
}

// int32 row sums of an int8 matrix: one warp per row
__global__ void __launch_bounds__(kThreads)
rowsum_s8_kernel(const int8_t* __restrict__ b, int64_t rows, int64_t cols, int64_t ldb,
                 int32_t* __restrict__ out) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int8_t* br = b + row * ldb;
  int acc = 0;
  for (int64_t i = lane; i < cols; i += 32) acc += br[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] = acc;
}

// =========================================================================
// host launchers
// =========================================================================
static bool layout_ok(int64_t outer, int64_t channels, int64_t inner) {
  return outer >= 0 && channels >= 1 && inner >= 0;
}

// Per-tensor parameters make the channel structure irrelevant: treat the tensor
// as one long segment so the vector path applies whatever the original shape.
static void collapse_if_scalar(int64_t& outer, int64_t& channels, int64_t& inner,
                               const float* scale, int64_t n_scale, const float* zp, int64_t n_zp) {
  const bool scalar_scale = (scale == nullptr) || n_scale == 1;
  const bool scalar_zp = (zp == nullptr) || n_zp == 1;
  if (channels == 1 || (scalar_scale && scalar_zp)) {
    inner = outer * channels * inner;
    outer = 1;
    channels = 1;
  }
}

static int chunks_for(int64_t inner) { return static_cast<int>((inner + kChunk - 1) / kChunk); }

static int32_t check_param_counts(int64_t channels, const float* scale, int64_t n_scale,
                                  const float* zp, int64_t n_zp) {
  if (scale && n_scale != 1 && n_scale != channels)
    return fail(LC_ERR_INVALID_ARG, "scale has %lld entries, expected 1 or %lld", (long long)n_scale,
                (long long)channels);
  if (zp && n_zp != 1 && n_zp != channels)
    return fail(LC_ERR_INVALID_ARG, "zero_point has %lld entries, expected 1 or %lld",
                (long long)n_zp, (long long)channels);
  return LC_OK;
}

static int strided_grid(int64_t total) {
  int64_t g = (total + kThreads - 1) / kThreads;
  int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

template <typename OutT>
static int32_t launch_quantize(const float* x, int64_t outer, int64_t channels, int64_t inner,
                               int64_t in_stride, int64_t out_stride, const ChannelParams& p,
                               float qmin, float qmax, OutT* out, int reverse, cudaStream_t st) {
  const int64_t segs = outer * channels;
  if (segs == 0 || inner == 0) return LC_OK;
  const bool dense = (in_stride == inner && out_stride == inner);
  dim3 cgrid;
  if (dense && columns_ok(outer, channels, inner, &cgrid) && aligned(x, 16) && aligned(out, 4 * sizeof(OutT))) {
    quantize_cols_kernel<OutT><<<cgrid, kThreads, 0, st>>>(x, out, outer, channels * inner, inner, p, qmin, qmax);
  } else if (inner >= kSegModeMinInner || channels == 1 || !dense) {
    const int cps = chunks_for(inner);
    const int64_t grid = segs * cps;
    if (grid > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "tensor too large for one launch");
    const bool vec = (inner % 4 == 0) && (in_stride % 4 == 0) && (out_stride % 4 == 0) &&
                     aligned(x, 16) && aligned(out, 4 * sizeof(OutT));
    if (vec)
      quantize_seg_kernel<OutT, true><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(
          x, out, channels, inner, in_stride, out_stride, cps, p, qmin, qmax, reverse);
    else
      quantize_seg_kernel<OutT, false><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(
          x, out, channels, inner, in_stride, out_stride, cps, p, qmin, qmax, reverse);
  } else {
    const int64_t total = segs * inner;
    quantize_strided_kernel<OutT><<<strided_grid(total), kThreads, 0, st>>>(x, out, total, channels,
                                                                           inner, p, qmin, qmax);
  }
  return check_launch("quantize");
}

template <typename InT, typename OutT>
static int32_t launch_dequantize(const InT* q, int64_t outer, int64_t channels, int64_t inner,
                                 const ChannelParams& p, OutT* out, cudaStream_t st) {
  const int64_t segs = outer * channels;
  if (segs == 0 || inner == 0) return LC_OK;
  dim3 cgrid;
  if (columns_ok(outer, channels, inner, &cgrid) && aligned(q, 4 * sizeof(InT)) && aligned(out, 4 * sizeof(OutT))) {
    dequantize_cols_kernel<InT, OutT><<<cgrid, kThreads, 0, st>>>(q, out, outer, channels * inner, inner, p);
  } else if (inner >= kSegModeMinInner || channels == 1) {
    const int cps = chunks_for(inner);
    const int64_t grid = segs * cps;
    if (grid > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "tensor too large for one launch");
    const bool vec = (inner % 4 == 0) && aligned(q, 4 * sizeof(InT)) && aligned(out, 4 * sizeof(OutT));
    if (vec)
      dequantize_seg_kernel<InT, OutT, true>
          <<<static_cast<unsigned>(grid), kThreads, 0, st>>>(q, out, channels, inner, cps, p);
    else
      dequantize_seg_kernel<InT, OutT, false>
          <<<static_cast<unsigned>(grid), kThreads, 0, st>>>(q, out, channels, inner, cps, p);
  } else {
    const int64_t total = segs * inner;
    dequantize_strided_kernel<InT, OutT>
        <<<strided_grid(total), kThreads, 0, st>>>(q, out, total, channels, inner, p);
  }
  return check_launch("dequantize");
}

template <typename InT>
static int32_t dispatch_dequantize_out(const InT* q, int64_t outer, int64_t channels, int64_t inner,
                                       const ChannelParams& p, void* out, int32_t out_dtype,
                                       cudaStream_t st) {
  if (out_dtype == LC_F32)
    return launch_dequantize<InT, float>(q, outer, channels, inner, p, static_cast<float*>(out), st);
  if (out_dtype == LC_BF16)
    return launch_dequantize<InT, __nv_bfloat16>(q, outer, channels, inner, p,
                                                 static_cast<__nv_bfloat16*>(out), st);
  return fail(LC_ERR_UNSUPPORTED, "dequantize: out_dtype %d not supported", out_dtype);
}

static int observe_grid(int64_t n) {
  int64_t g = (n + kChunk - 1) / kChunk;
  int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (cap > kMaxObserveCtas) cap = kMaxObserveCtas;
  if (g < 1) g = 1;
  return static_cast<int>(g < cap ? g : cap);
}

static int32_t launch_observe_tensor(const float* x, int64_t n, float* min_out, float* max_out,
                                     int accumulate, int with_qparams, const QParamSpec& spec,
                                     float* scale_out, float* zp_out, void* workspace,
                                     int64_t workspace_bytes, cudaStream_t st) {
  if (!workspace || workspace_bytes < static_cast<int64_t>(sizeof(TensorObserveScratch)))
    return fail(LC_ERR_WORKSPACE, "observe_tensor needs %lld bytes of zero-filled scratch",
                (long long)sizeof(TensorObserveScratch));
  if (n <= 0) return fail(LC_ERR_INVALID_ARG, "observe_tensor: empty input has no min/max");
  const int vec_ok = aligned(x, 16) ? 1 : 0;
  observe_tensor_kernel<<<observe_grid(n), kThreads, 0, st>>>(
      x, n, vec_ok, min_out, max_out, accumulate, with_qparams, spec, scale_out, zp_out,
      static_cast<TensorObserveScratch*>(workspace));
  return check_launch("observe_tensor");
}

template <typename OutT>
static int32_t launch_dynamic_rows(const float* x, int64_t rows, int64_t cols, int64_t ldx,
                                   const QParamSpec& spec, OutT* q, int64_t ldq, float* scale_out,
                                   float* zp_out, cudaStream_t st) {
  if (rows == 0) return LC_OK;
  if (rows > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "too many rows for one launch");
  const unsigned grid = static_cast<unsigned>(rows);
  const bool vec = (cols % 4 == 0) && (ldx % 4 == 0) && (ldq % 4 == 0) && aligned(x, 16) &&
                   aligned(q, 4 * sizeof(OutT));
#define LC_ROWS(BLOCK, ITEMS)                                                              \
  dynamic_quantize_rows_kernel<OutT, BLOCK, ITEMS><<<grid, BLOCK, 0, st>>>(x, cols, ldx, spec, q, \
                                                                          ldq, scale_out, zp_out)
#define LC_WARP_ROWS(ITEMS)                                                                                   \
  dynamic_quantize_rows_warp_kernel<OutT, ITEMS>                                                              \
      <<<static_cast<unsigned>((rows + kRowsPerCta - 1) / kRowsPerCta), kRowsPerCta * 32, 0, st>>>(x, rows, cols, ldx, \
                                                                                                    spec, q, ldq, scale_out, zp_out)
  if (vec && cols <= 2048) {
    if (cols <= 128) LC_WARP_ROWS(1);
    else if (cols <= 256) LC_WARP_ROWS(2);
    else if (cols <= 512) LC_WARP_ROWS(4);
    else if (cols <= 1024) LC_WARP_ROWS(8);
    else LC_WARP_ROWS(16);
  } else if (vec && cols <= 16384) {
    if (cols <= 4096) LC_ROWS(256, 4);
    else if (cols <= 8192) LC_ROWS(256, 8);
    else LC_ROWS(256, 16);
  } else {
    dynamic_quantize_rows_generic_kernel<OutT>
        <<<grid, kThreads, 0, st>>>(x, cols, ldx, spec, q, ldq, scale_out, zp_out);
  }
#undef LC_ROWS
#undef LC_WARP_ROWS
  return check_launch("dynamic_quantize_rows");
}

}  // namespace lc

// =========================================================================
// C ABI
// =========================================================================
using namespace lc;

extern "C" int64_t lc_observe_tensor_workspace_bytes(void) {
  return static_cast<int64_t>(sizeof(TensorObserveScratch));
}

extern "C" int32_t lc_observe_tensor_f32(const float* x, int64_t n, float* min_out, float* max_out,
                                         int32_t accumulate, int32_t symmetric, int32_t quant_min,
                                         int32_t quant_max, int32_t is_signed, float eps,
                                         float* scale_out, float* zp_out, void* workspace,
                                         int64_t workspace_bytes, void* stream) {
  if (!x || !min_out || !max_out) return fail(LC_ERR_INVALID_ARG, "observe_tensor: null pointer");
  if ((scale_out == nullptr) != (zp_out == nullptr))
    return fail(LC_ERR_INVALID_ARG, "observe_tensor: scale_out and zp_out go together");
  QParamSpec spec = make_qparam_spec(symmetric, quant_min, quant_max, is_signed, eps);
  return launch_observe_tensor(x, n, min_out, max_out, accumulate, scale_out != nullptr, spec,
                               scale_out, zp_out, workspace, workspace_bytes, as_stream(stream));
}

// ---- observe_tensor without caller scratch -------------------------------------------
// The scratch of the global-range kernel (ticket + per-CTA partials) lives in this
// file-scope device array instead of a caller buffer.  Every GPU that loads the library
// holds these sizeof(TensorObserveScratch) bytes (about 9.3 KB) until the process exits.
// In host code the array's name is only a handle for cudaGetSymbolAddress; the device
// address is looked up once per device and cached.
static __device__ __align__(256) unsigned char g_observe_static_scratch[sizeof(TensorObserveScratch)];

constexpr int64_t kObserveStaticMaxElems = int64_t{1} << 30;

// The address is looked up under a per-device mutex and cached only when the lookup succeeded, so
// a failed first call (no context yet, a transient error) is retried by the next one.  The cached
// address belongs to the device's primary context: `refresh` drops it, which the entry point asks
// for when the first use of the address fails (the context was torn down and rebuilt, e.g. by
// cudaDeviceReset, and the old address is stale).
static int32_t static_scratch_address(TensorObserveScratch** out, bool refresh) {
  constexpr int kMaxDevices = 64;
  static std::mutex locks[kMaxDevices];
  static void* addrs[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(LC_ERR_CUDA, "observe_tensor_static: no current CUDA device");
  std::lock_guard<std::mutex> hold(locks[dev]);
  if (refresh) addrs[dev] = nullptr;
  if (addrs[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&p, g_observe_static_scratch);
    if (err != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(LC_ERR_CUDA, "observe_tensor_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                  cudaGetErrorString(err));
    }
    addrs[dev] = p;
  }
  *out = static_cast<TensorObserveScratch*>(addrs[dev]);
  return LC_OK;
}

extern "C" int64_t lc_observe_tensor_static_max_elems(void) { return kObserveStaticMaxElems; }

extern "C" int32_t lc_observe_tensor_static_f32(const float* x, int64_t n, float* min_out,
                                                float* max_out, int32_t accumulate,
                                                int32_t symmetric, int32_t quant_min,
                                                int32_t quant_max, int32_t is_signed, float eps,
                                                float* scale_out, float* zp_out, void* stream) {
  if (!x || !min_out || !max_out)
    return fail(LC_ERR_INVALID_ARG, "observe_tensor_static: null pointer");
  if ((scale_out == nullptr) != (zp_out == nullptr))
    return fail(LC_ERR_INVALID_ARG, "observe_tensor_static: scale_out and zp_out go together");
  if (n <= 0) return fail(LC_ERR_INVALID_ARG, "observe_tensor_static: empty input has no min/max");
  if (n > kObserveStaticMaxElems)
    return fail(LC_ERR_UNSUPPORTED,
                "observe_tensor_static: %lld elements exceed the limit of %lld of the built-in scratch; "
                "use lc_observe_tensor_f32 with a caller workspace",
                (long long)n, (long long)kObserveStaticMaxElems);
  TensorObserveScratch* ws = nullptr;
  if (int32_t rc = static_scratch_address(&ws, false)) return rc;
  cudaStream_t st = as_stream(stream);
  // the array keeps whatever the previous call left: the ticket has to start at zero
  if (cudaMemsetAsync(ws, 0, 16, st) != cudaSuccess) {
    // a cached address that no longer belongs to a live context: look it up again, once
    cudaGetLastError();
    if (int32_t rc = static_scratch_address(&ws, true)) return rc;
    if (cudaMemsetAsync(ws, 0, 16, st) != cudaSuccess)
      return fail(LC_ERR_CUDA, "observe_tensor_static: %s", cudaGetErrorString(cudaGetLastError()));
  }
  QParamSpec spec = make_qparam_spec(symmetric, quant_min, quant_max, is_signed, eps);
  observe_tensor_kernel<<<observe_grid(n), kThreads, 0, st>>>(x, n, aligned(x, 16) ? 1 : 0, min_out,
                                                              max_out, accumulate, scale_out != nullptr,
                                                              spec, scale_out, zp_out, ws);
  return check_launch("observe_tensor_static");
}

extern "C" int32_t lc_observe_channel_f32(const float* x, int64_t outer, int64_t channels,
                                          int64_t inner, float* min_out, float* max_out,
                                          int32_t accumulate, void* stream) {
  if (!x || !min_out || !max_out) return fail(LC_ERR_INVALID_ARG, "observe_channel: null pointer");
  if (!layout_ok(outer, channels, inner) || outer * inner == 0)
    return fail(LC_ERR_INVALID_ARG, "observe_channel: empty reduction");
  cudaStream_t st = as_stream(stream);
  if (!accumulate) {
    fill_minmax_kernel<<<static_cast<unsigned>((channels + 255) / 256), 256, 0, st>>>(min_out, max_out,
                                                                                     channels);
  }
  dim3 cgrid;
  if (inner % 128 == 0 && aligned(x, 16) && columns_ok(outer, channels, inner, &cgrid)) {
    observe_channel_cols_kernel<<<cgrid, kThreads, 0, st>>>(x, outer, channels * inner, inner, min_out, max_out);
  } else if (inner >= kSegModeMinInner) {
    const int cps = chunks_for(inner);
    const int64_t grid = outer * channels * cps;
    if (grid > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "tensor too large for one launch");
    if (inner % 4 == 0 && aligned(x, 16))
      observe_channel_seg_kernel<true>
          <<<static_cast<unsigned>(grid), kThreads, 0, st>>>(x, channels, inner, cps, min_out, max_out);
    else
      observe_channel_seg_kernel<false>
          <<<static_cast<unsigned>(grid), kThreads, 0, st>>>(x, channels, inner, cps, min_out, max_out);
  } else {
    const int64_t width = channels * inner;
    const int rows_per_cta = 64;
    const int64_t gy = (outer + rows_per_cta - 1) / rows_per_cta;
    if (gy > 65535) return fail(LC_ERR_UNSUPPORTED, "observe_channel: outer too large");
    dim3 grid(static_cast<unsigned>((width + kThreads - 1) / kThreads), static_cast<unsigned>(gy));
    observe_channel_strided_kernel<<<grid, kThreads, 0, st>>>(x, outer, width, inner, rows_per_cta,
                                                             min_out, max_out);
  }
  return check_launch("observe_channel");
}

extern "C" int32_t lc_calculate_qparams_f32(const float* min_val, const float* max_val, int64_t n,
                                            int32_t symmetric, int32_t quant_min, int32_t quant_max,
                                            int32_t is_signed, float eps, float* scale_out,
                                            float* zp_out, void* stream) {
  if (!min_val || !max_val || !scale_out || !zp_out)
    return fail(LC_ERR_INVALID_ARG, "calculate_qparams: null pointer");
  if (n == 0) return LC_OK;
  QParamSpec spec = make_qparam_spec(symmetric, quant_min, quant_max, is_signed, eps);
  calculate_qparams_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, as_stream(stream)>>>(
      min_val, max_val, n, spec, scale_out, zp_out);
  return check_launch("calculate_qparams");
}

extern "C" int32_t lc_quantize_f32(const float* x, int64_t outer, int64_t channels, int64_t inner,
                                   const float* scale, int64_t n_scale, const float* zero_point,
                                   int64_t n_zp, float host_inv_scale, float host_zero_point,
                                   int32_t quant_min, int32_t quant_max, void* out,
                                   int32_t out_dtype, void* stream) {
  if (!layout_ok(outer, channels, inner)) return fail(LC_ERR_INVALID_ARG, "quantize: bad layout");
  if (outer * channels * inner == 0) return LC_OK;
  if (!x || !out) return fail(LC_ERR_INVALID_ARG, "quantize: null pointer");
  if (int32_t rc = check_param_counts(channels, scale, n_scale, zero_point, n_zp)) return rc;
  collapse_if_scalar(outer, channels, inner, scale, n_scale, zero_point, n_zp);
  ChannelParams p{scale, zero_point, n_scale, n_zp, host_inv_scale, 0.0f, host_zero_point};
  const float qmin = static_cast<float>(quant_min), qmax = static_cast<float>(quant_max);
  cudaStream_t st = as_stream(stream);
  switch (out_dtype) {
    case LC_S8:
      return launch_quantize<int8_t>(x, outer, channels, inner, inner, inner, p, qmin, qmax,
                                     static_cast<int8_t*>(out), 0, st);
    case LC_U8:
      return launch_quantize<uint8_t>(x, outer, channels, inner, inner, inner, p, qmin, qmax,
                                      static_cast<uint8_t*>(out), 0, st);
    case LC_S16:
      return launch_quantize<int16_t>(x, outer, channels, inner, inner, inner, p, qmin, qmax,
                                      static_cast<int16_t*>(out), 0, st);
    case LC_S32:
      return launch_quantize<int32_t>(x, outer, channels, inner, inner, inner, p, qmin, qmax,
                                      static_cast<int32_t*>(out), 0, st);
  }
  return fail(LC_ERR_UNSUPPORTED, "quantize: out_dtype %d not supported", out_dtype);
}

extern "C" int32_t lc_dequantize(const void* q, int32_t q_dtype, int64_t outer, int64_t channels,
                                 int64_t inner, const float* scale, int64_t n_scale,
                                 const float* zero_point, int64_t n_zp, float host_scale,
                                 float host_zero_point, void* out, int32_t out_dtype, void* stream) {
  if (!layout_ok(outer, channels, inner)) return fail(LC_ERR_INVALID_ARG, "dequantize: bad layout");
  if (outer * channels * inner == 0) return LC_OK;
  if (!q || !out) return fail(LC_ERR_INVALID_ARG, "dequantize: null pointer");
  if (int32_t rc = check_param_counts(channels, scale, n_scale, zero_point, n_zp)) return rc;
  collapse_if_scalar(outer, channels, inner, scale, n_scale, zero_point, n_zp);
  ChannelParams p{scale, zero_point, n_scale, n_zp, 0.0f, host_scale, host_zero_point};
  cudaStream_t st = as_stream(stream);
  switch (q_dtype) {
    case LC_S8:
      return dispatch_dequantize_out(static_cast<const int8_t*>(q), outer, channels, inner, p, out,
                                     out_dtype, st);
    case LC_U8:
      return dispatch_dequantize_out(static_cast<const uint8_t*>(q), outer, channels, inner, p, out,
                                     out_dtype, st);
    case LC_S16:
      return dispatch_dequantize_out(static_cast<const int16_t*>(q), outer, channels, inner, p, out,
                                     out_dtype, st);
    case LC_S32:
      return dispatch_dequantize_out(static_cast<const int32_t*>(q), outer, channels, inner, p, out,
                                     out_dtype, st);
  }
  return fail(LC_ERR_UNSUPPORTED, "dequantize: q_dtype %d not supported", q_dtype);
}

extern "C" int32_t lc_fake_quantize_merge_f32(const float* a, const float* b, float host_scalar, int32_t op,
                                              int64_t n, const float* scale, const float* zero_point,
                                              float host_inv_scale, float host_scale, float host_zero_point,
                                              int32_t quant_min, int32_t quant_max, float* out, void* stream) {
  if (n < 0 || op < kMergeAdd || op > kMergeAddRelu) return fail(LC_ERR_INVALID_ARG, "fake_quantize_merge: bad arguments");
  if (n == 0) return LC_OK;
  if (!a || !out) return fail(LC_ERR_INVALID_ARG, "fake_quantize_merge: null pointer");
  ChannelParams p{scale, zero_point, 1, 1, host_inv_scale, host_scale, host_zero_point};
  const float qmin = static_cast<float>(quant_min), qmax = static_cast<float>(quant_max);
  const int64_t grid = (n + kChunk - 1) / kChunk;
  if (grid > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "tensor too large for one launch");
  const bool vec = n % 4 == 0 && aligned(a, 16) && aligned(out, 16) && (!b || aligned(b, 16));
  cudaStream_t st = as_stream(stream);
#define LC_MERGE(OP)                                                                                          \
  do {                                                                                                        \
    if (vec)                                                                                                  \
      fake_quantize_merge_kernel<OP, true><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(a, b, host_scalar, out, \
                                                                                             n, p, qmin, qmax);     \
    else                                                                                                      \
      fake_quantize_merge_kernel<OP, false><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(a, b, host_scalar,    \
                                                                                              out, n, p, qmin, qmax); \
  } while (0)
  if (op == kMergeAdd) LC_MERGE(kMergeAdd);
  else if (op == kMergeMul) LC_MERGE(kMergeMul);
  else LC_MERGE(kMergeAddRelu);
#undef LC_MERGE
  return check_launch("fake_quantize_merge");
}

extern "C" int32_t lc_fake_quantize_f32(const float* x, int64_t outer, int64_t channels,
                                        int64_t inner, const float* scale, int64_t n_scale,
                                        const float* zero_point, int64_t n_zp, float host_inv_scale,
                                        float host_scale, float host_zero_point, int32_t quant_min,
                                        int32_t quant_max, float* out, float* mask_out,
                                        void* stream) {
  if (!layout_ok(outer, channels, inner)) return fail(LC_ERR_INVALID_ARG, "fake_quantize: bad layout");
  if (outer * channels * inner == 0) return LC_OK;
  if (!x || !out) return fail(LC_ERR_INVALID_ARG, "fake_quantize: null pointer");
  if (int32_t rc = check_param_counts(channels, scale, n_scale, zero_point, n_zp)) return rc;
  collapse_if_scalar(outer, channels, inner, scale, n_scale, zero_point, n_zp);
  ChannelParams p{scale, zero_point, n_scale, n_zp, host_inv_scale, host_scale, host_zero_point};
  const float qmin = static_cast<float>(quant_min), qmax = static_cast<float>(quant_max);
  cudaStream_t st = as_stream(stream);
  const int64_t segs = outer * channels;
  dim3 cgrid;
  if (columns_ok(outer, channels, inner, &cgrid) && aligned(x, 16) && aligned(out, 16) &&
      (!mask_out || aligned(mask_out, 16))) {
    fake_quantize_cols_kernel<<<cgrid, kThreads, 0, st>>>(x, out, mask_out, outer, channels * inner, inner, p, qmin, qmax);
  } else if (inner >= kSegModeMinInner || channels == 1) {
    const int cps = chunks_for(inner);
    const int64_t grid = segs * cps;
    if (grid > 0x7fffffffLL) return fail(LC_ERR_UNSUPPORTED, "tensor too large for one launch");
    const bool vec = (inner % 4 == 0) && aligned(x, 16) && aligned(out, 16) &&
                     (!mask_out || aligned(mask_out, 16));
    if (vec)
      fake_quantize_seg_kernel<true><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(
          x, out, mask_out, channels, inner, cps, p, qmin, qmax);
    else
      fake_quantize_seg_kernel<false><<<static_cast<unsigned>(grid), kThreads, 0, st>>>(
          x, out, mask_out, channels, inner, cps, p, qmin, qmax);
  } else {
    const int64_t total = segs * inner;
    fake_quantize_strided_kernel<<<strided_grid(total), kThreads, 0, st>>>(
        x, out, mask_out, total, channels, inner, p, qmin, qmax);
  }
  return check_launch("fake_quantize");
}

extern "C" int32_t lc_dynamic_quantize_rows_f32(const float* x, int64_t rows, int64_t cols,
                                                int64_t ldx, int32_t symmetric, int32_t quant_min,
                                                int32_t quant_max, int32_t is_signed, float eps,
                                                void* q_out, int32_t out_dtype, int64_t ldq,
                                                float* scale_out, float* zp_out, void* stream) {
  if (rows < 0 || cols <= 0 || ldx < cols || ldq < cols)
    return fail(LC_ERR_INVALID_ARG, "dynamic_quantize_rows: bad shape");
  if (!x || !q_out || !scale_out) return fail(LC_ERR_INVALID_ARG, "dynamic_quantize_rows: null pointer");
  QParamSpec spec = make_qparam_spec(symmetric, quant_min, quant_max, is_signed, eps);
  cudaStream_t st = as_stream(stream);
  switch (out_dtype) {
    case LC_S8:
      return launch_dynamic_rows<int8_t>(x, rows, cols, ldx, spec, static_cast<int8_t*>(q_out), ldq,
                                         scale_out, zp_out, st);
    case LC_U8:
      return launch_dynamic_rows<uint8_t>(x, rows, cols, ldx, spec, static_cast<uint8_t*>(q_out),
                                          ldq, scale_out, zp_out, st);
    case LC_S16:
      return launch_dynamic_rows<int16_t>(x, rows, cols, ldx, spec, static_cast<int16_t*>(q_out),
                                          ldq, scale_out, zp_out, st);
  }
  return fail(LC_ERR_UNSUPPORTED, "dynamic_quantize_rows: out_dtype %d not supported", out_dtype);
}

extern "C" int32_t lc_dynamic_quantize_tensor_f32(const float* x, int64_t rows, int64_t cols,
                                                  int64_t ldx, int32_t symmetric,
                                                  int32_t quant_min, int32_t quant_max,
                                                  int32_t is_signed, float eps, void* q_out,
                                                  int32_t out_dtype, int64_t ldq, float* scale_out,
                                                  float* zp_out, float* minmax_out, void* workspace,
                                                  int64_t workspace_bytes, void* stream) {
  if (rows <= 0 || cols <= 0 || ldq < cols)
    return fail(LC_ERR_INVALID_ARG, "dynamic_quantize_tensor: bad shape");
  if (ldx != cols)
    return fail(LC_ERR_UNSUPPORTED, "dynamic_quantize_tensor: input must be dense (ldx == cols)");
  if (!x || !q_out || !scale_out || !zp_out || !minmax_out)
    return fail(LC_ERR_INVALID_ARG, "dynamic_quantize_tensor: null pointer");
  QParamSpec spec = make_qparam_spec(symmetric, quant_min, quant_max, is_signed, eps);
  cudaStream_t st = as_stream(stream);
  if (rows * cols <= kSmallMaxElems && cols % 4 == 0 && aligned(x, 16) && ldq % 4 == 0 &&
      aligned(q_out, out_dtype == LC_S16 ? 8 : 4)) {
    switch (out_dtype) {
      case LC_S8:
        return launch_dynamic_quantize_small<int8_t>(x, rows, cols, spec, static_cast<int8_t*>(q_out), ldq, scale_out,
                                                     zp_out, minmax_out, st);
      case LC_U8:
        return launch_dynamic_quantize_small<uint8_t>(x, rows, cols, spec, static_cast<uint8_t*>(q_out), ldq, scale_out,
                                                      zp_out, minmax_out, st);
      case LC_S16:
        return launch_dynamic_quantize_small<int16_t>(x, rows, cols, spec, static_cast<int16_t*>(q_out), ldq, scale_out,
                                                      zp_out, minmax_out, st);
    }
    return fail(LC_ERR_UNSUPPORTED, "dynamic_quantize_tensor: out_dtype %d not supported", out_dtype);
  }
  if (int32_t rc = launch_observe_tensor(x, rows * cols, minmax_out, minmax_out + 1, 0, 1, spec,
                                         scale_out, zp_out, workspace, workspace_bytes, st))
    return rc;
  ChannelParams p{scale_out, zp_out, 1, 1, 0.0f, 0.0f, 0.0f};
  // dense output: one long segment; padded output: one segment per row
  const bool flat = (ldq == cols);
  const int64_t segs = flat ? 1 : rows, inner = flat ? rows * cols : cols;
  const int64_t is = flat ? inner : ldx, os = flat ? inner : ldq;
  switch (out_dtype) {
    case LC_S8:
      return launch_quantize<int8_t>(x, segs, 1, inner, is, os, p, spec.qmin, spec.qmax,
                                     static_cast<int8_t*>(q_out), 1, st);
    case LC_U8:
      return launch_quantize<uint8_t>(x, segs, 1, inner, is, os, p, spec.qmin, spec.qmax,
                                      static_cast<uint8_t*>(q_out), 1, st);
    case LC_S16:
      return launch_quantize<int16_t>(x, segs, 1, inner, is, os, p, spec.qmin, spec.qmax,
                                      static_cast<int16_t*>(q_out), 1, st);
  }
  return fail(LC_ERR_UNSUPPORTED, "dynamic_quantize_tensor: out_dtype %d not supported", out_dtype);
}

extern "C" int32_t lc_rowsum_s8(const int8_t* b, int64_t rows, int64_t cols, int64_t ldb,
                                int32_t* out, void* stream) {
  if (!b || !out || rows < 0 || cols < 0 || ldb < cols)
    return fail(LC_ERR_INVALID_ARG, "rowsum_s8: bad arguments");
  if (rows == 0) return LC_OK;
  const int rows_per_cta = kThreads / 32;
  rowsum_s8_kernel<<<static_cast<unsigned>((rows + rows_per_cta - 1) / rows_per_cta), kThreads, 0,
                     as_stream(stream)>>>(b, rows, cols, ldb, out);
  return check_launch("rowsum_s8");
}
