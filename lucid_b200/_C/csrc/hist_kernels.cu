// Fixed-width histogram of an fp32 tensor: the counting pass of the histogram observer
// (lucid/quantization/observer.py:852-870 calls lucid.histc once per calibration batch;
// bucketing arithmetic of lucid/_C/backend/cpu/methods/Reduction.cpp:839-888 as called from
// lucid/_C/ops/composite/Stats.cpp:48-96 and lucid/_ops/_adapters.py:1256-1279).
//
// HBM-bound: every element is read once with 16-byte loads.  Each CTA counts into a private
// shared-memory histogram (32-bit counters, one atomic per element), flushes the non-empty
// bins to 64-bit global counters, and the CTA that draws the last ticket turns the counters
// into fp32 counts (rounded once, like the reference's float64 -> input dtype cast) and
// clears them for the next call.
#include <cmath>
#include <mutex>

#include "common.cuh"

namespace lc {
namespace {

constexpr int kHistThreads = 256;
constexpr int kHistMaxBins = 16384;  // 64 KB of shared counters

// What the kernel needs to bucket one value.  The reference's arithmetic is float64
// (Reduction.cpp:858-883): skip v < lo, v > hi and NaN; bin = trunc((v - lo) / step), the
// right edge clamped into the last bin.  A float64 divide per element would make the kernel
// compute-bound at about a third of HBM bandwidth, so values are first placed in fp32:
// q32 = (v - lo32) * inv32 differs from the exact quotient by less than `delta` bins (host
// bound below), hence wherever q32 is at least delta away from every bin edge and from
// both ends of the range its integer part is the reference's bin.  Only the remaining sliver
// of values goes through the float64 formula.
struct HistSpec {
  double lo, hi, step;
  float lo32, inv32, delta, top;  // top = bins - delta
  int bins;
  int lo_exact;  // lo32 == lo: a value equal to lo32 is exactly the left end (bin 0)
};

__device__ __forceinline__ void count_one(float v, const HistSpec& h, unsigned int* sh) {
  const float q = __fmul_rn(__fsub_rn(v, h.lo32), h.inv32);
  const float fl = floorf(q);
  const float fr = q - fl;
  if (q >= h.delta && q <= h.top && fr > h.delta && fr < 1.0f - h.delta) {  // false for NaN
    atomicAdd(sh + static_cast<int>(fl), 1u);
    return;
  }
  // the left end of the range is where a ReLU's zeros (half of all activations) land
  if (v == h.lo32 && h.lo_exact) {
    atomicAdd(sh, 1u);
    return;
  }
  const double d = static_cast<double>(v);
  if (!(d >= h.lo) || d > h.hi) return;
  long long b = static_cast<long long>(__ddiv_rn(__dsub_rn(d, h.lo), h.step));
  if (b >= h.bins) b = h.bins - 1;
  atomicAdd(sh + b, 1u);
}

__global__ void __launch_bounds__(kHistThreads)
histc_kernel(const float* __restrict__ x, int64_t n, int vec_ok, const HistSpec h,
             unsigned long long* __restrict__ gcounts, unsigned int* __restrict__ ticket,
             float* __restrict__ out, int accumulate) {
  extern __shared__ unsigned int sh[];
  __shared__ int is_last;
  const int bins = h.bins;
  for (int b = threadIdx.x; b < bins; b += kHistThreads) sh[b] = 0u;
  __syncthreads();
  unsigned int* const mine = sh;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kHistThreads + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * kHistThreads;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    int64_t i = tid;
    for (; i + 3 * nthreads < n4; i += 4 * nthreads) {  // four independent 16-byte loads in flight
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcs(x4 + i + u * nthreads);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        count_one(v[u].x, h, mine);
        count_one(v[u].y, h, mine);
        count_one(v[u].z, h, mine);
        count_one(v[u].w, h, mine);
      }
    }
    for (; i < n4; i += nthreads) {
      const float4 v = __ldcs(x4 + i);
      count_one(v.x, h, mine);
      count_one(v.y, h, mine);
      count_one(v.z, h, mine);
      count_one(v.w, h, mine);
    }
    for (int64_t k = (n4 << 2) + tid; k < n; k += nthreads) count_one(x[k], h, mine);
  } else {
    for (int64_t k = tid; k < n; k += nthreads) count_one(x[k], h, mine);
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kHistThreads) {
    const unsigned int c = sh[b];
    if (c) atomicAdd(gcounts + b, static_cast<unsigned long long>(c));
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicInc(ticket, gridDim.x - 1) == gridDim.x - 1;  // wraps to 0
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int b = threadIdx.x; b < bins; b += kHistThreads) {
    const unsigned long long c = __ldcg(gcounts + b);
    gcounts[b] = 0ull;
    const float f = static_cast<float>(static_cast<double>(c));
    out[b] = accumulate ? __fadd_rn(out[b], f) : f;
  }
}

}  // namespace
}  // namespace lc

using namespace lc;

extern "C" int64_t lc_histc_workspace_bytes(int32_t bins) {
  return bins > 0 ? 16 + 8 * static_cast<int64_t>(bins) : 0;
}

extern "C" int32_t lc_histc_f32(const float* x, int64_t n, int32_t bins, double lo, double hi, float* out,
                                int32_t accumulate, void* workspace, int64_t workspace_bytes, void* stream) {
  if (bins <= 0 || bins > kHistMaxBins)
    return fail(LC_ERR_UNSUPPORTED, "histc: bins must be in [1, %d], got %d", kHistMaxBins, bins);
  if (n < 0 || !out) return fail(LC_ERR_INVALID_ARG, "histc: bad arguments");
  if (!(lo < hi) || !(hi - lo < INFINITY) || lo != lo || hi != hi)
    return fail(LC_ERR_INVALID_ARG, "histc: the range [%g, %g] must be finite and not empty", lo, hi);
  if (!workspace || workspace_bytes < lc_histc_workspace_bytes(bins) || !aligned(workspace, 16))
    return fail(LC_ERR_WORKSPACE, "histc: workspace of %lld bytes needed (16-byte aligned, zeroed once)",
                (long long)lc_histc_workspace_bytes(bins));
  if (n > 0 && !x) return fail(LC_ERR_INVALID_ARG, "histc: null input");
  cudaStream_t st = as_stream(stream);
  static std::once_flag flags[64];
  static cudaError_t results[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(LC_ERR_CUDA, "no current CUDA device");
  std::call_once(flags[dev], [&]() {
    results[dev] = cudaFuncSetAttribute(histc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHistMaxBins * 4);
  });
  if (results[dev] != cudaSuccess)
    return fail(LC_ERR_CUDA, "histc: cannot reserve shared memory: %s", cudaGetErrorString(results[dev]));
  HistSpec h;
  h.lo = lo;
  h.hi = hi;
  h.step = (hi - lo) / static_cast<double>(bins);
  h.bins = bins;
  h.lo32 = static_cast<float>(lo);
  h.inv32 = static_cast<float>(1.0 / h.step);
  // |q32 - (v - lo) / step| < 2^-24 |lo| / step (lo rounded to fp32) + 2^-24 bins (the
  // subtraction) + 2^-23 bins (inv32 and the product), for v inside the range
  const double mag = (fabs(lo) > fabs(hi) ? fabs(lo) : fabs(hi)) / h.step + bins;
  const double delta = ldexp(mag, -22) + 1e-6;
  h.delta = delta < 0.25 && h.lo32 > -INFINITY && h.inv32 < INFINITY ? static_cast<float>(delta) : 2.0f;  // 2: never fast
  h.top = static_cast<float>(bins) - h.delta;
  h.lo_exact = static_cast<double>(h.lo32) == lo ? 1 : 0;
  // enough CTAs to fill the machine a few times over, few enough that clearing and flushing
  // the shared histograms (up to 64 KB each) stays cheap
  int64_t grid = (n + kHistThreads * 16 - 1) / (kHistThreads * 16);
  const int64_t per_sm = bins * 4 <= 16 * 1024 ? 8 : (bins * 4 <= 32 * 1024 ? 4 : 2);
  const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  unsigned int* ticket = static_cast<unsigned int*>(workspace);
  unsigned long long* gcounts = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(workspace) + 16);
  histc_kernel<<<static_cast<unsigned>(grid), kHistThreads, bins * 4, st>>>(
      x, n, aligned(x, 16) ? 1 : 0, h, gcounts, ticket, out, accumulate);
  return check_launch("histc");
}
