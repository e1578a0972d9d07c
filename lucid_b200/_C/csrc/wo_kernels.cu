// Weight-only quantized Linear for decode batch sizes (HBM-bound: the weight
// matrix is read once, activations stay in floating point).
//
//  * per-output-channel symmetric int8 weights (lc_wo_linear_s8):
//      - 16-bit activations: the int8 weights are widened to bf16/f16 in
//        registers and contracted on the tensor cores with mma.sync m16n8k16
//        (weights are the 16-row operand, the batch is the 8-column operand).
//        tcgen05 needs both operands in shared memory and a 128-row tile, which
//        buys nothing for a memory-bound 1..32-column product;
//      - fp32 activations: fp32 FMA, one warp per output row;
//  * the group-wise affine format of engine.quantized.{quantize,dequantize,
//    quantized_matmul} (lucid/_C/ops/quantized/QuantizedMatmul.cpp:111-207).
#include <mutex>

#include "common.cuh"

namespace lc {

// streaming 16-byte load that does not displace the activations held in L1
__device__ __forceinline__ int4 ld_stream_v4(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// ---- int8 -> 16-bit float pairs ---------------------------------------------
// `u` holds four offset-binary bytes (s8 ^ 0x80).  Returns bytes (lo, lo+1) as a
// packed pair of XT.
template <typename XT>
__device__ __forceinline__ uint32_t widen_pair(uint32_t u, int lo);

// f16: 0x6400 | byte is 1024 + byte exactly; subtracting 1152 gives the s8 value.
template <>
__device__ __forceinline__ uint32_t widen_pair<__half>(uint32_t u, int lo) {
  const uint32_t sel = lo == 0 ? 0x7170u : 0x7372u;  // {0x64, b[lo+1], 0x64, b[lo]}
  uint32_t h = __byte_perm(u, 0x64646464u, sel);
  const uint32_t magic = 0x64806480u;  // 1152.0 in both halves
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&h), *reinterpret_cast<const __half2*>(&magic));
  return *reinterpret_cast<uint32_t*>(&r);
}

// bf16: the 16-bit pattern 0x00uu read as bf16 is exactly u * 2^-133 for every byte u (codes
// below 128 are subnormals, codes from 128 up are the smallest normals, and the two ranges
// join linearly), so two exact packed bf16 operations, x * 2^120 and then fma(x, 2^13, -128),
// give the signed weight s8 = u - 128 for two weights at once.  One byte-permute per pair
// runs on the integer pipe; the arithmetic runs on the (twice as wide) FMA pipe.
template <>
__device__ __forceinline__ uint32_t widen_pair<__nv_bfloat16>(uint32_t u, int lo) {
  const uint32_t sel = lo == 0 ? 0x4140u : 0x4342u;  // {0x00, b[lo+1], 0x00, b[lo]}
  uint32_t d = __byte_perm(u, 0u, sel);
  const uint32_t two120 = 0x7B807B80u;  // 2^120 in both halves
  const uint32_t two13 = 0x46004600u;   // 2^13
  const uint32_t m128 = 0xC300C300u;    // -128
  asm("mul.rn.bf16x2 %0, %0, %1;\n\tfma.rn.bf16x2 %0, %0, %2, %3;" : "+r"(d) : "r"(two120), "r"(two13), "r"(m128));
  return d;
}

template <typename XT>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1,
                                                         uint32_t a2, uint32_t a3, uint32_t b0,
                                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1,
                                                  uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename XT>
__device__ __forceinline__ XT from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

template <typename XT>
__device__ __forceinline__ float to_float(XT v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

// What follows the scale and the bias in the statically quantized Linear
// (lucid/nn/quantized/linear.py:206-214, lucid/nn/quantized/intrinsic.py:40): an optional ReLU and
// the fake-quantize onto the calibrated per-tensor output grid (device scalars; null = none).
struct WoEpilogue {
  int relu;
  const float* fq_scale;
  const float* fq_zp;
  float qmin, qmax;
};
__device__ __forceinline__ float wo_finish(float v, const WoEpilogue& e) {
  if (e.relu) v = v < 0.0f ? 0.0f : v;  // NaN stays
  if (e.fq_scale) {
    const float s = __ldg(e.fq_scale);
    v = fake_quant_value(v, s, __fdiv_rn(1.0f, s), __ldg(e.fq_zp), e.qmin, e.qmax);
  }
  return v;
}

// both halves of a packed 16-bit pair, widened exactly to fp32
template <typename XT>
__device__ __forceinline__ float2 unpack_pair(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack_pair<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

constexpr int kWoWarps = 8;
constexpr int kWoThreads = kWoWarps * 32;

// CTA = 16*RT output rows, the K range split over 8 warps in interleaved 64-byte
// steps (so the 8 warps together read 512 contiguous bytes of every row per
// round), NT batch tiles of 8.  Lane (g = lane/4, t = lane%4) loads 16 weight
// bytes of rows g and g+8 at k = 64*step + 16*t; MMA sub-step j consumes bytes
// 4j..4j+3 of that chunk, and the activation fragment is loaded with the same
// permutation of k, so the sum over k is unchanged.
template <typename XT, int RT, int NT>
__global__ void __launch_bounds__(kWoThreads)
wo_linear_mma_kernel(const XT* __restrict__ x, int64_t B, int64_t K, int64_t ldx,
                     const int8_t* __restrict__ w, int64_t ldw, int64_t N,
                     const float* __restrict__ sw, const float* __restrict__ bias,
                     XT* __restrict__ y, int64_t ldy, const WoEpilogue epi) {
  __shared__ float red[kWoWarps][RT * 16][NT * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * (16 * RT);
  const int64_t ksteps = (K + 63) >> 6;

  float acc[RT][NT][4];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rt][nt][i] = 0.0f;

#pragma unroll 2
  for (int64_t s = warp; s < ksteps; s += kWoWarps) {
    const int64_t k = (s << 6) + t * 16;
    const bool k_ok = k < K;  // K is a multiple of 16, so a chunk is in or out as a whole
    int4 wa[RT][2];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t row = n0 + rt * 16 + g + 8 * h;
        wa[rt][h] = (k_ok && row < N) ? ld_stream_v4(w + row * ldw + k) : make_int4(0, 0, 0, 0);
      }
    uint32_t xa[NT][8];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int64_t b = nt * 8 + g;
      if (k_ok && b < B) {
        const uint4* px = reinterpret_cast<const uint4*>(x + b * ldx + k);
        uint4 lo = __ldg(px), hi = __ldg(px + 1);
        xa[nt][0] = lo.x; xa[nt][1] = lo.y; xa[nt][2] = lo.z; xa[nt][3] = lo.w;
        xa[nt][4] = hi.x; xa[nt][5] = hi.y; xa[nt][6] = hi.z; xa[nt][7] = hi.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) xa[nt][i] = 0u;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        const int* w0 = reinterpret_cast<const int*>(&wa[rt][0]);
        const int* w1 = reinterpret_cast<const int*>(&wa[rt][1]);
        const uint32_t u0 = static_cast<uint32_t>(w0[j]) ^ 0x80808080u;
        const uint32_t u1 = static_cast<uint32_t>(w1[j]) ^ 0x80808080u;
        const uint32_t a0 = widen_pair<XT>(u0, 0), a2 = widen_pair<XT>(u0, 2);
        const uint32_t a1 = widen_pair<XT>(u1, 0), a3 = widen_pair<XT>(u1, 2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          mma_16816<XT>(acc[rt][nt], a0, a1, a2, a3, xa[nt][2 * j], xa[nt][2 * j + 1]);
      }
    }
  }

  // split-K reduction across the 8 warps, then scale + bias
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      red[warp][rt * 16 + g][nt * 8 + 2 * t] = acc[rt][nt][0];
      red[warp][rt * 16 + g][nt * 8 + 2 * t + 1] = acc[rt][nt][1];
      red[warp][rt * 16 + g + 8][nt * 8 + 2 * t] = acc[rt][nt][2];
      red[warp][rt * 16 + g + 8][nt * 8 + 2 * t + 1] = acc[rt][nt][3];
    }
  __syncthreads();
  constexpr int ROWS = RT * 16, COLS = NT * 8;
  for (int o = threadIdx.x; o < ROWS * COLS; o += kWoThreads) {
    const int r = o % ROWS, bcol = o / ROWS;
    const int64_t n = n0 + r;
    if (n < N && bcol < B) {
      float sum = 0.0f;
#pragma unroll
      for (int wp = 0; wp < kWoWarps; ++wp) sum += red[wp][r][bcol];
      float v = sum * (sw ? __ldg(sw + n) : 1.0f);
      if (bias) v += __ldg(bias + n);
      y[static_cast<int64_t>(bcol) * ldy + n] = from_float<XT>(wo_finish(v, epi));
    }
  }
}

// ---- ring variant for weight matrices that do not fit the caches ------------------------
// A persistent CTA owns a contiguous share of the matrix (see RingPlan).  A producer thread streams
// the weights into shared memory with tiled TMA loads (one 16- or 32-row x 1024-byte box per item;
// per-row 1-D bulk copies were tried first and are limited by the copy engine's per-request cost),
// so ~190 KB of loads are in flight per SM without living in registers.  Rows and columns outside the
// matrix are zero-filled by TMA.  The consumer warps split every item along K into 64-byte units (16
// warps: one unit each; 8 warps, with two CTAs per SM: two units each), hand the int8 weights to
// mma.sync m16n8k16 as 16-bit patterns (see RawOperand) and accumulate in fp32.  Activations are loaded
// by the consumer lanes themselves for one batch tile, or staged per K chunk by the producer for more.
// Row tiles are processed in passes of at most TMAX tiles so the per-warp partial sums stay in
// registers; each pass runs over all of K and ends with a split-K reduction across the warps through
// shared memory.  Every mbarrier wait is bounded; a wait that runs out records a code in g_wo_status
// and the CTA drains its copies and returns.
namespace ring {
constexpr int KC = 1024;               // bytes of K per item (and per activation chunk)
constexpr int W_PITCH = KC;            // dense TMA box rows (the 2-way bank conflict of the two
                                       // 16-byte loads per item is not measurable)
constexpr int STAGE = 16 * W_PITCH;    // 16384
constexpr int X_PITCH = KC * 2;        // activation row pitch (16-bit elements)
constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s at 2 GHz
// A CTA is one producer warp and CW consumer warps; the consumer warps split the KC bytes of an item
// row into 64-byte units, KC / (64 * CW) per warp.
//   CW = 16: one CTA per SM with all of its shared memory.
//   CW = 8:  two CTAs per SM, half the shared memory each and two units per warp.  The serial stretches
//            of a pass (activation chunk set-up, split-K reduction, epilogue, the wait for the preceding
//            grid) then overlap with the other CTA's streaming, and the CTAs of the next launch move in
//            one at a time while this launch still runs on the other half of the SM.
__host__ __device__ constexpr int threads(int cw) { return cw * 32 + 32; }
__host__ __device__ constexpr int ctas_per_sm(int cw) { return cw == 16 ? 1 : 2; }
// dynamic shared memory of a CTA; two CTAs of 115584 + 1 KB (system) + static fit into an SM's 228 KB
__host__ __device__ constexpr int smem_budget(int cw) { return cw == 16 ? 225 * 1024 : 115584; }
// split-K partials of a whole pass: [tile][warp][16 rows][pitch]; the half-size CTA has no room for padding
__host__ __device__ constexpr int red_pitch(int nt, int cw) { return cw == 16 ? nt * 8 + 1 : nt * 8; }
__host__ __device__ constexpr int red_bytes(int nt, int tmax, int cw) { return tmax * cw * 16 * red_pitch(nt, cw) * 4; }
__host__ __device__ constexpr int x_bytes(int nt, int xb) { return xb * nt * 8 * X_PITCH; }
// group-wise format: GP_STAGES slots x {scales, biases} x tmax*16 rows x (groups per K chunk) floats, filled by
// the copy engine as swizzled boxes (1 KB for their alignment, 64 bytes for the slots' mbarriers)
constexpr int GP_STAGES = 3;
__host__ __device__ constexpr int group_array_bytes(int gs, int tmax) { return gs ? tmax * 16 * (KC / gs) * 4 : 0; }
__host__ __device__ constexpr int group_bytes(int gs, int tmax) {
  return gs ? GP_STAGES * 2 * group_array_bytes(gs, tmax) + 1024 + 64 : 0;
}
// a ring stage holds `grp` vertically adjacent 16-row tiles of one K chunk, fetched by one TMA box
// (`bits` = 4: two codes per byte, so the KC elements of an item row are KC / 2 bytes and a tile half a STAGE)
__host__ __device__ constexpr int stages(int nt, int tmax, int xb, int grp, int gs, int cw, int bits = 8) {
  // 256 bytes: alignment of the ring to 128 bytes and the mbarriers (at most 2 * 9 + 2 * 3 of 8 bytes)
  return (smem_budget(cw) - 256 - red_bytes(nt, tmax, cw) - x_bytes(nt, xb) - group_bytes(gs, tmax)) /
         (STAGE * bits / 8 * grp);
}
}  // namespace ring

__device__ int g_wo_status = 0;

__device__ __forceinline__ uint32_t wo_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool wo_mbar_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  long long t0 = 0;  // the clock is only read once a first attempt has failed
  for (;;) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (t0 == 0)
      t0 = clock64();
    else if (clock64() - t0 > ring::kWaitCycles)
      return false;
  }
}
__device__ __forceinline__ void wo_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void wo_mbar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void wo_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ float wo_lds32f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 wo_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 wo_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Raw-operand scheme of the ring kernel: the offset-binary byte u = s8 + 128 is fed to the
// tensor core as the 16-bit pattern 0x00uu, which reads as u * 2^-24 in f16 and u * 2^-133 in
// bf16 (subnormals joining the first normals linearly), so widening a pair of weights is one
// byte-permute and no arithmetic.  The sum over k of x * 128 (per-lane FP32 sums of the activations for
// per-channel weights, an all-ones MMA per unit for group-wise ones) is subtracted, with the
// power-of-two scale, when the partial sums are parked: y = C1 * sum(x*u') - 128 * sum(x).  bf16
// activations are multiplied by 2^32 first (exact) so that no product falls into the fp32 subnormal
// range.
template <typename XT>
struct RawOperand;
template <>
struct RawOperand<__half> {
  static constexpr uint32_t kOnes = 0x3C003C00u;
  __device__ static float acc_scale() { return __int_as_float((127 + 24) << 23); }   // 2^24
  __device__ static float sum_scale() { return 128.0f; }
  __device__ static void prescale(uint32_t&) {}
};
template <>
struct RawOperand<__nv_bfloat16> {
  static constexpr uint32_t kOnes = 0x3F803F80u;
  __device__ static float acc_scale() { return __int_as_float((127 + 101) << 23); }  // 2^(133-32)
  __device__ static float sum_scale() { return __int_as_float((127 - 25) << 23); }   // 128 * 2^-32
  __device__ static void prescale(uint32_t& v) {
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(v) : "r"(0x4F804F80u));  // x * 2^32, exact
  }
};

// Work of the ring kernel is counted in units of (16-row tile, K chunk).  CTA c owns the contiguous unit
// range [c*U/G, (c+1)*U/G) in tile-major order and walks it as passes: a first tile it enters in the
// middle of K, runs of whole tiles (up to TMAX at a time, K outermost inside a pass so that an
// activation chunk is loaded once for all of them, tiles fetched GRP per TMA box), and a last tile it
// leaves in the middle of K.  With U a whole number of tiles per CTA (no scratch) there are only whole
// tiles.  With scratch, U/G may be fractional: every CTA then streams the same number of bytes (+-1
// unit) whatever the matrix shape, and a tile whose K range is shared by several CTAs is finished by
// whichever of them arrives last: each parks the raw sums of its K range in its own slot of the
// scratch (no atomics on data), takes a ticket of the tile, and the holder of the last ticket adds the
// slots in CTA order -- a fixed order, so results do not depend on timing -- and applies the epilogue.
struct RingPlan {
  long long units_real;   // tiles * K chunks
  long long units;        // what the CTA ranges divide: units_real, or a whole number of tiles per CTA (no scratch)
  int grid;               // G
  float* partial;         // [G][2][16*COLS] raw sums: slot 0 = a pass that starts inside its tile, 1 = one that starts it
  int* tickets;           // [tiles], zero before the launch and zero again after it
};

struct RingPass {
  int tile0, n_tiles, kc0, kc1;
  bool partial;
};

// (unit indices fit 32 bits -- the launcher refuses matrices of 2^31 units, 32 TB, and more -- and 32-bit
// divisions keep the walk off the critical path between a CTA's start and its first copy)
template <int TMAX>
struct RingWalk {
  unsigned u, u_end;
  unsigned num_kc;
  __device__ RingWalk(long long begin, long long end, int chunks)
      : u(static_cast<unsigned>(begin)), u_end(static_cast<unsigned>(end)), num_kc(static_cast<unsigned>(chunks)) {}
  __device__ bool next(RingPass& p) {
    if (u >= u_end) return false;
    const unsigned tile = u / num_kc, left = u_end - u;
    const unsigned kc0 = u - tile * num_kc;
    if (kc0 != 0 || left < num_kc) {
      const unsigned kc1 = left < num_kc - kc0 ? kc0 + left : num_kc;
      p = {static_cast<int>(tile), 1, static_cast<int>(kc0), static_cast<int>(kc1), true};
      u += kc1 - kc0;
    } else {
      unsigned nt = left / num_kc;
      nt = nt < TMAX ? nt : TMAX;
      p = {static_cast<int>(tile), static_cast<int>(nt), 0, static_cast<int>(num_kc), false};
      u += nt * num_kc;
    }
    return true;
  }
};

__device__ __forceinline__ long long ring_first_unit(long long c, long long units, int grid) { return c * units / grid; }
// the CTA whose range holds unit u
__device__ __forceinline__ int ring_owner(long long u, long long units, int grid) {
  return static_cast<int>(((u + 1) * grid + units - 1) / units - 1);
}

// XB = number of activation-chunk buffers staged in shared memory by the producer; XB = 0 (one batch
// tile): the consumer lanes load their activation fragments straight from global memory.
// GRP = row tiles per TMA box (1 or 2).  tmap_w has GRP*16-row boxes; tmap_w1 has 16-row boxes for the odd
// last tile of a pass.  (With one CTA per SM the 32-row box measured 2 % faster; with two CTAs per SM the
// 16-row box, twice as many stages deep, measured 3 % faster.)
// GS = 0: per-output-channel symmetric int8 weights (sw = one scale per row).
// GS = 64 or 128: the 8-bit group-wise affine format (lucid/_C/ops/quantized/QuantizedMatmul.cpp:143-207):
// the packed words ARE the codes as unsigned bytes in K order, `sw` / `bias` are the [N, K / GS] group
// scales and biases.  A 64-byte unit of a row lies inside one group, so the four MMAs of a unit
// give the group's raw sum, which enters the running total as s * sum(x * c) + b * sum(x) -- the second
// sum being an all-ones MMA over the unit's activations.
// CW = consumer warps per CTA (16, or 8 with two CTAs per SM): see namespace ring.
// BITS = 4 (group-wise format only): eight codes per packed word, first code in the low bits.  An item row
// is still KC elements, now KC / 2 bytes, so a 16 KB box holds two row tiles (GRP = 2); a lane reads the 8
// bytes that hold its 16 codes, masks out code pairs (c0, c4), (c1, c5), (c2, c6), (c3, c7) of each word
// -- a nibble in the low bits of a 16-bit half is the raw operand pattern as it stands -- and its
// activation fragments are permuted once per chunk to match.
// YF32: the result is written as fp32 although the activations are 16-bit (`y` then points to floats, `ldy` counts
// floats): what a caller needs who hands in an fp32 activation as bf16 addends in separate rows and adds the
// rows of the result up afterwards.
template <typename XT, int NT, int TMAX, int XB, bool SWIGLU, int GRP, int GS = 0, int CW = 16, int BITS = 8,
          bool YF32 = false>
__global__ void __launch_bounds__(ring::threads(CW), ring::ctas_per_sm(CW))
wo_linear_ring_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w1,
                      const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_gs,
                      const __grid_constant__ CUtensorMap tmap_gb,
                      const XT* __restrict__ xg, int64_t ldx,
                      int64_t B, int64_t K, int64_t N, const float* __restrict__ sw,
                      const float* __restrict__ bias, XT* __restrict__ y, int64_t ldy, const RingPlan plan,
                      int overlap, const WoEpilogue epi) {
  // XB = 0 (batches of up to 8): a warp reads 128 contiguous bytes per unit of each of its 8 batch rows;
  // the activations are L2-resident and the loads of chunk kc + 1 are issued at the top of chunk kc.
  // That takes the activation boxes out of the SM's TMA queue -- for a long-K matrix they were every
  // second request -- and gives their shared memory to the ring.
  constexpr bool XDIRECT = XB == 0;
  // direct loads of one batch tile are issued one chunk ahead; with more tiles there are no registers for a
  // second set of fragments: the loads are issued where they are needed and the other CTA of the SM streams
  // while this one waits for them
  constexpr bool XPREF = XDIRECT && NT == 1;
  constexpr int XBN = XB > 0 ? XB : 1;  // (divisor of dead code in the direct instantiation)
  static_assert(GS == 0 || GS == 64 || GS == 128, "group sizes a 64-byte unit fits into");
  static_assert(GS == 0 || !SWIGLU, "the fused SwiGLU epilogue is for per-channel weights");
  static_assert(CW == 16 || CW == 8, "16 consumer warps, or 8 with two CTAs per SM");
  using namespace ring;
  constexpr int kConsumerWarps = CW, kConsumerThreads = CW * 32;
  constexpr int U = KC / (64 * CW);  // 64-element units of an item row per warp
  constexpr int S = stages(NT, TMAX, XB, GRP, GS, CW, BITS);
  constexpr int WP = W_PITCH * BITS / 8;  // bytes of an item row
  constexpr int TSTAGE = STAGE * BITS / 8;  // bytes of one 16-row tile of an item
  constexpr int GSTAGE = TSTAGE * GRP;
  static_assert(BITS == 8 || (BITS == 4 && GS != 0), "4-bit codes come in the group-wise format only");
  static_assert(!YF32 || (GS != 0 && !SWIGLU), "fp32 results of 16-bit activations: group-wise format only");
  static_assert(S >= 3, "ring too shallow");
  static_assert(GRP == 1 || (GRP == 2 && TMAX % 2 == 0), "one or two row tiles per box");
  constexpr int COLS = NT * 8, RP = red_pitch(NT, CW);
  extern __shared__ uint8_t wo_smem_raw[];
  const uint32_t base = (wo_smem_u32(wo_smem_raw) + 127u) & ~127u;
  const uint32_t x_base = base + S * GSTAGE;
  const uint32_t red_base = x_base + x_bytes(NT, XB);
  // group scales / biases: boxes of [16 TMAX rows x groups of a K chunk] floats per array, swizzled by the copy
  // engine so that the eight rows a warp reads at one group column fall into eight different banks
  constexpr int GPC = GS ? KC / (GS ? GS : 1) : 1;  // groups per K chunk: 16 or 8
  constexpr int GA = group_array_bytes(GS, TMAX);
  const uint32_t gp_base = (red_base + red_bytes(NT, TMAX, CW) + 1023u) & ~1023u;
  const uint32_t gbar_base = gp_base + GP_STAGES * 2 * GA;
  auto gfull_bar = [&](int s) { return gbar_base + 8u * s; };
  auto gempty_bar = [&](int s) { return gbar_base + 8u * (GP_STAGES + s); };
  const uint32_t bar_base = red_base + red_bytes(NT, TMAX, CW) + group_bytes(GS, TMAX);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  auto xfull_bar = [&](int s) { return bar_base + 8u * (2 * S + s); };
  auto xempty_bar = [&](int s) { return bar_base + 8u * (2 * S + XB + s); };
  float* red = reinterpret_cast<float*>(wo_smem_raw + (red_base - wo_smem_u32(wo_smem_raw)));

  __shared__ int s_last_ticket;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the copy engine's first use of a tensor map costs a fetch of its 128 bytes: start it before anything else
  if (warp == CW && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    if (GRP > 1) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w1)) : "memory");
    if (XB > 0) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    if (GS != 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_gs)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_gb)) : "memory");
    }
  }
  const int num_kc = static_cast<int>((K + KC - 1) / KC);
  const int nb = static_cast<int>(B);
  long long u_begin = ring_first_unit(blockIdx.x, plan.units, plan.grid);
  long long u_end = ring_first_unit(blockIdx.x + 1, plan.units, plan.grid);
  u_begin = u_begin < plan.units_real ? u_begin : plan.units_real;
  u_end = u_end < plan.units_real ? u_end : plan.units_real;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(kConsumerWarps) : "memory");
    }
    for (int s = 0; s < XB; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(xfull_bar(s)), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(xempty_bar(s)), "r"(kConsumerWarps) : "memory");
    }
    for (int s = 0; s < (GS ? GP_STAGES : 0); ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gfull_bar(s)), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gempty_bar(s)), "r"(kConsumerWarps) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Programmatic dependent launch: let the next kernel on the stream be scheduled onto SMs as
  // this grid's CTAs leave them (it orders itself with griddepcontrol.wait where it needs to).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kConsumerWarps) {
    // ===================== producer =====================
    if (lane == 0) {
      int stage = 0, xi = 0, gstage = 0;
      uint32_t phase = 0, gphase = 0;
      uint32_t armed_mask = 0, armed_parity = 0, xarmed_mask = 0, xarmed_parity = 0;  // bit per stage
      uint32_t garmed_mask = 0, garmed_parity = 0;
      bool ok = true;
      // Weights do not depend on the kernel before this one: when the launch may overlap it,
      // fill the ring with the first items of the first pass (in consumption order), and only
      // then wait for the preceding grid, whose output the activations are.  Without overlap
      // the wait returns at once and loads are issued in consumption order (the first
      // activation chunk must not queue behind a ring-full of weights).
      int prefilled = 0;
      if (overlap) {
        RingWalk<TMAX> first(u_begin, u_end, num_kc);
        RingPass ps;
        if (first.next(ps)) {
          for (int kc = ps.kc0; kc < ps.kc1 && prefilled < S; ++kc)
            for (int j = 0; j < ps.n_tiles && prefilled < S; j += GRP, ++prefilled) {
              const bool whole = j + GRP <= ps.n_tiles;
              wo_mbar_expect(full_bar(prefilled), whole ? GSTAGE : TSTAGE);
              wo_tma_load_2d(base + prefilled * GSTAGE, whole ? &tmap_w : &tmap_w1, kc * (WP / 4),
                             (ps.tile0 + j) << 4, full_bar(prefilled));
              armed_mask |= 1u << prefilled;  // parity 0
            }
        }
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int issued = 0;  // weight items walked so far (the first `prefilled` are already in flight)
      RingWalk<TMAX> walk(u_begin, u_end, num_kc);
      RingPass ps;
      while (ok && walk.next(ps)) {
        for (int kc = ps.kc0; kc < ps.kc1 && ok; ++kc, ++xi) {
          const int xb = xi % XBN;
          const uint32_t xphase = static_cast<uint32_t>((xi / XBN) & 1);
          if (!XDIRECT && !wo_mbar_wait(xempty_bar(xb), xphase ^ 1u)) {
            atomicCAS(&g_wo_status, 0, 1);
            ok = false;
            break;
          }
          // group-wise format: scales and biases of the pass's rows for the groups of this chunk (rows past N
          // and groups past K read as zero)
          if (GS != 0) {
            if (!wo_mbar_wait(gempty_bar(gstage), gphase ^ 1u)) {
              atomicCAS(&g_wo_status, 0, 1);
              ok = false;
              break;
            }
            wo_mbar_expect(gfull_bar(gstage), 2 * GA);
            wo_tma_load_2d(gp_base + gstage * 2 * GA, &tmap_gs, kc * GPC, ps.tile0 << 4, gfull_bar(gstage));
            wo_tma_load_2d(gp_base + gstage * 2 * GA + GA, &tmap_gb, kc * GPC, ps.tile0 << 4, gfull_bar(gstage));
            garmed_mask |= 1u << gstage;
            garmed_parity = (garmed_parity & ~(1u << gstage)) | (gphase << gstage);
            if (++gstage == GP_STAGES) {
              gstage = 0;
              gphase ^= 1u;
            }
          }
          // activations: [COLS rows x KC elements] box of 8-byte units, rows >= B read as zero
          if (!XDIRECT) {
            wo_mbar_expect(xfull_bar(xb), COLS * X_PITCH);
            wo_tma_load_2d(x_base + xb * COLS * X_PITCH, &tmap_x, kc * (KC / 4), 0, xfull_bar(xb));
            xarmed_mask |= 1u << xb;
            xarmed_parity = (xarmed_parity & ~(1u << xb)) | (xphase << xb);
          }
          for (int j = 0; j < ps.n_tiles; j += GRP, ++issued) {
            if (issued >= prefilled) {
              if (!wo_mbar_wait(empty_bar(stage), phase ^ 1u)) {
                atomicCAS(&g_wo_status, 0, 1);
                ok = false;
                break;
              }
              const bool whole = j + GRP <= ps.n_tiles;
              wo_mbar_expect(full_bar(stage), whole ? GSTAGE : TSTAGE);
              wo_tma_load_2d(base + stage * GSTAGE, whole ? &tmap_w : &tmap_w1, kc * (WP / 4), (ps.tile0 + j) << 4,
                             full_bar(stage));
              armed_mask |= 1u << stage;
              armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
            }
            if (++stage == S) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      // do not leave while one of this CTA's bulk copies may still be landing
      for (int s = 0; s < S; ++s)
        if (armed_mask & (1u << s)) wo_mbar_wait(full_bar(s), (armed_parity >> s) & 1u);
      for (int s = 0; s < XB; ++s)
        if (xarmed_mask & (1u << s)) wo_mbar_wait(xfull_bar(s), (xarmed_parity >> s) & 1u);
      for (int s = 0; s < (GS ? GP_STAGES : 0); ++s)
        if (garmed_mask & (1u << s)) wo_mbar_wait(gfull_bar(s), (garmed_parity >> s) & 1u);
    }
  } else {
    // ===================== consumers =====================
    // nothing to do before the activations exist; the bounded waits below start counting
    // only once the preceding grid is complete
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int g = lane >> 2, t = lane & 3;
    const int kwarp = warp * (64 * U);   // first byte of this warp's units inside an item row
    const int kbase = kwarp + t * 16;    // this lane's 16 bytes of unit 0; unit u lies 64 u bytes further
    int stage = 0, xi = 0, gstage = 0;
    uint32_t phase = 0, gphase = 0;
    bool ok = true;
    RingWalk<TMAX> walk(u_begin, u_end, num_kc);
    RingPass ps;
    while (walk.next(ps)) {
      const int pass_tiles = ps.n_tiles;
      // A tile's MMAs of one unit all add into the same accumulator.  With very few accumulators per warp
      // (at most two tile x batch combinations) even and odd K steps add into separate sets that are
      // summed when the pass is parked; otherwise the MMAs of a box are issued tile-inner and the other
      // warps fill the tensor pipe between dependent instructions.
      constexpr int AS = (GS == 0 && TMAX * NT <= 2) ? 2 : 1;
      float acc[AS][TMAX][NT][4];
#pragma unroll
      for (int a = 0; a < AS; ++a)
#pragma unroll
        for (int j = 0; j < TMAX; ++j)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[a][j][nt][i] = 0.0f;
      float xlane[NT][2];  // per-channel weights: this lane's share of sum_k x[batch nt*8+g][k], two chains
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) xlane[nt][0] = xlane[nt][1] = 0.0f;

      // direct activation loads: lane (g, t) takes elements [kc * KC + kbase + 64 u, +16) of batch rows nt * 8 + g
      constexpr int XN = XDIRECT ? NT : 1;
      uint32_t xnext[XPREF ? XN : 1][U][8];
#pragma unroll
      for (int nt = 0; nt < (XPREF ? XN : 1); ++nt)
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int i = 0; i < 8; ++i) xnext[nt][u][i] = 0u;
      auto load_x = [&](int kc_for, uint32_t (&out)[XN][U][8]) {
#pragma unroll
        for (int nt = 0; nt < XN; ++nt)
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int64_t k = static_cast<int64_t>(kc_for) * KC + kbase + 64 * u;
            const int b = nt * 8 + g;
            if (kc_for >= 0 && k < K && b < nb) {
              const uint4* px = reinterpret_cast<const uint4*>(xg + static_cast<int64_t>(b) * ldx + k);
              const uint4 lo = __ldg(px), hi = __ldg(px + 1);
              out[nt][u][0] = lo.x; out[nt][u][1] = lo.y; out[nt][u][2] = lo.z; out[nt][u][3] = lo.w;
              out[nt][u][4] = hi.x; out[nt][u][5] = hi.y; out[nt][u][6] = hi.z; out[nt][u][7] = hi.w;
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) out[nt][u][i] = 0u;
            }
          }
      };
      if constexpr (XPREF) load_x(ps.kc0, xnext);

      for (int kc = ps.kc0; kc < ps.kc1 && (GS != 0 || ok); ++kc, ++xi) {
        const int xb = xi % XBN;
        const uint32_t xphase = static_cast<uint32_t>((xi / XBN) & 1);
        do {  // (a warp whose wait ran out still takes part in the barriers below)
        if (!ok) break;
        if (!XDIRECT && !wo_mbar_wait(xfull_bar(xb), xphase)) {
          atomicCAS(&g_wo_status, 0, 2);
          ok = false;
          break;
        }
        if (GS != 0 && !wo_mbar_wait(gfull_bar(gstage), gphase)) {  // this chunk's group scales and biases
          atomicCAS(&g_wo_status, 0, 2);
          ok = false;
          break;
        }
        // activation fragments of this chunk: 16 consecutive elements per unit and batch row.  Elements past
        // the end of K and batch rows past B are zero (the direct loads are guarded, the staged boxes are
        // zero-filled by the copy engine), and so are the weights past the end of K: nothing below needs a
        // guard on k.
        uint32_t xa[NT][U][8];
        if constexpr (XPREF) {
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) xa[0][u][i] = xnext[0][u][i];
          load_x(kc + 1 < ps.kc1 ? kc + 1 : -1, xnext);  // in flight while this chunk is multiplied
        } else if constexpr (XDIRECT) {
          load_x(kc, xa);
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint32_t xs = x_base + (xb * COLS + nt * 8 + g) * X_PITCH + (kbase + 64 * u) * 2;
              const uint4 lo = wo_lds128(xs), hi = wo_lds128(xs + 16);
              xa[nt][u][0] = lo.x; xa[nt][u][1] = lo.y; xa[nt][u][2] = lo.z; xa[nt][u][3] = lo.w;
              xa[nt][u][4] = hi.x; xa[nt][u][5] = hi.y; xa[nt][u][6] = hi.z; xa[nt][u][7] = hi.w;
            }
        }
        if constexpr (GS == 0) {
          // Per-channel weights: only sum_k x over the whole pass is needed (the 128 of the offset-binary
          // codes comes out once, when the pass is parked), so every lane adds up its own activations of the
          // chunk on the FP32 pipe, in two chains, and the lanes are combined at the end of the pass.
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int i = 0; i < 8; i += 2) {
                const float2 p0 = unpack_pair<XT>(xa[nt][u][i]), p1 = unpack_pair<XT>(xa[nt][u][i + 1]);
                xlane[nt][0] += p0.x + p0.y;
                xlane[nt][1] += p1.x + p1.y;
              }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) RawOperand<XT>::prescale(xa[nt][u][i]);
        if constexpr (BITS == 4) {
          // element pairs (0,1)(2,3)(4,5)(6,7) of every eight -> (0,4)(1,5)(2,6)(3,7), the order the masked
          // nibbles of a packed word come in
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int h = 0; h < 8; h += 4) {
                const uint32_t r0 = xa[nt][u][h], r1 = xa[nt][u][h + 1], r2 = xa[nt][u][h + 2], r3 = xa[nt][u][h + 3];
                xa[nt][u][h] = __byte_perm(r0, r2, 0x5410u);
                xa[nt][u][h + 1] = __byte_perm(r0, r2, 0x7632u);
                xa[nt][u][h + 2] = __byte_perm(r1, r3, 0x5410u);
                xa[nt][u][h + 3] = __byte_perm(r1, r3, 0x7632u);
              }
        }
        // group-wise weights: sum of the activations of every unit (= of a piece of one group), per batch column
        // 2t and 2t + 1, from an all-ones MMA in two chains; already scaled to sum(x)
        float xgrp[GS ? U : 1][NT][2];
        if constexpr (GS != 0) {
          const float cx = RawOperand<XT>::sum_scale() * 0.0078125f;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            float s2[2][NT][4];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
              for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) s2[a][nt][i] = 0.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int nt = 0; nt < NT; ++nt)
                mma_16816<XT>(s2[q & 1][nt], RawOperand<XT>::kOnes, RawOperand<XT>::kOnes, RawOperand<XT>::kOnes,
                              RawOperand<XT>::kOnes, xa[nt][u][2 * q], xa[nt][u][2 * q + 1]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              xgrp[u][nt][0] = (s2[0][nt][0] + s2[1][nt][0]) * cx;
              xgrp[u][nt][1] = (s2[0][nt][1] + s2[1][nt][1]) * cx;
            }
          }
        }
        // group-wise weights: scale and bias of rows g and g + 8 of tile j for the group a unit lies in come
        // from the box the copy engine wrote: rows of GPC floats whose 16-byte pieces it exchanged by row
        // (64-byte rows: piece ^= (row >> 1) & 3; 32-byte rows: piece ^= (row >> 2) & 1)
        const uint32_t gcur = gp_base + gstage * 2 * GA;
        auto group_at = [&](int row, int gcol) {
          const int piece = (gcol >> 2) ^ (GPC == 16 ? (row >> 1) & 3 : (row >> 2) & 1);
          return static_cast<uint32_t>(row * (GPC * 4) + (piece << 4) + ((gcol & 3) << 2));
        };
        auto read_group = [&](int j, int gcol, float (&out)[4]) {  // s[row g], s[row g + 8], b[row g], b[row g + 8]
          const uint32_t lo = gcur + group_at(j * 16 + g, gcol), hi = gcur + group_at(j * 16 + g + 8, gcol);
          out[0] = wo_lds32f(lo);
          out[1] = wo_lds32f(hi);
          out[2] = wo_lds32f(lo + GA);
          out[3] = wo_lds32f(hi + GA);
        };
#pragma unroll
        for (int jb = 0; jb < TMAX; jb += GRP) {
          if (jb < pass_tiles && ok) {
            if (!wo_mbar_wait(full_bar(stage), phase)) {
              atomicCAS(&g_wo_status, 0, 2);
              ok = false;
            } else {
              const uint32_t lane_src = base + stage * GSTAGE + g * WP + kbase * BITS / 8;
#pragma unroll
              for (int u = 0; u < U; ++u) {
                // weights of the box's tiles for this unit: 16 bytes of row g and of row g + 8 each; the second
                // tile of a box may be absent (odd last tile of a pass: warp-uniform skip)
                uint32_t wr[GRP][2][4];
#pragma unroll
                for (int jj = 0; jj < GRP; ++jj) {
                  uint4 w0 = make_uint4(0u, 0u, 0u, 0u), w1 = make_uint4(0u, 0u, 0u, 0u);
                  if (GRP == 1 || jb + jj < pass_tiles) {
                    if constexpr (BITS == 8) {
                      w0 = wo_lds128(lane_src + jj * TSTAGE + 64 * u);
                      w1 = wo_lds128(lane_src + jj * TSTAGE + 64 * u + 8 * WP);
                    } else {  // 16 codes = 8 bytes; .x / .y hold them, .z / .w stay unused
                      const uint2 h0 = wo_lds64(lane_src + jj * TSTAGE + 32 * u);
                      const uint2 h1 = wo_lds64(lane_src + jj * TSTAGE + 32 * u + 8 * WP);
                      w0.x = h0.x; w0.y = h0.y;
                      w1.x = h1.x; w1.y = h1.y;
                    }
                  }
                  wr[jj][0][0] = w0.x; wr[jj][0][1] = w0.y; wr[jj][0][2] = w0.z; wr[jj][0][3] = w0.w;
                  wr[jj][1][0] = w1.x; wr[jj][1][1] = w1.y; wr[jj][1][2] = w1.z; wr[jj][1][3] = w1.w;
                }
                if constexpr (GS == 0) {
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
#pragma unroll
                    for (int jj = 0; jj < GRP; ++jj) {
                      if (GRP == 1 || jb + jj < pass_tiles) {
                        const uint32_t u0 = wr[jj][0][q] ^ 0x80808080u, u1 = wr[jj][1][q] ^ 0x80808080u;
                        const uint32_t a0 = __byte_perm(u0, 0u, 0x4140u), a2 = __byte_perm(u0, 0u, 0x4342u);
                        const uint32_t a1 = __byte_perm(u1, 0u, 0x4140u), a3 = __byte_perm(u1, 0u, 0x4342u);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                          mma_16816<XT>(acc[q % AS][jb + jj][nt], a0, a1, a2, a3, xa[nt][u][2 * q], xa[nt][u][2 * q + 1]);
                      }
                    }
                  }
                } else {
                  const int gcol = (kwarp + 64 * u) / (GS ? GS : 1);
                  float gq[GRP][4];
                  float part[GRP][NT][4];
#pragma unroll
                  for (int jj = 0; jj < GRP; ++jj) {
                    read_group(jb + jj, gcol, gq[jj]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                      for (int i = 0; i < 4; ++i) part[jj][nt][i] = 0.0f;
                  }
#pragma unroll
                  for (int q = 0; q < 4; ++q) {  // the codes are unsigned bytes already
#pragma unroll
                    for (int jj = 0; jj < GRP; ++jj) {
                      if (GRP == 1 || jb + jj < pass_tiles) {
                        uint32_t a0, a1, a2, a3;
                        if constexpr (BITS == 8) {
                          a0 = __byte_perm(wr[jj][0][q], 0u, 0x4140u), a2 = __byte_perm(wr[jj][0][q], 0u, 0x4342u);
                          a1 = __byte_perm(wr[jj][1][q], 0u, 0x4140u), a3 = __byte_perm(wr[jj][1][q], 0u, 0x4342u);
                        } else {  // MMA q takes codes 4 (q & 1) .. + 3 and four further on of word q / 2
                          const uint32_t v0 = wr[jj][0][q >> 1] >> (8 * (q & 1)), v1 = wr[jj][1][q >> 1] >> (8 * (q & 1));
                          a0 = v0 & 0x000F000Fu, a2 = (v0 >> 4) & 0x000F000Fu;
                          a1 = v1 & 0x000F000Fu, a3 = (v1 >> 4) & 0x000F000Fu;
                        }
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                          mma_16816<XT>(part[jj][nt], a0, a1, a2, a3, xa[nt][u][2 * q], xa[nt][u][2 * q + 1]);
                      }
                    }
                  }
                  // raw sums -> values: sum(x c) = part * acc_scale; sum(x) is xgrp
                  const float c1 = RawOperand<XT>::acc_scale();
#pragma unroll
                  for (int jj = 0; jj < GRP; ++jj) {
                    if (GRP == 1 || jb + jj < pass_tiles) {
                      float (&tot)[NT][4] = acc[0][jb + jj];
#pragma unroll
                      for (int nt = 0; nt < NT; ++nt) {
                        const float x0 = xgrp[u][nt][0], x1 = xgrp[u][nt][1];
                        tot[nt][0] = fmaf(part[jj][nt][0] * c1, gq[jj][0], fmaf(x0, gq[jj][2], tot[nt][0]));
                        tot[nt][1] = fmaf(part[jj][nt][1] * c1, gq[jj][0], fmaf(x1, gq[jj][2], tot[nt][1]));
                        tot[nt][2] = fmaf(part[jj][nt][2] * c1, gq[jj][1], fmaf(x0, gq[jj][3], tot[nt][2]));
                        tot[nt][3] = fmaf(part[jj][nt][3] * c1, gq[jj][1], fmaf(x1, gq[jj][3], tot[nt][3]));
                      }
                    }
                  }
                }
              }
              // The slot goes back to the copy engine, which writes it through the async proxy: order this warp's
              // (generic-proxy) reads of the slot before that.  The release of the arrive alone was observed not
              // to be enough -- a form of this kernel with twice the MMAs per box read, on launches that found
              // nothing in the L2, bytes of the box that came six chunks later; with this fence it does not.
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) wo_mbar_arrive(empty_bar(stage));
              if (++stage == S) {
                stage = 0;
                phase ^= 1u;
              }
            }
          }
        }
        if (!XDIRECT) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // as for the weight slots
        __syncwarp();
        if (!XDIRECT && lane == 0 && ok) wo_mbar_arrive(xempty_bar(xb));
        } while (false);
        if (GS != 0) {  // the slot of the group parameters goes back to the copy engine (as for the weight slots)
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) wo_mbar_arrive(gempty_bar(gstage));
          if (++gstage == GP_STAGES) {
            gstage = 0;
            gphase ^= 1u;
          }
        }
      }

      // ---- split-K reduction of this pass across the consumer warps ----
      // every warp parks its partial sums of all tiles of the pass, one barrier, then the
      // consumer threads add the partials of each output in a fixed order (deterministic)
      //
      // The scales and biases of the outputs this thread will finish are requested first: their latency
      // (global memory, about a microsecond under load) passes while the sums are parked.
      constexpr int OUT_ROWS = SWIGLU ? 8 : 16, HALVES = SWIGLU ? 2 : 1;
      constexpr int PT = (TMAX * OUT_ROWS * COLS + kConsumerThreads - 1) / kConsumerThreads;
      float p_scale[PT][HALVES], p_bias[PT][HALVES];
      if constexpr (GS == 0) {
#pragma unroll
        for (int i = 0; i < PT; ++i) {
          const int o = threadIdx.x + i * kConsumerThreads;
          const int r = o % OUT_ROWS, j = (o / OUT_ROWS) / COLS;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const int64_t n = ((static_cast<int64_t>(ps.tile0) + j) << 4) + r + 8 * h;
            const bool live = j < pass_tiles && n < N;
            p_scale[i][h] = (live && sw) ? __ldg(sw + n) : 1.0f;
            p_bias[i][h] = (live && bias) ? __ldg(bias + n) : 0.0f;
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");  // previous pass fully summed
      // sum_k x of this warp's K slices for the batch columns 2t and 2t+1 this lane's accumulators belong to:
      // the lane sums (batch row g, slice t) are added over the quad, then fetched from quads 2t and 2t+1
      float xcol[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float sq = xlane[nt][0] + xlane[nt][1];
        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
        xcol[nt][0] = __shfl_sync(0xffffffffu, sq, (2 * t) * 4);
        xcol[nt][1] = __shfl_sync(0xffffffffu, sq, (2 * t + 1) * 4);
      }
#pragma unroll
      for (int j = 0; j < TMAX; ++j) {
        if (j < pass_tiles) {
          float* mine = red + (j * kConsumerWarps + warp) * 16 * RP;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            // per-channel weights: raw sums -> sum(x * s8), the offset 128 * sum(x) taken out once per pass
            const float c1 = GS ? 1.0f : RawOperand<XT>::acc_scale(), c2 = GS ? 0.0f : 128.0f;
            float a4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a4[i] = AS == 2 ? acc[0][j][nt][i] + acc[AS - 1][j][nt][i] : acc[0][j][nt][i];
            const float x0 = xcol[nt][0], x1 = xcol[nt][1];
            mine[g * RP + nt * 8 + 2 * t] = a4[0] * c1 - x0 * c2;
            mine[g * RP + nt * 8 + 2 * t + 1] = a4[1] * c1 - x1 * c2;
            mine[(g + 8) * RP + nt * 8 + 2 * t] = a4[2] * c1 - x0 * c2;
            mine[(g + 8) * RP + nt * 8 + 2 * t + 1] = a4[3] * c1 - x1 * c2;
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");

      // For a pass over part of K: park the CTA's raw sums in its scratch slot, take a ticket of
      // the tile, and go on only if every other CTA that shares the tile has already parked its own.
      constexpr int kSlotFloats = 16 * COLS;
      int n_sharers = 1, first_sharer = 0;
      bool finish = true;
      if (ps.partial) {
        const long long box_first = static_cast<long long>(ps.tile0) * num_kc;
        first_sharer = ring_owner(box_first, plan.units, plan.grid);
        n_sharers = ring_owner(box_first + num_kc - 1, plan.units, plan.grid) - first_sharer + 1;
        float* slot = plan.partial + (static_cast<size_t>(blockIdx.x) * 2 + (u_begin > box_first ? 0 : 1)) * kSlotFloats;
        {
          for (int o = threadIdx.x; o < pass_tiles * 16 * COLS; o += kConsumerThreads) {
            const int r = o & 15, bcol = (o >> 4) % COLS, j = (o >> 4) / COLS;
            const float* src = red + j * kConsumerWarps * 16 * RP + r * RP + bcol;
            float sum = 0.0f;
#pragma unroll
            for (int wp = 0; wp < kConsumerWarps; ++wp) sum += src[wp * 16 * RP];
            slot[(j * 16 + r) * COLS + bcol] = sum;
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
        if (threadIdx.x == 0) {
          const int old = atomicAdd(plan.tickets + ps.tile0, 1);
          s_last_ticket = old == n_sharers - 1;
          if (old == n_sharers - 1) plan.tickets[ps.tile0] = 0;  // every sharer has drawn: ready for the next launch
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
        finish = s_last_ticket != 0;
        if (finish) __threadfence();
      }
      if (finish) {
        // sum over the consumer warps (a pass over all of K) or over the sharers' slots, in CTA order
        auto total = [&](int j, int r, int bcol) -> float {
          if (!ps.partial) {
            const float* src = red + j * kConsumerWarps * 16 * RP + r * RP + bcol;
            float sum = 0.0f;
#pragma unroll
            for (int wp = 0; wp < kConsumerWarps; ++wp) sum += src[wp * 16 * RP];
            return sum;
          }
          float sum = 0.0f;
          for (int c = 0; c < n_sharers; ++c) {
            const long long cta = first_sharer + c;
            const int which = ring_first_unit(cta, plan.units, plan.grid) > static_cast<long long>(ps.tile0) * num_kc ? 0 : 1;
            sum += __ldcg(plan.partial + (static_cast<size_t>(cta) * 2 + which) * kSlotFloats + (j * 16 + r) * COLS + bcol);
          }
          return sum;
        };
#pragma unroll
        for (int i = 0; i < PT; ++i) {
          const int o = threadIdx.x + i * kConsumerThreads;
          if (o < pass_tiles * OUT_ROWS * COLS) {
            const int r = o % OUT_ROWS, bcol = (o / OUT_ROWS) % COLS, j = (o / OUT_ROWS) / COLS;
            const int64_t tile = static_cast<int64_t>(ps.tile0) + j;
            if constexpr (SWIGLU) {
              // rows r and r+8 of a tile are the gate and the up projection of the same hidden unit:
              // out[b, 8*tile + r] = silu(gate) * up, one rounding to the activation type
              const int64_t nu = (tile << 4) + r + 8, h = (tile << 3) + r;
              if (nu < N && bcol < nb) {
                float gv = __fmul_rn(total(j, r, bcol), p_scale[i][0]);
                float uv = __fmul_rn(total(j, r + 8, bcol), p_scale[i][HALVES - 1]);
                if (bias) {
                  gv = __fadd_rn(gv, p_bias[i][0]);
                  uv = __fadd_rn(uv, p_bias[i][HALVES - 1]);
                }
                y[static_cast<int64_t>(bcol) * ldy + h] = from_float<XT>(gv / (1.0f + __expf(-gv)) * uv);
              }
            } else {
              const int64_t n = (tile << 4) + r;
              if (n < N && bcol < nb) {
                float v = total(j, r, bcol);
                if constexpr (GS == 0) {
                  v = __fmul_rn(v, p_scale[i][0]);
                  if (bias) v = __fadd_rn(v, p_bias[i][0]);
                }
                if constexpr (YF32)
                  reinterpret_cast<float*>(y)[static_cast<int64_t>(bcol) * ldy + n] = wo_finish(v, epi);
                else
                  y[static_cast<int64_t>(bcol) * ldy + n] = from_float<XT>(wo_finish(v, epi));
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
}

// generic path (any activation type, any K): one warp per output row, fp32 FMA,
// the batch handled in chunks of BT
template <typename XT, int BT>
__global__ void __launch_bounds__(kWoThreads)
wo_linear_fma_kernel(const XT* __restrict__ x, int64_t B, int64_t K, int64_t ldx,
                     const int8_t* __restrict__ w, int64_t ldw, int64_t N,
                     const float* __restrict__ sw, const float* __restrict__ bias,
                     XT* __restrict__ y, int64_t ldy, const WoEpilogue epi) {
  const int lane = threadIdx.x & 31;
  const int64_t n = static_cast<int64_t>(blockIdx.x) * kWoWarps + (threadIdx.x >> 5);
  if (n >= N) return;
  const int8_t* wr = w + n * ldw;
  for (int64_t b0 = 0; b0 < B; b0 += BT) {
    float acc[BT];
#pragma unroll
    for (int i = 0; i < BT; ++i) acc[i] = 0.0f;
    for (int64_t k = lane; k < K; k += 32) {
      const float wv = static_cast<float>(wr[k]);
#pragma unroll
      for (int i = 0; i < BT; ++i)
        if (b0 + i < B) acc[i] = fmaf(to_float<XT>(x[(b0 + i) * ldx + k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < BT; ++i) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
      if (lane == 0 && b0 + i < B) {
        float v = acc[i] * (sw ? __ldg(sw + n) : 1.0f);
        if (bias) v += __ldg(bias + n);
        y[(b0 + i) * ldy + n] = from_float<XT>(wo_finish(v, epi));
      }
    }
  }
}

// ---- group-wise affine format -------------------------------------------------
// one thread per packed 32-bit word; the threads of a group reduce min/max with
// shuffles (a group spans gs / (32/bits) in {4, 8, 16, 32} adjacent lanes)
template <int BITS>
__global__ void __launch_bounds__(256)
group_quantize_kernel(const float* __restrict__ w, int64_t words_total, int words_per_row, int64_t K,
                      int group_size, uint32_t* __restrict__ packed, float* __restrict__ scales,
                      float* __restrict__ biases) {
  constexpr int PER = 32 / BITS;
  const int64_t word = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = word < words_total;
  const int64_t row = live ? word / words_per_row : 0;
  const int wcol = live ? static_cast<int>(word % words_per_row) : 0;
  float v[PER];
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = live ? __ldg(w + row * K + static_cast<int64_t>(wcol) * PER + i) : 0.0f;
    if (live) {
      mn = fminf(mn, v[i]);
      mx = fmaxf(mx, v[i]);
    }
  }
  const int lanes = group_size / PER;  // power of two, <= 32; groups never straddle a warp
  for (int o = lanes >> 1; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (!live) return;
  const float levels = static_cast<float>((1 << BITS) - 1);
  const float scale = __fdiv_rn(__fsub_rn(mx, mn), levels);
  const float safe = scale > 0.0f ? scale : 1.0f;
  uint32_t word_bits = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float tq = rintf(__fdiv_rn(__fsub_rn(v[i], mn), safe));
    tq = fminf(fmaxf(tq, 0.0f), levels);
    word_bits |= static_cast<uint32_t>(__float2int_rn(tq)) << (BITS * i);
  }
  packed[word] = word_bits;
  const int64_t first = static_cast<int64_t>(wcol) * PER;
  if (first % group_size == 0) {
    const int64_t gidx = row * (K / group_size) + first / group_size;
    scales[gidx] = scale;
    biases[gidx] = mn;
  }
}

template <int BITS>
__global__ void __launch_bounds__(256)
group_dequantize_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scales,
                        const float* __restrict__ biases, int64_t words_total, int words_per_row,
                        int64_t K, int group_size, float* __restrict__ out) {
  constexpr int PER = 32 / BITS;
  const int64_t word = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (word >= words_total) return;
  const int64_t row = word / words_per_row;
  const int64_t first = (word % words_per_row) * PER;
  const int64_t gidx = row * (K / group_size) + first / group_size;
  const float s = __ldg(scales + gidx), b = __ldg(biases + gidx);
  const uint32_t bits = __ldg(packed + word);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const float c = static_cast<float>((bits >> (BITS * i)) & ((1u << BITS) - 1u));
    out[row * K + first + i] = __fadd_rn(__fmul_rn(c, s), b);
  }
}

// N consecutive elements starting at an address aligned to N elements, as floats
template <typename XT, int N>
__device__ __forceinline__ void load_run(const XT* p, float (&out)[N]);
template <>
__device__ __forceinline__ void load_run<float, 4>(const float* p, float (&o)[4]) {
  const float4 v = __ldg(reinterpret_cast<const float4*>(p));
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <>
__device__ __forceinline__ void load_run<float, 8>(const float* p, float (&o)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <typename XT, int N>
__device__ __forceinline__ void load_run(const XT* p, float (&o)[N]) {  // 16-bit types
  static_assert(sizeof(XT) == 2 && (N == 4 || N == 8), "unsupported run");
  XT tmp[N];
  if (N == 4) {
    *reinterpret_cast<uint2*>(tmp) = __ldg(reinterpret_cast<const uint2*>(p));
  } else {
    *reinterpret_cast<uint4*>(tmp) = __ldg(reinterpret_cast<const uint4*>(p));
  }
#pragma unroll
  for (int e = 0; e < N; ++e) o[e] = to_float<XT>(tmp[e]);
}

// y[b,n] = sum_k x[b,k] * (c[n,k]*s + bias): one warp per output row, lanes stride
// over packed words, fp32 accumulation, batch in chunks of BT
template <typename XT, int BITS, int BT>
__global__ void __launch_bounds__(kWoThreads)
group_matmul_kernel(const XT* __restrict__ x, int64_t B, int64_t K, const uint32_t* __restrict__ packed,
                    const float* __restrict__ scales, const float* __restrict__ biases, int64_t N,
                    int group_size, XT* __restrict__ y) {
  constexpr int PER = 32 / BITS;
  const int lane = threadIdx.x & 31;
  const int64_t n = static_cast<int64_t>(blockIdx.x) * kWoWarps + (threadIdx.x >> 5);
  if (n >= N) return;
  const int64_t words = K / PER;
  const int64_t groups = K / group_size;
  const uint32_t* pr = packed + n * words;
  // batch tiles of BT are spread over blockIdx.y: they run concurrently, the 1 MB-scale
  // weight is re-read from L2
  for (int64_t b0 = static_cast<int64_t>(blockIdx.y) * BT; b0 < B; b0 += static_cast<int64_t>(gridDim.y) * BT) {
    float acc[BT];
#pragma unroll
    for (int i = 0; i < BT; ++i) acc[i] = 0.0f;
    for (int64_t wd = lane; wd < words; wd += 32) {
      const uint32_t bits = __ldg(pr + wd);
      const int64_t k0 = wd * PER;
      const int64_t gidx = n * groups + k0 / group_size;
      const float s = __ldg(scales + gidx), bb = __ldg(biases + gidx);
      float wv[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e)
        wv[e] = fmaf(static_cast<float>((bits >> (BITS * e)) & ((1u << BITS) - 1u)), s, bb);
      // PER (4 or 8) consecutive activations of each batch row with 16-byte loads; all loads
      // of the tile are issued before the first FMA needs one
      float xv[BT][PER];
#pragma unroll
      for (int i = 0; i < BT; ++i) {
        if (b0 + i < B) {
          load_run<XT, PER>(x + (b0 + i) * K + k0, xv[i]);
        } else {
#pragma unroll
          for (int e = 0; e < PER; ++e) xv[i][e] = 0.0f;
        }
      }
#pragma unroll
      for (int i = 0; i < BT; ++i)
#pragma unroll
        for (int e = 0; e < PER; ++e) acc[i] = fmaf(xv[i][e], wv[e], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < BT; ++i) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
      if (lane == 0 && b0 + i < B) y[(b0 + i) * N + n] = from_float<XT>(acc[i]);
    }
  }
}

// ---- launchers ------------------------------------------------------------------
template <typename XT>
static int32_t launch_wo_mma(const XT* x, int64_t B, int64_t K, int64_t ldx, const int8_t* w,
                             int64_t ldw, int64_t N, const float* sw, const float* bias, XT* y,
                             int64_t ldy, const WoEpilogue& epi, cudaStream_t st) {
  // enough CTAs to cover every SM at least twice before widening the row tile
  const bool wide = (N / 32) >= 2 * static_cast<int64_t>(sm_count());
  const int rows = wide ? 32 : 16;
  const unsigned grid = static_cast<unsigned>((N + rows - 1) / rows);
#define LC_WO(RT, NT) \
  wo_linear_mma_kernel<XT, RT, NT><<<grid, kWoThreads, 0, st>>>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, epi)
  if (wide) {
    if (B <= 8) LC_WO(2, 1);
    else if (B <= 16) LC_WO(2, 2);
    else LC_WO(2, 4);
  } else {
    if (B <= 8) LC_WO(1, 1);
    else if (B <= 16) LC_WO(1, 2);
    else LC_WO(1, 4);
  }
#undef LC_WO
  return check_launch("wo_linear_s8 (mma)");
}

// scratch of the balanced schedule: per CTA two slots of raw sums, then one ticket per tile
struct RingScratch {
  void* ptr;
  int64_t bytes;
};
constexpr int64_t kRingSlotBytes = 16 * 32 * 4;  // 16 rows * largest COLS floats

template <typename XT, int NT, int TMAX, int XB, bool SWIGLU, int GRP, int GS = 0, int CW = 16, int BITS = 8,
          bool YF32 = false>
static int32_t launch_wo_ring_inst(const XT* x, int64_t B, int64_t K, int64_t ldx, const int8_t* w,
                                   int64_t ldw, int64_t N, const float* sw, const float* bias, XT* y,
                                   int64_t ldy, bool overlap, const WoEpilogue& epi, const RingScratch& scratch,
                                   cudaStream_t st) {
  auto kernel = wo_linear_ring_kernel<XT, NT, TMAX, XB, SWIGLU, GRP, GS, CW, BITS, YF32>;
  static std::once_flag flags[64];
  static cudaError_t results[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(LC_ERR_CUDA, "no current CUDA device");
  std::call_once(flags[dev], [&]() {
    results[dev] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ring::smem_budget(CW));
    if (results[dev] == cudaSuccess && ring::ctas_per_sm(CW) > 1)  // room for both CTAs of an SM
      results[dev] = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  });
  if (results[dev] != cudaSuccess)
    return fail(LC_ERR_CUDA, "wo_linear_s8: cannot reserve shared memory: %s", cudaGetErrorString(results[dev]));
  // weights as [N, K/4] 4-byte units (box 256 x 16*GRP = 1024 bytes x 16*GRP rows), activations as
  // [B, K/4] 8-byte units (box 256 x COLS = 2048 bytes per row)
  CUtensorMap map_w, map_w1, map_x;
  // (K and ldw count elements; a row of 4-bit codes is half as many bytes)
  if (int32_t rc = encode_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, w, static_cast<uint64_t>(K * BITS / 32),
                                        static_cast<uint64_t>(N), static_cast<uint64_t>(ldw * BITS / 8),
                                        ring::KC * BITS / 32, 16 * GRP, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (int32_t rc = encode_tensor_map_2d(&map_w1, CU_TENSOR_MAP_DATA_TYPE_UINT32, w, static_cast<uint64_t>(K * BITS / 32),
                                        static_cast<uint64_t>(N), static_cast<uint64_t>(ldw * BITS / 8),
                                        ring::KC * BITS / 32, 16, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (int32_t rc = encode_tensor_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_INT64, x, static_cast<uint64_t>(K / 4),
                                        static_cast<uint64_t>(B), static_cast<uint64_t>(ldx) * 2, ring::KC / 4,
                                        NT * 8, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  // group-wise format: sw / bias are the [N, K / GS] scales and biases; a box is the groups of one K chunk for the
  // rows of a whole pass, swizzled for conflict-free reads (other formats: placeholders, never dereferenced)
  CUtensorMap map_gs = map_w, map_gb = map_w;
  if (GS != 0) {
    const uint64_t n_groups = static_cast<uint64_t>(K / (GS ? GS : 1));
    const CUtensorMapSwizzle swz = GS == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    if (int32_t rc = encode_tensor_map_2d(&map_gs, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, sw, n_groups, static_cast<uint64_t>(N),
                                          n_groups * 4, ring::KC / (GS ? GS : 1), 16 * TMAX, swz))
      return rc;
    if (int32_t rc = encode_tensor_map_2d(&map_gb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, bias, n_groups, static_cast<uint64_t>(N),
                                          n_groups * 4, ring::KC / (GS ? GS : 1), 16 * TMAX, swz))
      return rc;
  }
  const int64_t tiles = (N + 15) / 16;
  const int64_t num_kc = (K + ring::KC - 1) / ring::KC;
  const int64_t sms = static_cast<int64_t>(sm_count()) * ring::ctas_per_sm(CW);  // CTAs resident at once
  RingPlan plan;
  plan.units_real = tiles * num_kc;
  if (plan.units_real >= (int64_t{1} << 31))
    return fail(LC_ERR_UNSUPPORTED, "wo_linear_s8 (ring): %lld (tile, K chunk) units exceed 2^31", (long long)plan.units_real);
  const int64_t need = sms * 2 * kRingSlotBytes + tiles * 4;
  if (scratch.ptr && scratch.bytes >= need && aligned(scratch.ptr, 16)) {
    // every CTA the same number of (tile, K chunk) units, tiles shared along K where ranges meet
    plan.grid = static_cast<int>(plan.units_real < sms ? plan.units_real : sms);
    plan.units = plan.units_real;
    plan.partial = static_cast<float*>(scratch.ptr);
    plan.tickets = reinterpret_cast<int*>(static_cast<uint8_t*>(scratch.ptr) + sms * 2 * kRingSlotBytes);
  } else {
    // no scratch: whole tiles only, the same number for every CTA.  (Filling every resident CTA slot with
    // counts at most one apart -- 296 CTAs of 6 or 7 tiles instead of 256 of 7 for the decode MLP's gate / up
    // matrix -- measured 1.0-1.4 us SLOWER at batches of up to 8, equal at 16: the shorter second passes cost
    // more than the idle slots, which the next launch's CTAs use to prefetch.)
    const int64_t per = (tiles + sms - 1) / sms;
    plan.grid = static_cast<int>((tiles + per - 1) / per);
    plan.units = plan.grid * per * num_kc;
    plan.partial = nullptr;
    plan.tickets = nullptr;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
  cfg.blockDim = dim3(ring::threads(CW));
  cfg.dynamicSmemBytes = ring::smem_budget(CW);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, map_w, map_w1, map_x, map_gs, map_gb, x, ldx, B, K, N, sw, bias, y, ldy, plan,
                                             overlap ? 1 : 0, epi);
  if (err != cudaSuccess) return fail(LC_ERR_CUDA, "wo_linear_s8 (ring): %s", cudaGetErrorString(err));
  return check_launch("wo_linear_s8 (ring)");
}

template <typename XT, bool SWIGLU = false>
static int32_t launch_wo_tma(const XT* x, int64_t B, int64_t K, int64_t ldx, const int8_t* w, int64_t ldw,
                             int64_t N, const float* sw, const float* bias, XT* y, int64_t ldy,
                             bool overlap, const WoEpilogue& epi, const RingScratch& scratch, cudaStream_t st) {
  const int64_t tiles = (N + 15) / 16, sms = sm_count();
  // Batches of up to 8: two half-size CTAs per SM (8 consumer warps, two 64-byte units per warp and row), 16-row
  // boxes through a six-deep ring.  One row tile per CTA (short, wide matrices) keeps even and odd K steps in
  // separate accumulators; otherwise passes of up to four tiles.  Measured on the decode MLP (batch 1, us): 34.7
  // so, 35.9 with 32-row boxes three deep, 38.4 with passes of eight tiles (register spills), 38.9 with one
  // full-size CTA per SM.
  if (B <= 8) {
    const bool single = (tiles + 2 * sms - 1) / (2 * sms) <= 1;
    return single ? launch_wo_ring_inst<XT, 1, 1, 0, SWIGLU, 1, 0, 8>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st)
                  : launch_wo_ring_inst<XT, 1, 4, 0, SWIGLU, 1, 0, 8>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st);
  }
  // Batches of 9..16 with many row tiles per CTA: the same two-CTA form with two batch tiles (measured on the
  // fused gate / up pass of the decode MLP: 31.2 us against 35.1 us for the form below).  Otherwise one CTA
  // per SM with the activations staged in shared memory; few row tiles per CTA get a small reduction buffer
  // and more activation chunks in flight.
  const bool few = (tiles + sms - 1) / sms <= 2;
  if (B <= 16)  // many tiles per CTA: the two-CTA form with two batch tiles (activation fragments loaded where needed)
    return few ? launch_wo_ring_inst<XT, 2, 2, 3, SWIGLU, 1>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st)
               : launch_wo_ring_inst<XT, 2, 4, 0, SWIGLU, 1, 0, 8>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st);
  // 17..32 rows: two passes over the weights with at most 16 rows each (measured on the decode MLP at batch 32:
  // 97 us against 128 us for one pass with four batch tiles, whose passes hold a single row tile).  The
  // second launch reads nothing the first one writes, so it may always prefetch its weights under it.
  if (int32_t rc = launch_wo_tma<XT, SWIGLU>(x, 16, K, ldx, w, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st)) return rc;
  return launch_wo_tma<XT, SWIGLU>(x + 16 * ldx, B - 16, K, ldx, w, ldw, N, sw, bias, y + 16 * ldy, ldy, true, epi, scratch, st);
}

template <typename XT>
static int32_t launch_wo_fma(const XT* x, int64_t B, int64_t K, int64_t ldx, const int8_t* w,
                             int64_t ldw, int64_t N, const float* sw, const float* bias, XT* y,
                             int64_t ldy, const WoEpilogue& epi, cudaStream_t st) {
  const unsigned grid = static_cast<unsigned>((N + kWoWarps - 1) / kWoWarps);
  if (B <= 1)
    wo_linear_fma_kernel<XT, 1><<<grid, kWoThreads, 0, st>>>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, epi);
  else if (B <= 4)
    wo_linear_fma_kernel<XT, 4><<<grid, kWoThreads, 0, st>>>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, epi);
  else
    wo_linear_fma_kernel<XT, 8><<<grid, kWoThreads, 0, st>>>(x, B, K, ldx, w, ldw, N, sw, bias, y, ldy, epi);
  return check_launch("wo_linear_s8 (fma)");
}

template <typename XT>
static int32_t wo_linear_typed(const void* x, int64_t B, int64_t K, int64_t ldx, const int8_t* w,
                               int64_t ldw, int64_t N, const float* sw, const float* bias, void* y,
                               int64_t ldy, bool overlap, const WoEpilogue& epi, const RingScratch& scratch,
                               cudaStream_t st) {
  const XT* xt = static_cast<const XT*>(x);
  XT* yt = static_cast<XT*>(y);
  const bool mma_ok = sizeof(XT) == 2 && K % 16 == 0 && ldw % 16 == 0 && ldx % 8 == 0 &&
                      aligned(w, 16) && aligned(x, 16);
  for (int64_t b0 = 0; b0 < B; b0 += 32) {
    const int64_t bc = (B - b0 < 32) ? (B - b0) : 32;
    int32_t rc;
    if constexpr (sizeof(XT) == 2) {
      // weights beyond a few MB are streamed through the shared-memory ring; small ones
      // are latency-bound and use the direct-load kernel
      const bool big = N * K >= (int64_t{4} << 20);
      rc = !mma_ok ? launch_wo_fma<XT>(xt + b0 * ldx, bc, K, ldx, w, ldw, N, sw, bias, yt + b0 * ldy, ldy, epi, st)
           : big   ? launch_wo_tma<XT>(xt + b0 * ldx, bc, K, ldx, w, ldw, N, sw, bias, yt + b0 * ldy, ldy, overlap, epi, scratch, st)
                   : launch_wo_mma<XT>(xt + b0 * ldx, bc, K, ldx, w, ldw, N, sw, bias, yt + b0 * ldy, ldy, epi, st);
    } else {
      rc = launch_wo_fma<XT>(xt + b0 * ldx, bc, K, ldx, w, ldw, N, sw, bias, yt + b0 * ldy, ldy, epi, st);
    }
    if (rc) return rc;
  }
  return LC_OK;
}

template <typename XT, int BITS>
static int32_t launch_group_matmul(const XT* x, int64_t B, int64_t K, const uint32_t* packed,
                                   const float* scales, const float* biases, int64_t N, int gs, XT* y,
                                   cudaStream_t st) {
  const unsigned gx = static_cast<unsigned>((N + kWoWarps - 1) / kWoWarps);
  if (B <= 1) {
    group_matmul_kernel<XT, BITS, 1><<<gx, kWoThreads, 0, st>>>(x, B, K, packed, scales, biases, N, gs, y);
  } else if (B <= 4) {
    group_matmul_kernel<XT, BITS, 4><<<gx, kWoThreads, 0, st>>>(x, B, K, packed, scales, biases, N, gs, y);
  } else {
    const dim3 grid(gx, static_cast<unsigned>((B + 7) / 8 < 64 ? (B + 7) / 8 : 64));
    group_matmul_kernel<XT, BITS, 8><<<grid, kWoThreads, 0, st>>>(x, B, K, packed, scales, biases, N, gs, y);
  }
  return check_launch("group_matmul");
}

// Group-wise weights of a few MB and more on the streaming kernel (16-bit activations; 8-bit or 4-bit codes
// in groups of 64 or 128): the packed words are the codes in K order, so the
// weight is streamed exactly like a per-channel int8 matrix -- an item row of 1024 elements being 1024 or
// 512 bytes -- and the group scales / biases are read by the consumer warps.
template <typename XT, int GS, int BITS, bool YF32 = false>
static int32_t launch_group_ring(const XT* x, int64_t B, int64_t K, const uint8_t* codes, const float* scales,
                                 const float* biases, int64_t N, XT* y, bool overlap, const RingScratch& scratch,
                                 cudaStream_t st) {
  const WoEpilogue none = {0, nullptr, nullptr, 0.0f, 0.0f};
  const int8_t* w = reinterpret_cast<const int8_t*>(codes);
  const int64_t tiles = (N + 15) / 16, sms = sm_count();
  const bool few = (tiles + sms - 1) / sms <= 2;
  // row r of the result (fp32 results: `y` points to floats)
  auto yrow = [&](int64_t r) {
    return YF32 ? reinterpret_cast<XT*>(reinterpret_cast<float*>(y) + r * N) : y + r * N;
  };
  for (int64_t b0 = 0; b0 < B; b0 += 32) {
    const int64_t bc = B - b0 < 32 ? B - b0 : 32;
    const XT* xb = x + b0 * K;
    XT* yb = yrow(b0);
    int32_t rc;
    if constexpr (BITS == 4) {
      // 16 KB boxes of two row tiles; up to 8 rows on two half-size CTAs per SM, 9..16 with the activations
      // staged in shared memory, more as two such passes
      (void)few;
      if (bc <= 8) {
        rc = launch_wo_ring_inst<XT, 1, 4, 0, false, 2, GS, 8, 4, YF32>(xb, bc, K, K, w, K, N, scales, biases, yb, N, overlap, none, scratch, st);
      } else {
        const int64_t first = bc < 16 ? bc : 16;
        rc = launch_wo_ring_inst<XT, 2, 4, 2, false, 2, GS, 16, 4, YF32>(xb, first, K, K, w, K, N, scales, biases, yb, N, overlap, none, scratch, st);
        if (!rc && bc > 16)
          rc = launch_wo_ring_inst<XT, 2, 4, 2, false, 2, GS, 16, 4, YF32>(xb + 16 * K, bc - 16, K, K, w, K, N, scales, biases, yrow(b0 + 16), N,
                                                                           true, none, scratch, st);
      }
    } else if (bc <= 8)  // two half-size CTAs per SM, passes of four tiles in 16-row boxes, four deep (measured: 19.7 us on
                         // [14336, 4096] at group size 64 against 22.5 us with passes of two tiles in 32-row boxes)
      rc = launch_wo_ring_inst<XT, 1, 4, 0, false, 1, GS, 8, 8, YF32>(xb, bc, K, K, w, K, N, scales, biases, yb, N, overlap, none, scratch, st);
    else if (bc <= 16)
      rc = few ? launch_wo_ring_inst<XT, 2, 2, 3, false, 1, GS, 16, 8, YF32>(xb, bc, K, K, w, K, N, scales, biases, yb, N, overlap, none, scratch, st)
               : launch_wo_ring_inst<XT, 2, 4, 2, false, 1, GS, 16, 8, YF32>(xb, bc, K, K, w, K, N, scales, biases, yb, N, overlap, none, scratch, st);
    else {  // two passes with at most 16 rows each, as for per-channel weights
      rc = launch_wo_ring_inst<XT, 2, 4, 2, false, 1, GS, 16, 8, YF32>(xb, 16, K, K, w, K, N, scales, biases, yb, N, overlap, none, scratch, st);
      if (!rc)
        rc = launch_wo_ring_inst<XT, 2, 4, 2, false, 1, GS, 16, 8, YF32>(xb + 16 * K, bc - 16, K, K, w, K, N, scales, biases, yrow(b0 + 16), N,
                                                                         true, none, scratch, st);
    }
    if (rc) return rc;
  }
  return LC_OK;
}

static int32_t check_group_args(int64_t N, int64_t K, int32_t gs, int32_t bits) {
  if (bits != 4 && bits != 8) return fail(LC_ERR_UNSUPPORTED, "group format: bits must be 4 or 8, got %d", bits);
  if (gs != 32 && gs != 64 && gs != 128)
    return fail(LC_ERR_UNSUPPORTED, "group format: group_size must be 32, 64 or 128, got %d", gs);
  if (N < 0 || K <= 0 || K % gs != 0)
    return fail(LC_ERR_INVALID_ARG, "group format: K=%lld must be a positive multiple of group_size=%d",
                (long long)K, gs);
  return LC_OK;
}

}  // namespace lc

using namespace lc;

extern "C" int32_t lc_wo_linear_s8(const void* x, int32_t x_dtype, int64_t batch, int64_t K,
                                   int64_t ldx, const int8_t* wq, int64_t ldw, int64_t N,
                                   const float* sw, const float* bias, void* y, int64_t ldy,
                                   int32_t flags, void* stream) {
  return lc_wo_linear_s8_ex(x, x_dtype, batch, K, ldx, wq, ldw, N, sw, bias, 0, nullptr, nullptr, 0, 0, y, ldy, flags,
                            nullptr, 0, stream);
}

extern "C" int64_t lc_wo_linear_workspace_bytes(int64_t N) {
  if (N < 0) return 0;
  return static_cast<int64_t>(sm_count()) * 2 * 2 * kRingSlotBytes + ((N + 15) / 16) * 4;  // two CTAs per SM at most
}

extern "C" int32_t lc_wo_linear_s8_ex(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                                      const int8_t* wq, int64_t ldw, int64_t N, const float* sw, const float* bias,
                                      int32_t relu, const float* out_scale, const float* out_zp, int32_t quant_min,
                                      int32_t quant_max, void* y, int64_t ldy, int32_t flags, void* workspace,
                                      int64_t workspace_bytes, void* stream) {
  const bool overlap = (flags & LC_WO_OVERLAP_PREVIOUS) != 0;
  if (batch < 0 || N < 0 || K <= 0 || ldx < K || ldw < K || ldy < N)
    return fail(LC_ERR_INVALID_ARG, "wo_linear_s8: bad shape");
  if ((out_scale == nullptr) != (out_zp == nullptr))
    return fail(LC_ERR_INVALID_ARG, "wo_linear_s8: out_scale and out_zp go together");
  if (batch == 0 || N == 0) return LC_OK;
  if (!x || !wq || !y) return fail(LC_ERR_INVALID_ARG, "wo_linear_s8: null pointer");
  cudaStream_t st = as_stream(stream);
  const WoEpilogue epi = {relu ? 1 : 0, out_scale, out_zp, static_cast<float>(quant_min),
                          static_cast<float>(quant_max)};
  const RingScratch scratch = {workspace, workspace ? workspace_bytes : 0};
  switch (x_dtype) {
    case LC_F32:
      return wo_linear_typed<float>(x, batch, K, ldx, wq, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st);
    case LC_BF16:
      return wo_linear_typed<__nv_bfloat16>(x, batch, K, ldx, wq, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st);
    case LC_F16:
      return wo_linear_typed<__half>(x, batch, K, ldx, wq, ldw, N, sw, bias, y, ldy, overlap, epi, scratch, st);
  }
  return fail(LC_ERR_UNSUPPORTED, "wo_linear_s8: x_dtype %d not supported", x_dtype);
}

extern "C" int32_t lc_wo_swiglu_s8(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                                   const int8_t* wq, int64_t ldw, int64_t N2, const float* sw,
                                   const float* bias, void* y, int64_t ldy, int32_t flags, void* stream) {
  return lc_wo_swiglu_s8_ex(x, x_dtype, batch, K, ldx, wq, ldw, N2, sw, bias, y, ldy, flags, nullptr, 0, stream);
}

extern "C" int32_t lc_wo_swiglu_s8_ex(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                                      const int8_t* wq, int64_t ldw, int64_t N2, const float* sw,
                                      const float* bias, void* y, int64_t ldy, int32_t flags, void* workspace,
                                      int64_t workspace_bytes, void* stream) {
  const bool overlap = (flags & LC_WO_OVERLAP_PREVIOUS) != 0;
  if (batch < 0 || N2 < 0 || K <= 0 || ldx < K || ldw < K || ldy < N2 / 2)
    return fail(LC_ERR_INVALID_ARG, "wo_swiglu_s8: bad shape");
  if (N2 % 16) return fail(LC_ERR_INVALID_ARG, "wo_swiglu_s8: the interleaved weight needs a multiple of 16 rows");
  if (batch == 0 || N2 == 0) return LC_OK;
  if (!x || !wq || !y) return fail(LC_ERR_INVALID_ARG, "wo_swiglu_s8: null pointer");
  if (batch > 32) return fail(LC_ERR_UNSUPPORTED, "wo_swiglu_s8: batch %lld > 32", (long long)batch);
  if (K % 16 || ldw % 16 || ldx % 8 || !aligned(wq, 16) || !aligned(x, 16))
    return fail(LC_ERR_UNSUPPORTED, "wo_swiglu_s8: K, ldw must be multiples of 16, ldx of 8, pointers 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  const WoEpilogue none = {0, nullptr, nullptr, 0.0f, 0.0f};
  const RingScratch scratch = {workspace, workspace ? workspace_bytes : 0};
  if (x_dtype == LC_BF16)
    return launch_wo_tma<__nv_bfloat16, true>(static_cast<const __nv_bfloat16*>(x), batch, K, ldx, wq, ldw, N2, sw,
                                              bias, static_cast<__nv_bfloat16*>(y), ldy, overlap, none, scratch, st);
  if (x_dtype == LC_F16)
    return launch_wo_tma<__half, true>(static_cast<const __half*>(x), batch, K, ldx, wq, ldw, N2, sw, bias,
                                       static_cast<__half*>(y), ldy, overlap, none, scratch, st);
  return fail(LC_ERR_UNSUPPORTED, "wo_swiglu_s8: activations must be bf16 or f16");
}

extern "C" int32_t lc_wo_linear_status(int32_t* host_code, int32_t clear) {
  if (!host_code) return fail(LC_ERR_INVALID_ARG, "wo_linear_status: null pointer");
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_wo_status, sizeof(int)) != cudaSuccess)
    return fail(LC_ERR_CUDA, "wo_linear_status: %s", cudaGetErrorString(cudaGetLastError()));
  *host_code = v;
  if (clear && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_wo_status, &zero, sizeof(int)) != cudaSuccess)
      return fail(LC_ERR_CUDA, "wo_linear_status: %s", cudaGetErrorString(cudaGetLastError()));
  }
  return LC_OK;
}

extern "C" int32_t lc_group_quantize_f32(const float* w, int64_t N, int64_t K, int32_t group_size,
                                         int32_t bits, int32_t* packed, float* scales,
                                         float* biases, void* stream) {
  if (int32_t rc = check_group_args(N, K, group_size, bits)) return rc;
  if (N == 0) return LC_OK;
  if (!w || !packed || !scales || !biases) return fail(LC_ERR_INVALID_ARG, "group_quantize: null pointer");
  const int per = 32 / bits;
  const int words_per_row = static_cast<int>(K / per);
  const int64_t total = N * words_per_row;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  uint32_t* pk = reinterpret_cast<uint32_t*>(packed);
  if (bits == 8)
    group_quantize_kernel<8><<<grid, 256, 0, as_stream(stream)>>>(w, total, words_per_row, K, group_size, pk, scales, biases);
  else
    group_quantize_kernel<4><<<grid, 256, 0, as_stream(stream)>>>(w, total, words_per_row, K, group_size, pk, scales, biases);
  return check_launch("group_quantize");
}

extern "C" int32_t lc_group_dequantize(const int32_t* packed, const float* scales,
                                       const float* biases, int64_t N, int64_t K,
                                       int32_t group_size, int32_t bits, float* out, void* stream) {
  if (int32_t rc = check_group_args(N, K, group_size, bits)) return rc;
  if (N == 0) return LC_OK;
  if (!packed || !scales || !biases || !out) return fail(LC_ERR_INVALID_ARG, "group_dequantize: null pointer");
  const int per = 32 / bits;
  const int words_per_row = static_cast<int>(K / per);
  const int64_t total = N * words_per_row;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  const uint32_t* pk = reinterpret_cast<const uint32_t*>(packed);
  if (bits == 8)
    group_dequantize_kernel<8><<<grid, 256, 0, as_stream(stream)>>>(pk, scales, biases, total, words_per_row, K, group_size, out);
  else
    group_dequantize_kernel<4><<<grid, 256, 0, as_stream(stream)>>>(pk, scales, biases, total, words_per_row, K, group_size, out);
  return check_launch("group_dequantize");
}

extern "C" int32_t lc_group_matmul(const void* x, int32_t x_dtype, int64_t batch, int64_t K,
                                   const int32_t* packed, const float* scales, const float* biases,
                                   int64_t N, int32_t group_size, int32_t bits, void* y,
                                   void* stream) {
  return lc_group_matmul_ex(x, x_dtype, batch, K, packed, scales, biases, N, group_size, bits, y, 0, nullptr, 0, stream);
}

extern "C" int32_t lc_group_matmul_ex(const void* x, int32_t x_dtype, int64_t batch, int64_t K,
                                      const int32_t* packed, const float* scales, const float* biases,
                                      int64_t N, int32_t group_size, int32_t bits, void* y, int32_t flags,
                                      void* workspace, int64_t workspace_bytes, void* stream) {
  if (int32_t rc = check_group_args(N, K, group_size, bits)) return rc;
  if (batch < 0) return fail(LC_ERR_INVALID_ARG, "group_matmul: bad batch");
  if (batch == 0 || N == 0) return LC_OK;
  if (!x || !packed || !scales || !biases || !y) return fail(LC_ERR_INVALID_ARG, "group_matmul: null pointer");
  // the kernels read 4 or 8 activations per load instruction: rows must start on 16-byte boundaries
  // (K is a multiple of the group size, so every row does once the first one does)
  if (!aligned(x, 16) || !aligned(packed, 4) || !aligned(scales, 4) || !aligned(biases, 4))
    return fail(LC_ERR_UNSUPPORTED, "group_matmul: x must be 16-byte aligned (packed, scales, biases 4-byte aligned)");
  cudaStream_t st = as_stream(stream);
  const uint32_t* pk = reinterpret_cast<const uint32_t*>(packed);
  // codes in groups of 64 / 128, 16-bit activations: the streaming kernel for packed weights of 4 MB and more,
  // and for smaller ones from five rows on, where the direct kernel's FP32 multiply-adds take over its time
  // (measured, N = K = 1024 / 2048, 4-bit codes: 8 rows 6.2 / 10.9 us direct against 4.3 / 5.4 us streamed, 32 rows
  // 12.6 / 32.8 against 8.8 / 11.9 us; one row 2.9 / 4.8 against 4.2 / 5.2 us)
  const bool stream_ok = (group_size == 64 || group_size == 128) &&
                         (x_dtype == LC_BF16 || x_dtype == LC_F16) && K % (4 * group_size) == 0 && K >= ring::KC &&
                         (N * K * bits >= (int64_t{32} << 20) || (batch >= 5 && N >= 1024 && K >= 1024)) &&
                         aligned(packed, 16) && aligned(x, 16) &&
                         aligned(scales, 16) && aligned(biases, 16);  // (rows of group parameters in 16-byte steps)
  const bool out_f32 = (flags & LC_GROUP_OUT_F32) != 0;
  if (out_f32 && !(stream_ok && x_dtype == LC_BF16))
    return fail(LC_ERR_UNSUPPORTED, "group_matmul: fp32 results of bf16 activations are written by the streaming kernel only "
                                    "(packed weights of 4 MB and more, groups of 64 / 128, K a multiple of four groups)");
  if (stream_ok) {
    const bool overlap = (flags & LC_WO_OVERLAP_PREVIOUS) != 0;
    const RingScratch scratch = {workspace, workspace ? workspace_bytes : 0};
    const uint8_t* codes = reinterpret_cast<const uint8_t*>(packed);
#define LC_GR(XT, GS, BITS) \
  launch_group_ring<XT, GS, BITS>(static_cast<const XT*>(x), batch, K, codes, scales, biases, N, static_cast<XT*>(y), overlap, scratch, st)
#define LC_GRF(GS, BITS) \
  launch_group_ring<__nv_bfloat16, GS, BITS, true>(static_cast<const __nv_bfloat16*>(x), batch, K, codes, scales, biases, N, \
                                                   static_cast<__nv_bfloat16*>(y), overlap, scratch, st)
    if (out_f32) {
      if (bits == 4) return group_size == 64 ? LC_GRF(64, 4) : LC_GRF(128, 4);
      return group_size == 64 ? LC_GRF(64, 8) : LC_GRF(128, 8);
    }
#undef LC_GRF
    if (bits == 4) {
      if (x_dtype == LC_BF16) return group_size == 64 ? LC_GR(__nv_bfloat16, 64, 4) : LC_GR(__nv_bfloat16, 128, 4);
      return group_size == 64 ? LC_GR(__half, 64, 4) : LC_GR(__half, 128, 4);
    }
    if (x_dtype == LC_BF16) return group_size == 64 ? LC_GR(__nv_bfloat16, 64, 8) : LC_GR(__nv_bfloat16, 128, 8);
    return group_size == 64 ? LC_GR(__half, 64, 8) : LC_GR(__half, 128, 8);
#undef LC_GR
  }
#define LC_GM(XT)                                                                                     \
  (bits == 8 ? launch_group_matmul<XT, 8>(static_cast<const XT*>(x), batch, K, pk, scales, biases, N, \
                                          group_size, static_cast<XT*>(y), st)                        \
             : launch_group_matmul<XT, 4>(static_cast<const XT*>(x), batch, K, pk, scales, biases, N, \
                                          group_size, static_cast<XT*>(y), st))
  switch (x_dtype) {
    case LC_F32:
      return LC_GM(float);
    case LC_BF16:
      return LC_GM(__nv_bfloat16);
    case LC_F16:
      return LC_GM(__half);
  }
#undef LC_GM
  return fail(LC_ERR_UNSUPPORTED, "group_matmul: x_dtype %d not supported", x_dtype);
}
