// int8 Linear for B200: tcgen05.mma kind::i8 (s8 x s8 or u8 x s8 -> s32 in TMEM),
// TMA-fed 128B-swizzled operand tiles, persistent warp-specialised CTAs and a
// fused dequantize(+zero-point)(+bias) epilogue.
//
//   acc[m,n] = sum_k a[m,k] * b[n,k]        both operands K-major, exactly the
//                                           reference's (out,in) weight layout
//   out      = f32(acc - zx*wsum[n]) * sx[m] * sw[n] + bias[n]
//
// CTA = 192 threads: warp 0 issues TMA loads, warp 1 owns TMEM and issues the
// MMAs, warps 2..5 drain the accumulator (one TMEM lane quadrant each).  The
// accumulator is double-buffered in TMEM (2 x 256 columns) so the epilogue of
// tile i overlaps the main loop of tile i+1.  No multicast is used anywhere.
//
// The same kernels run the weight-only Linear (float activations, int8 weight codes) for more
// rows than a GEMV handles, in two more instantiations:
//  * kModeDigits, for fp32 activations: every row of x is scaled by a power of two (exact) so that
//    its largest entry lies in [2^29, 2^30), rounded to an integer (every entry within 2^-6 of the
//    row maximum keeps all 24 bits; the absolute error of the rest is below 2^-30 of the row maximum)
//    and cut into four signed base-256 digits.  The digit planes of 32 rows form one 128-row tile of
//    A (lanes 32d .. 32d+31 of the accumulator hold digit d), the product runs on kind::i8 with exact
//    int32 accumulation, and the epilogue recombines ((a3*256 + a2)*256 + a1)*256 + a0 in 64-bit
//    integers: the whole dot product is exact and is rounded to fp32 once.
//  * kModeF16, for bf16 / f16 activations: tcgen05.mma kind::f16 with fp32 accumulation; the int8
//    codes are exact in either type.  (The kernel also accepts up to three bf16 addends of an fp32
//    activation side by side along K.  Every product is then exact, but the tensor core truncates
//    when it adds into the fp32 accumulator: measured 2.3e-6 of the output RMS at K = 512 and
//    3.5e-5 at K = 8192, against ~5e-7 of an IEEE fp32 GEMM -- which is why fp32 activations take
//    the digit form.)
// The epilogue of both applies the per-channel weight scale, an optional weight zero-point term,
// the bias, an optional ReLU and an optional requantization onto a calibrated per-tensor grid.
//
// Every wait on an mbarrier is bounded: when the bound is hit the waiting role
// records a code in the caller's status word, leaves its loop, the CTA waits
// (bounded) for its own TMA copies in flight, frees its TMEM and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace lc {
namespace gemm {

constexpr int BM = 128;          // rows of A per tile  (UMMA M)
constexpr int BN = 256;          // rows of B per tile  (UMMA N)
constexpr int BK = 128;          // bytes of K per stage = one 128B swizzle atom
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit operands
constexpr int STAGES = 3;
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;  // 512 = all of TMEM
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 320;          // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_THREADS = 256;          // two warps per TMEM lane quadrant, alternating 32-column chunks
constexpr int GROUP_M = 16;      // tile rasterisation: bands of 16 M-tiles share B in L2
constexpr int STG_PITCH = 36;                         // words per staged row: conflict-free 16-byte access
constexpr int STG_WARP_WORDS = 32 * STG_PITCH;
constexpr int STG_BYTES = (EPI_THREADS / 32) * STG_WARP_WORDS * 4;  // epilogue transpose buffers
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + STG_BYTES;

constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s at 2 GHz

// what the kernels are instantiated for
constexpr int kModeI8 = 0;      // int8 x int8 -> int32, dequantizing epilogue (dynamic Linear)
constexpr int kModeF16 = 1;     // 16-bit float operands, fp32 accumulation, weight-only epilogue
constexpr int kModeDigits = 2;  // int8 digit planes of fp32 activations x int8 codes, exact, weight-only epilogue

enum : int { ST_PRODUCER = 1, ST_MMA = 2, ST_EPILOGUE = 3 };

struct Params {
  int64_t M, N, K;
  const float* sx;      // 1 or M
  int sx_per_row;
  const float* zx;      // device scalar holding an integer value, or null
  const int32_t* wsum;  // [N] or null
  const float* sw;      // [N] or null
  const float* bias;    // [N] or null
  void* outs[8];        // destinations of the output tile (this GPU's buffer first; peers' after)
  int n_out;
  int out_dtype;
  int64_t ldo;
  int out_vec;          // rows of `out` allow 16-byte stores
  int fast_f32;         // 0, or 1 + (zero-point correction) + 2 * (bias): the compiled-in fp32 epilogue applies
  int32_t* status;
  int multicast;        // outs[0] is a multicast address: stores go out as multimem.st and the switch replicates them
  int wait_test;        // test hook: the producer role issues nothing and every wait gives up after a few thousand cycles
  // weight-only instantiations (kModeF16, kModeDigits) only
  int64_t rows_out;     // kModeDigits: rows of the output (M counts digit-plane rows, 4 per output row)
  int kb_wrap;          // K blocks of the weight; A holds n_terms times as many and B's K coordinate wraps
  const float* rowsum;  // [M] sum_k x[m,k] or null   } weight zero-point term rowsum[m] * colcorr[n]
  const float* colcorr; // [N] -zw[n]*sw[n] or null   }
  int relu;
  const float* fq_scale;  // device scalars of the output grid, or null: no requantization
  const float* fq_zp;
  float fq_min, fq_max;
};

// ---- PTX wrappers ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait: false when the bound was hit
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, long long budget = kWaitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > budget) return false;
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// barrier over the 128 epilogue threads that also ANDs a predicate, so that all
// four warps take the same decision after a bounded wait
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred pin, pout;\n\t"
      "setp.ne.u32 pin, %1, 0;\n\t"
      "bar.red.and.pred pout, 1, %2, pin;\n\t"
      "selp.u32 %0, 1, 0, pout;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(ok)), "n"(EPI_THREADS)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as 128-byte rows with
// the 128B swizzle (what a SWIZZLE_128B TMA box of 128 bytes x rows produces):
// start address >> 4 in bits [0,14), leading byte offset (unused by swizzled
// K-major layouts, canonical value 1) in [16,30), stride byte offset = 1024 B
// between 8-row groups in [32,46), descriptor version 1 in [46,48), layout
// type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::i8: D format s32 (2) in bits [4,6), A format
// in [7,10) and B format in [10,13) (0 = u8, 1 = s8), both operands K-major
// (bits 15, 16 = 0), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc(bool a_unsigned, int n = BN) {
  return (2u << 4) | ((a_unsigned ? 0u : 1u) << 7) | (1u << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

// The single-CTA kernel comes in tile widths BNT = 256, 64 and 32 columns: one row tile of A
// (M <= 128, the single quantized Linear of a small batch) gives only N / 256 CTAs at the full
// width, each pulling its slice of the weight through one TMA queue; narrower tiles spread the
// same weight over up to 148 SMs.  Stage and TMEM budgets follow the width.
template <int BNT>
struct NarrowCfg {
  static constexpr int kStages = BNT == 256 ? 3 : 6;
  static constexpr int kStageBytes = A_BYTES + BNT * BK;
  static constexpr int kTmemCols = ACC_STAGES * BNT;  // 512, 128 or 64: powers of two >= 32
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + STG_BYTES;
};

__device__ __forceinline__ void tile_coords(int64_t t, int64_t tiles_m, int64_t tiles_n, int64_t& tm,
                                            int64_t& tn) {
  const int64_t group = static_cast<int64_t>(GROUP_M) * tiles_n;
  const int64_t g = t / group;
  const int64_t first_m = g * GROUP_M;
  const int64_t gm = (tiles_m - first_m < GROUP_M) ? (tiles_m - first_m) : GROUP_M;
  const int64_t r = t % group;
  tm = first_m + r % gm;
  tn = r / gm;
}

__device__ __forceinline__ void report(int32_t* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// Second half of every epilogue chunk: the warp's 32 x 32 staged values (row-major, STG_PITCH
// words per row; floats unless the output is int32) go out as whole 64- or 128-byte row
// segments (4 or 8 rows per instruction) to every destination buffer.  Writing whole segments
// matters most when a destination is another GPU's memory.
__device__ __forceinline__ void store_staged(const Params& p, const uint32_t* stg, int c, int64_t row_base,
                                             int64_t n0, int lane) {
  const int64_t col0 = n0 + c * 32;
  if (p.out_dtype == LC_BF16 || p.out_dtype == LC_F16) {
    const int sub = lane & 3, rr = lane >> 2;  // 4 lanes x 16 bytes per row, 8 rows per pass
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rloc = i * 8 + rr;
      const int64_t row = row_base + rloc, col = col0 + sub * 8;
      const float4 lo = *reinterpret_cast<const float4*>(stg + rloc * STG_PITCH + sub * 8);
      const float4 hi = *reinterpret_cast<const float4*>(stg + rloc * STG_PITCH + sub * 8 + 4);
      if (row < p.M && col < p.N) {
        uint4 w;
        if (p.out_dtype == LC_BF16) {
          __nv_bfloat162 h0 = __floats2bfloat162_rn(lo.x, lo.y), h1 = __floats2bfloat162_rn(lo.z, lo.w);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(hi.x, hi.y), h3 = __floats2bfloat162_rn(hi.z, hi.w);
          w.x = *reinterpret_cast<uint32_t*>(&h0);
          w.y = *reinterpret_cast<uint32_t*>(&h1);
          w.z = *reinterpret_cast<uint32_t*>(&h2);
          w.w = *reinterpret_cast<uint32_t*>(&h3);
        } else {
          __half2 h0 = __floats2half2_rn(lo.x, lo.y), h1 = __floats2half2_rn(lo.z, lo.w);
          __half2 h2 = __floats2half2_rn(hi.x, hi.y), h3 = __floats2half2_rn(hi.z, hi.w);
          w.x = *reinterpret_cast<uint32_t*>(&h0);
          w.y = *reinterpret_cast<uint32_t*>(&h1);
          w.z = *reinterpret_cast<uint32_t*>(&h2);
          w.w = *reinterpret_cast<uint32_t*>(&h3);
        }
        for (int d = 0; d < p.n_out; ++d) {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.outs[d]) + row * p.ldo + col;
          if (p.out_vec && col + 8 <= p.N) {
            *reinterpret_cast<uint4*>(o) = w;
          } else {
            const __nv_bfloat16* hv = reinterpret_cast<const __nv_bfloat16*>(&w);
            for (int e = 0; e < 8; ++e)
              if (col + e < p.N) o[e] = hv[e];
          }
        }
      }
    }
  } else {
    const int sub = lane & 7, rr = lane >> 3;  // 8 lanes x 16 bytes per row, 4 rows per pass
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rloc = i * 4 + rr;
      const int64_t row = row_base + rloc, col = col0 + sub * 4;
      const uint4 w = *reinterpret_cast<const uint4*>(stg + rloc * STG_PITCH + sub * 4);
      if (row < p.M && col < p.N) {
        if (p.n_out == 1 && p.out_vec && col + 4 <= p.N) {
          uint32_t* o = static_cast<uint32_t*>(p.outs[0]) + row * p.ldo + col;
          if (p.multicast)  // one store; NVSwitch writes it into every GPU's copy of the buffer
            asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(__uint_as_float(w.x)),
                         "f"(__uint_as_float(w.y)), "f"(__uint_as_float(w.z)), "f"(__uint_as_float(w.w))
                         : "memory");
          else
            *reinterpret_cast<uint4*>(o) = w;
          continue;
        }
        for (int d = 0; d < p.n_out; ++d) {
          uint32_t* o = static_cast<uint32_t*>(p.outs[d]) + row * p.ldo + col;
          if (p.out_vec && col + 4 <= p.N) {
            *reinterpret_cast<uint4*>(o) = w;
          } else {
            const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
            for (int e = 0; e < 4; ++e)
              if (col + e < p.N) o[e] = wv[e];
          }
        }
      }
    }
  }
  __syncwarp();
}

// Epilogue chunk of the weight-only instantiation: the accumulator holds fp32 sums of
// x[m,k] * code[n,k]; out = requant(relu(acc * sw[n] + rowsum[m] * colcorr[n] + bias[n])), every
// step one IEEE fp32 operation as in the reference's eager epilogue
// (lucid/nn/quantized/linear.py:206-214: linear, activation, fake_quantize).
__device__ __forceinline__ void drain_chunk_wo(const Params& p, const uint32_t (&r)[32], int c, int64_t row_base,
                                               int64_t n0, int lane, float rs, const float* s_sw,
                                               const float* s_bias, const float* s_cc, float fq_s, float fq_inv,
                                               float fq_z, uint32_t* stg) {
  uint32_t* mine = stg + lane * STG_PITCH;
  const bool has_cc = p.colcorr != nullptr, has_bias = p.bias != nullptr, relu = p.relu != 0,
             fq = p.fq_scale != nullptr;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 sv = *reinterpret_cast<const float4*>(s_sw + c * 32 + j);
    float f[4] = {__fmul_rn(__uint_as_float(r[j]), sv.x), __fmul_rn(__uint_as_float(r[j + 1]), sv.y),
                  __fmul_rn(__uint_as_float(r[j + 2]), sv.z), __fmul_rn(__uint_as_float(r[j + 3]), sv.w)};
    if (has_cc) {
      const float4 cv = *reinterpret_cast<const float4*>(s_cc + c * 32 + j);
      f[0] = __fadd_rn(f[0], __fmul_rn(rs, cv.x));
      f[1] = __fadd_rn(f[1], __fmul_rn(rs, cv.y));
      f[2] = __fadd_rn(f[2], __fmul_rn(rs, cv.z));
      f[3] = __fadd_rn(f[3], __fmul_rn(rs, cv.w));
    }
    if (has_bias) {
      const float4 bv = *reinterpret_cast<const float4*>(s_bias + c * 32 + j);
      f[0] = __fadd_rn(f[0], bv.x);
      f[1] = __fadd_rn(f[1], bv.y);
      f[2] = __fadd_rn(f[2], bv.z);
      f[3] = __fadd_rn(f[3], bv.w);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (relu) f[e] = f[e] < 0.0f ? 0.0f : f[e];  // NaN compares false and stays
      if (fq) f[e] = fake_quant_value(f[e], fq_s, fq_inv, fq_z, p.fq_min, p.fq_max);
    }
    *reinterpret_cast<float4*>(mine + j) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __syncwarp();
  store_staged(p, stg, c, row_base, n0, lane);
}

// Epilogue chunk of the digit instantiation.  The four epilogue warps that share a column chunk
// hold the four digit planes of the same 32 output rows (warp q: lanes 32q .. 32q+31 = digit q).
// Each parks its raw int32 sums in its staging buffer; after a barrier over the four warps, warp q
// recombines output rows 8q .. 8q+7 (lane = column), applies the epilogue and stores 128-byte row
// segments.  `group_stg` is the first of the group's four staging buffers, `bar` its barrier id.
__device__ __forceinline__ void drain_chunk_digits(const Params& p, const uint32_t (&r)[32], int c, int64_t row_base,
                                                   int64_t n0, int q, int lane, const float* s_sw,
                                                   const float* s_bias, const float* s_cc, float fq_s, float fq_inv,
                                                   float fq_z, uint32_t* group_stg, int bar) {
  uint32_t* mine = group_stg + q * STG_WARP_WORDS + lane * STG_PITCH;
#pragma unroll
  for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(mine + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
  asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
  const int64_t col = n0 + c * 32 + lane;
  const bool col_ok = col < p.N;
  const float swv = s_sw[c * 32 + lane], bv = s_bias[c * 32 + lane], cv = s_cc[c * 32 + lane];
  const bool has_cc = p.colcorr != nullptr, has_bias = p.bias != nullptr, relu = p.relu != 0,
             fq = p.fq_scale != nullptr;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = q * 8 + i;
    const int64_t row = row_base + rr;
    const int* src = reinterpret_cast<const int*>(group_stg) + rr * STG_PITCH + lane;
    const long long v = ((static_cast<long long>(src[3 * STG_WARP_WORDS]) * 256 + src[2 * STG_WARP_WORDS]) * 256 +
                         src[STG_WARP_WORDS]) * 256 + src[0];
    if (row < p.rows_out && col_ok) {
      // one rounding of the exact integer sum; the row scale is a power of two
      float f = __fmul_rn(__fmul_rn(__ll2float_rn(v), __ldg(p.sx + row)), swv);
      if (has_cc) f = __fadd_rn(f, __fmul_rn(__ldg(p.rowsum + row), cv));
      if (has_bias) f = __fadd_rn(f, bv);
      if (relu) f = f < 0.0f ? 0.0f : f;  // NaN compares false and stays
      if (fq) f = fake_quant_value(f, fq_s, fq_inv, fq_z, p.fq_min, p.fq_max);
      static_cast<float*>(p.outs[0])[row * p.ldo + col] = f;
    }
  }
  asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");  // the buffers are free for the next chunk
}

// One 32-row x 32-column chunk of the accumulator: lane = row computes the 32 outputs,
// the warp transposes them through shared memory, then stores rows as whole 64/128-byte
// segments (4 or 8 rows per instruction) to every destination buffer.  Writing whole
// segments matters most when a destination is another GPU's memory.
__device__ __forceinline__ void drain_chunk(const Params& p, const uint32_t (&r)[32], int c,
                                            int64_t row_base, int64_t n0, int lane, float sxr,
                                            const float* s_sw, const float* s_bias, const int* s_corr,
                                            uint32_t* stg) {
  uint32_t* mine = stg + lane * STG_PITCH;
  const bool has_corr = p.zx != nullptr, has_bias = p.bias != nullptr, has_sw = p.sw != nullptr;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    int a[4] = {static_cast<int>(r[j]), static_cast<int>(r[j + 1]), static_cast<int>(r[j + 2]),
                static_cast<int>(r[j + 3])};
    if (has_corr) {
      const int4 cr = *reinterpret_cast<const int4*>(s_corr + c * 32 + j);
      a[0] -= cr.x;
      a[1] -= cr.y;
      a[2] -= cr.z;
      a[3] -= cr.w;
    }
    uint32_t w[4];
    if (p.out_dtype == LC_S32) {
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = static_cast<uint32_t>(a[e]);
    } else {
      float f[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = __fmul_rn(static_cast<float>(a[e]), sxr);
      if (has_sw) {
        const float4 sv = *reinterpret_cast<const float4*>(s_sw + c * 32 + j);
        f[0] = __fmul_rn(f[0], sv.x);
        f[1] = __fmul_rn(f[1], sv.y);
        f[2] = __fmul_rn(f[2], sv.z);
        f[3] = __fmul_rn(f[3], sv.w);
      }
      if (has_bias) {
        const float4 bv = *reinterpret_cast<const float4*>(s_bias + c * 32 + j);
        f[0] = __fadd_rn(f[0], bv.x);
        f[1] = __fadd_rn(f[1], bv.y);
        f[2] = __fadd_rn(f[2], bv.z);
        f[3] = __fadd_rn(f[3], bv.w);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = __float_as_uint(f[e]);
    }
    *reinterpret_cast<uint4*>(mine + j) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __syncwarp();
  store_staged(p, stg, c, row_base, n0, lane);
}

// The common case of drain_chunk with everything that can be decided per launch compiled in:
// fp32 output to one buffer with 16-byte aligned rows, per-column weight scales, chunk fully
// inside N.  Short-K products (an encoder's projections) are bound by this epilogue, and the
// general form spends about half of its instructions on launch-invariant branches and 64-bit
// index arithmetic.
template <bool CORR, bool BIAS>
__device__ __forceinline__ void drain_chunk_f32(const Params& p, const uint32_t (&r)[32], int c,
                                                int64_t row_base, int64_t n0, int lane, float sxr,
                                                const float* s_sw, const float* s_bias, const int* s_corr,
                                                uint32_t* stg) {
  uint32_t* mine = stg + lane * STG_PITCH;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    int a[4] = {static_cast<int>(r[j]), static_cast<int>(r[j + 1]), static_cast<int>(r[j + 2]),
                static_cast<int>(r[j + 3])};
    if (CORR) {
      const int4 cr = *reinterpret_cast<const int4*>(s_corr + c * 32 + j);
      a[0] -= cr.x;
      a[1] -= cr.y;
      a[2] -= cr.z;
      a[3] -= cr.w;
    }
    const float4 sv = *reinterpret_cast<const float4*>(s_sw + c * 32 + j);
    float f[4] = {__fmul_rn(__fmul_rn(static_cast<float>(a[0]), sxr), sv.x),
                  __fmul_rn(__fmul_rn(static_cast<float>(a[1]), sxr), sv.y),
                  __fmul_rn(__fmul_rn(static_cast<float>(a[2]), sxr), sv.z),
                  __fmul_rn(__fmul_rn(static_cast<float>(a[3]), sxr), sv.w)};
    if (BIAS) {
      const float4 bv = *reinterpret_cast<const float4*>(s_bias + c * 32 + j);
      f[0] = __fadd_rn(f[0], bv.x);
      f[1] = __fadd_rn(f[1], bv.y);
      f[2] = __fadd_rn(f[2], bv.z);
      f[3] = __fadd_rn(f[3], bv.w);
    }
    *reinterpret_cast<float4*>(mine + j) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __syncwarp();
  const int sub = lane & 7, rr = lane >> 3;  // 8 lanes x 16 bytes per row, 4 rows per pass
  float* o = static_cast<float*>(p.outs[0]) + (row_base + rr) * p.ldo + (n0 + c * 32 + sub * 4);
  const int64_t step = 4 * p.ldo;
  const int64_t rows_left = p.M - row_base - rr;  // row i*4 + rr exists while i*4 < rows_left
  const uint32_t* src = stg + rr * STG_PITCH + sub * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 w = *reinterpret_cast<const uint4*>(src + i * 4 * STG_PITCH);
    if (i * 4 < rows_left) *reinterpret_cast<uint4*>(o) = w;
    o += step;
  }
  __syncwarp();
}

// picks the compiled-in form when the launch and the chunk allow it
__device__ __forceinline__ void drain(const Params& p, const uint32_t (&r)[32], int c, int64_t row_base,
                                      int64_t n0, int lane, float sxr, const float* s_sw, const float* s_bias,
                                      const int* s_corr, uint32_t* stg) {
  if (p.fast_f32 && n0 + c * 32 + 32 <= p.N) {
    switch (p.fast_f32) {
      case 1: drain_chunk_f32<false, false>(p, r, c, row_base, n0, lane, sxr, s_sw, s_bias, s_corr, stg); return;
      case 2: drain_chunk_f32<true, false>(p, r, c, row_base, n0, lane, sxr, s_sw, s_bias, s_corr, stg); return;
      case 3: drain_chunk_f32<false, true>(p, r, c, row_base, n0, lane, sxr, s_sw, s_bias, s_corr, stg); return;
      default: drain_chunk_f32<true, true>(p, r, c, row_base, n0, lane, sxr, s_sw, s_bias, s_corr, stg); return;
    }
  }
  drain_chunk(p, r, c, row_base, n0, lane, sxr, s_sw, s_bias, s_corr, stg);
}

template <int BNT, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
qlinear_i8_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const Params p, const uint32_t idesc) {
  // tile width and what follows from it (these shadow the full-width constants of the namespace)
  constexpr int BN = BNT, STAGES = NarrowCfg<BNT>::kStages, STAGE_BYTES = NarrowCfg<BNT>::kStageBytes,
                TMEM_COLS = NarrowCfg<BNT>::kTmemCols;
  static_assert(2 * STAGES * 8 + 4 * ACC_STAGES * 8 <= 256, "barrier area");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(16) float s_sw[BN];
  __shared__ __align__(16) float s_bias[BN];
  __shared__ __align__(16) int s_corr[BN];
  __shared__ uint32_t s_tmem_base;

  pdl_launch_dependents();
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = tiles_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + ACC_STAGES + s); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long budget = p.wait_test ? 20000LL : kWaitCycles;

  const int64_t tiles_m = (p.M + BM - 1) / BM;
  const int64_t tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int num_kb = static_cast<int>((p.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), EPI_THREADS / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"(static_cast<uint32_t>(TMEM_COLS))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  // barriers, TMEM and descriptors are set up: everything from here on reads what the kernel
  // before this one produced (the quantized activations, their scales) or writes the output
  pdl_wait();

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t armed_parity[STAGES];
      bool armed[STAGES];
      for (int s = 0; s < STAGES; ++s) armed[s] = false;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // under the wait test the producer issues nothing, so every consumer wait runs out
      for (int64_t t = blockIdx.x; t < num_tiles && ok && !p.wait_test; t += gridDim.x) {
        int64_t tm, tn;
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        const int m0 = static_cast<int>(tm * BM), n0 = static_cast<int>(tn * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, budget)) {
            report(p.status, ST_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t a_dst = tiles_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, kb * BK, m0, full_bar(stage));
          tma_load_2d(a_dst + A_BYTES, &tmap_b, (MODE == kModeF16 ? kb % p.kb_wrap : kb) * BK, n0, full_bar(stage));
          armed[stage] = true;
          armed_parity[stage] = phase;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // do not leave while one of this CTA's bulk copies may still be landing
      for (int s = 0; s < STAGES; ++s)
        if (armed[s]) mbar_wait(full_bar(s), armed_parity[s]);
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int64_t it = 0;
      bool ok = true;
      for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int as = static_cast<int>(it & 1);
        const uint32_t aphase = static_cast<uint32_t>((it >> 1) & 1);
        if (!mbar_wait(acc_empty_bar(as), aphase ^ 1u, budget)) {
          report(p.status, ST_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(as * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, budget)) {
            report(p.status, ST_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = tiles_base + stage * STAGE_BYTES;
          const uint64_t a_desc = make_smem_desc(a_src);
          const uint64_t b_desc = make_smem_desc(a_src + A_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            // advancing K inside the swizzle atom = advancing the start address
            const uint64_t koff = static_cast<uint64_t>((j * UMMA_K) >> 4);
            if constexpr (MODE == kModeF16)
              tc_mma_f16(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | j) != 0 ? 1u : 0u);
            else
              tc_mma_i8(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));  // frees the smem slot once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(acc_full_bar(as));
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int et = threadIdx.x - 64;        // 0..255
    uint32_t* stg = reinterpret_cast<uint32_t*>(smem_raw + (bar_base + 256u - smem_u32(smem_raw))) +
                    (warp - 2) * STG_WARP_WORDS;
    const float sx_scalar = (p.sx && !p.sx_per_row) ? __ldg(p.sx) : 1.0f;
    const int zx_i = p.zx ? __float2int_rn(__ldg(p.zx)) : 0;
    // output grid of the weight-only epilogue (device scalars; 1 / s by IEEE division as the
    // reference's fake_quantize computes it for a tensor scale)
    const float fq_s = (MODE != kModeI8 && p.fq_scale) ? __ldg(p.fq_scale) : 1.0f;
    const float fq_inv = __fdiv_rn(1.0f, fq_s);
    const float fq_z = (MODE != kModeI8 && p.fq_zp) ? __ldg(p.fq_zp) : 0.0f;
    int64_t it = 0;
    for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      int64_t tm, tn;
      tile_coords(t, tiles_m, tiles_n, tm, tn);
      const int64_t m0 = tm * BM, n0 = tn * BN;
      // per-column epilogue constants of this tile, staged once for all rows
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      for (int j = et; j < BN; j += EPI_THREADS) {
        const int64_t n = n0 + j;
        const bool in = n < p.N;
        s_sw[j] = (in && p.sw) ? __ldg(p.sw + n) : 1.0f;
        s_bias[j] = (in && p.bias) ? __ldg(p.bias + n) : 0.0f;
        if constexpr (MODE != kModeI8)
          reinterpret_cast<float*>(s_corr)[j] = (in && p.colcorr) ? __ldg(p.colcorr + n) : 0.0f;
        else
          s_corr[j] = (in && p.wsum) ? zx_i * __ldg(p.wsum + n) : 0;
      }
      const int as = static_cast<int>(it & 1);
      const uint32_t aphase = static_cast<uint32_t>((it >> 1) & 1);
      // also publishes the staged constants to the other epilogue warps
      if (!epilogue_all(mbar_wait(acc_full_bar(as), aphase, budget))) {
        report(p.status, ST_EPILOGUE);
        break;
      }
      tc_fence_after();
      const int64_t row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const float sxr = MODE == kModeDigits ? 0.0f  // per-row values are read where the digits are combined
                        : MODE == kModeF16 ? ((p.rowsum && row_ok) ? __ldg(p.rowsum + row) : 0.0f)
                                           : (p.sx_per_row ? (row_ok ? __ldg(p.sx + row) : 0.0f) : sx_scalar);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(as * BN);
#pragma unroll 1
      for (int c = (warp - 2) >> 2; c < BN / 32; c += 2) {
        uint32_t r[32];
        tc_ld_32x32(t_row + static_cast<uint32_t>(c * 32), r);
        tc_wait_ld();
        if (n0 + c * 32 < p.N) {
          if constexpr (MODE == kModeF16)
            drain_chunk_wo(p, r, c, m0 + q * 32, n0, lane, sxr, s_sw, s_bias, reinterpret_cast<const float*>(s_corr),
                           fq_s, fq_inv, fq_z, stg);
          else if constexpr (MODE == kModeDigits)
            drain_chunk_digits(p, r, c, m0 >> 2, n0, q, lane, s_sw, s_bias, reinterpret_cast<const float*>(s_corr), fq_s,
                               fq_inv, fq_z, stg - (warp - 2) * STG_WARP_WORDS + ((warp - 2) >> 2) * 4 * STG_WARP_WORDS,
                               2 + ((warp - 2) >> 2));
          else
            drain(p, r, c, m0 + q * 32, n0, lane, sxr, s_sw, s_bias, s_corr, stg);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(as));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(TMEM_COLS))
                 : "memory");
  }
}

// =============================================================================================
// CTA-pair variant: tcgen05.mma.cta_group::2, one 256 x 256 output tile per 2-CTA cluster.
// CTA r of the pair owns rows [128r, 128r+128) of the tile (its TMEM holds that half of the
// accumulator) and loads its own A rows plus HALF of B (rows [128r, 128r+128) of the N tile);
// the pair's tensor cores read both halves of B.  Compared with the single-CTA kernel each
// CTA moves 32 KB instead of 48 KB through L2 and shared memory per 128 bytes of K, which is
// what that kernel is bound by.  No multicast loads: every TMA load is a plain per-CTA load
// whose completion is signalled on the leader CTA's mbarrier.
//   leader (rank 0): arms full[stage] with the bytes of both CTAs, issues the MMAs, and
//   commits with a 2-CTA multicast arrive so both CTAs' empty[stage] / acc_full[] flip;
//   both CTAs' epilogue warps release the accumulator on the leader's acc_empty[].
// =============================================================================================
namespace pair {
constexpr int BNH = BN / 2;                 // rows of B each CTA loads
constexpr int STAGES2 = 5;
constexpr int A_BYTES2 = BM * BK;           // 16 KB
constexpr int B_BYTES2 = BNH * BK;          // 16 KB
constexpr int STAGE_BYTES2 = A_BYTES2 + B_BYTES2;
constexpr int SMEM_BYTES2 = STAGES2 * STAGE_BYTES2 + 1024 + 256 + STG_BYTES;
}  // namespace pair

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// plain (non-multicast) TMA load whose completion is signalled on a barrier that may live in
// the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far retire
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}" ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_pair(bool a_unsigned) {
  return (2u << 4) | ((a_unsigned ? 0u : 1u) << 7) | (1u << 10) |
         (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>((2 * BM) >> 4) << 24);
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
qlinear_i8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b, const Params p, const uint32_t idesc) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(16) float s_sw[BN];
  __shared__ __align__(16) float s_bias[BN];
  __shared__ __align__(16) int s_corr[BN];
  __shared__ uint32_t s_tmem_base;

  pdl_launch_dependents();
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = tiles_base + STAGES2 * STAGE_BYTES2;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES2 + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES2 + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES2 + ACC_STAGES + s); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long budget = p.wait_test ? 20000LL : kWaitCycles;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int64_t pair_id = blockIdx.x >> 1;
  const int64_t num_pairs = gridDim.x >> 1;

  const int64_t tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int64_t tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int num_kb = static_cast<int>((p.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(acc_full_bar(s), 1);
      mbar_init(acc_empty_bar(s), 2 * (EPI_THREADS / 32));  // epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"(static_cast<uint32_t>(TMEM_COLS))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  // barriers, TMEM and descriptors are set up: everything from here on reads what the kernel
  // before this one produced (the quantized activations, their scales) or writes the output
  pdl_wait();

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      uint32_t armed_parity[STAGES2];
      bool armed[STAGES2];
      for (int s = 0; s < STAGES2; ++s) armed[s] = false;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // under the wait test the producers issue nothing, so every consumer wait runs out
      for (int64_t t = pair_id; t < num_tiles && ok && !p.wait_test; t += num_pairs) {
        int64_t tm, tn;
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        const int m0 = static_cast<int>(tm * 2 * BM + rank * BM);
        const int n0 = static_cast<int>(tn * BN + rank * BNH);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, budget)) {
            report(p.status, ST_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t a_dst = tiles_base + stage * STAGE_BYTES2;
          const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
          if (leader) {
            mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES2);
            armed[stage] = true;
            armed_parity[stage] = phase;
          }
          tma_load_2d_pair(a_dst, &tmap_a, kb * BK, m0, lead_full);
          tma_load_2d_pair(a_dst + A_BYTES2, &tmap_b, (MODE == kModeF16 ? kb % p.kb_wrap : kb) * BK, n0, lead_full);
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // the leader's full barriers count the bytes of both CTAs: once they have completed no
      // bulk copy of the pair is still landing (the peer stays until the final cluster barrier)
      for (int s = 0; s < STAGES2; ++s)
        if (armed[s]) mbar_wait(full_bar(s), armed_parity[s]);
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA only) =====================
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int64_t it = 0;
      bool ok = true;
      for (int64_t t = pair_id; t < num_tiles && ok; t += num_pairs, ++it) {
        const int as = static_cast<int>(it & 1);
        const uint32_t aphase = static_cast<uint32_t>((it >> 1) & 1);
        if (!mbar_wait(acc_empty_bar(as), aphase ^ 1u, budget)) {
          report(p.status, ST_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(as * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, budget)) {
            report(p.status, ST_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = tiles_base + stage * STAGE_BYTES2;
          const uint64_t a_desc = make_smem_desc(a_src);
          const uint64_t b_desc = make_smem_desc(a_src + A_BYTES2);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t koff = static_cast<uint64_t>((j * UMMA_K) >> 4);
            if constexpr (MODE == kModeF16)
              tc_mma_f16_pair(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | j) != 0 ? 1u : 0u);
            else
              tc_mma_i8_pair(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(stage));
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit_pair(acc_full_bar(as));
      }
    }
  } else {
    // ===================== epilogue (warps 2..5, both CTAs) =====================
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    uint32_t* stg = reinterpret_cast<uint32_t*>(smem_raw + (bar_base + 256u - smem_u32(smem_raw))) +
                    (warp - 2) * STG_WARP_WORDS;
    const float sx_scalar = (p.sx && !p.sx_per_row) ? __ldg(p.sx) : 1.0f;
    const int zx_i = p.zx ? __float2int_rn(__ldg(p.zx)) : 0;
    // output grid of the weight-only epilogue (device scalars; 1 / s by IEEE division as the
    // reference's fake_quantize computes it for a tensor scale)
    const float fq_s = (MODE != kModeI8 && p.fq_scale) ? __ldg(p.fq_scale) : 1.0f;
    const float fq_inv = __fdiv_rn(1.0f, fq_s);
    const float fq_z = (MODE != kModeI8 && p.fq_zp) ? __ldg(p.fq_zp) : 0.0f;
    int64_t it = 0;
    for (int64_t t = pair_id; t < num_tiles; t += num_pairs, ++it) {
      int64_t tm, tn;
      tile_coords(t, tiles_m, tiles_n, tm, tn);
      const int64_t m0 = tm * 2 * BM + rank * BM, n0 = tn * BN;
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      for (int j = et; j < BN; j += EPI_THREADS) {
        const int64_t n = n0 + j;
        const bool in = n < p.N;
        s_sw[j] = (in && p.sw) ? __ldg(p.sw + n) : 1.0f;
        s_bias[j] = (in && p.bias) ? __ldg(p.bias + n) : 0.0f;
        if constexpr (MODE != kModeI8)
          reinterpret_cast<float*>(s_corr)[j] = (in && p.colcorr) ? __ldg(p.colcorr + n) : 0.0f;
        else
          s_corr[j] = (in && p.wsum) ? zx_i * __ldg(p.wsum + n) : 0;
      }
      const int as = static_cast<int>(it & 1);
      const uint32_t aphase = static_cast<uint32_t>((it >> 1) & 1);
      if (!epilogue_all(mbar_wait(acc_full_bar(as), aphase, budget))) {
        report(p.status, ST_EPILOGUE);
        break;
      }
      tc_fence_after();
      const int64_t row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const float sxr = MODE == kModeDigits ? 0.0f  // per-row values are read where the digits are combined
                        : MODE == kModeF16 ? ((p.rowsum && row_ok) ? __ldg(p.rowsum + row) : 0.0f)
                                           : (p.sx_per_row ? (row_ok ? __ldg(p.sx + row) : 0.0f) : sx_scalar);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(as * BN);
#pragma unroll 1
      for (int c = (warp - 2) >> 2; c < BN / 32; c += 2) {
        uint32_t r[32];
        tc_ld_32x32(t_row + static_cast<uint32_t>(c * 32), r);
        tc_wait_ld();
        if (n0 + c * 32 < p.N) {
          if constexpr (MODE == kModeF16)
            drain_chunk_wo(p, r, c, m0 + q * 32, n0, lane, sxr, s_sw, s_bias, reinterpret_cast<const float*>(s_corr),
                           fq_s, fq_inv, fq_z, stg);
          else if constexpr (MODE == kModeDigits)
            drain_chunk_digits(p, r, c, m0 >> 2, n0, q, lane, s_sw, s_bias, reinterpret_cast<const float*>(s_corr), fq_s,
                               fq_inv, fq_z, stg - (warp - 2) * STG_WARP_WORDS + ((warp - 2) >> 2) * 4 * STG_WARP_WORDS,
                               2 + ((warp - 2) >> 2));
          else
            drain(p, r, c, m0 + q * 32, n0, lane, sxr, s_sw, s_bias, s_corr, stg);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar(as), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or leaves while the other may still use the pair
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(TMEM_COLS))
                 : "memory");
  }
}

// ---- host side ---------------------------------------------------------------
// 2-D uint8 tensor [rows, K] with row stride ld, box = 128 bytes x box_rows, 128B swizzle,
// out-of-bounds elements read as zero (so M, N and K tails need no special code).
static int32_t make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld,
                        int box_rows) {
  return encode_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, base, static_cast<uint64_t>(K),
                              static_cast<uint64_t>(rows), static_cast<uint64_t>(ld), BK,
                              static_cast<uint32_t>(box_rows), CU_TENSOR_MAP_SWIZZLE_128B);
}

template <typename Kernel>
static cudaError_t reserve_smem(Kernel kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

static int32_t ensure_smem_attr() {
  constexpr int kMaxDevices = 64;
  static std::once_flag flags[kMaxDevices];
  static cudaError_t results[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(LC_ERR_CUDA, "no current CUDA device");
  std::call_once(flags[dev], [dev]() {
    cudaError_t e = reserve_smem(qlinear_i8_kernel<256, kModeI8>, NarrowCfg<256>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<64, kModeI8>, NarrowCfg<64>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<32, kModeI8>, NarrowCfg<32>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_pair_kernel<kModeI8>, pair::SMEM_BYTES2);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<256, kModeF16>, NarrowCfg<256>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<64, kModeF16>, NarrowCfg<64>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<32, kModeF16>, NarrowCfg<32>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_pair_kernel<kModeF16>, pair::SMEM_BYTES2);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<256, kModeDigits>, NarrowCfg<256>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<64, kModeDigits>, NarrowCfg<64>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_kernel<32, kModeDigits>, NarrowCfg<32>::kSmemBytes);
    if (e == cudaSuccess) e = reserve_smem(qlinear_i8_pair_kernel<kModeDigits>, pair::SMEM_BYTES2);
    results[dev] = e;
  });
  if (results[dev] != cudaSuccess)
    return fail(LC_ERR_CUDA, "cannot reserve %d bytes of shared memory: %s", SMEM_BYTES,
                cudaGetErrorString(results[dev]));
  return LC_OK;
}

// Instruction descriptor for kind::f16 with fp32 accumulation: D format f32 (1) in bits [4,6),
// A and B formats in [7,10) and [10,13) (0 = f16, 1 = bf16), both K-major, N >> 3 in [17,23),
// M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_f16(bool bf16, int n, int m) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Picks the kernel (CTA pair or single CTA at one of three tile widths) and launches it; shared
// by the int8 and the weight-only entry points.  `weight_bytes` decides between latency-bound and
// bandwidth-bound tile widths of the single-CTA kernel.
template <int MODE>
static int32_t launch_gemm(const void* a, int64_t a_row_bytes, int64_t lda_bytes, const void* b,
                           int64_t b_row_bytes, int64_t ldb_bytes, Params& p, int variant, uint32_t idesc_pair,
                           bool idesc_a_flag, int64_t weight_bytes, cudaStream_t st, const char* what) {
  const int64_t M = p.M, N = p.N;
  // CTA pairs pay off once there is more than one 128-row tile of A; a single row tile
  // would leave half of every pair idle
  const bool use_pair = variant == 2 || (variant == 0 && M > BM);
  // tile width of the single-CTA kernel (variant 1 forces the full width): weights of up to
  // 8 MB are latency-bound, and the widest of 64 / 32 columns that still gives every SM a tile
  // spreads them over the machine (C1: 16 CTAs x 11.1 us -> 128 CTAs x 6.8 us); every narrower
  // tile re-reads its 128 rows of A, so larger weights keep the full width (measured: 58 MB at
  // 64 columns takes 31 us against 19 us)
  const int64_t sms = sm_count();
  int bnt = BN;
  if (!use_pair && variant == 0 && weight_bytes <= (int64_t{8} << 20)) {
    const int64_t tiles_m = (M + BM - 1) / BM;
    if (tiles_m * ((N + 255) / 256) < sms) bnt = tiles_m * ((N + 63) / 64) >= sms ? 64 : 32;
  }
  CUtensorMap map_a, map_b;
  if (int32_t rc = make_map(&map_a, a, M, a_row_bytes, lda_bytes, BM)) return rc;
  if (int32_t rc = make_map(&map_b, b, N, b_row_bytes, ldb_bytes, use_pair ? pair::BNH : bnt)) return rc;
  if (int32_t rc = ensure_smem_attr()) return rc;
  if (use_pair) {
    const int64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const int64_t pairs = tiles < sms / 2 ? tiles : sms / 2;
    // launched so that its set-up (barriers, TMEM allocation) may overlap the tail of the kernel
    // that produced its operands; it waits for that kernel before its first load
    const cudaError_t err = launch_overlapped(qlinear_i8_pair_kernel<MODE>, dim3(static_cast<unsigned>(2 * pairs)),
                                              dim3(NUM_THREADS), pair::SMEM_BYTES2, st, map_a, map_b, p, idesc_pair);
    if (err != cudaSuccess) return fail(LC_ERR_CUDA, "%s (cta pair): %s", what, cudaGetErrorString(err));
    return check_launch(what);
  }
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + bnt - 1) / bnt);
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  const uint32_t idesc = MODE == kModeF16 ? make_idesc_f16(idesc_a_flag, bnt, BM) : make_idesc(idesc_a_flag, bnt);
  cudaError_t err;
  if (bnt == 256)
    err = launch_overlapped(qlinear_i8_kernel<256, MODE>, dim3(grid), dim3(NUM_THREADS), NarrowCfg<256>::kSmemBytes, st,
                            map_a, map_b, p, idesc);
  else if (bnt == 64)
    err = launch_overlapped(qlinear_i8_kernel<64, MODE>, dim3(grid), dim3(NUM_THREADS), NarrowCfg<64>::kSmemBytes, st,
                            map_a, map_b, p, idesc);
  else
    err = launch_overlapped(qlinear_i8_kernel<32, MODE>, dim3(grid), dim3(NUM_THREADS), NarrowCfg<32>::kSmemBytes, st,
                            map_a, map_b, p, idesc);
  if (err != cudaSuccess) return fail(LC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return check_launch(what);
}

}  // namespace gemm
}  // namespace lc

using namespace lc;

extern "C" int32_t lc_qlinear_i8(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b,
                                 int64_t ldb, int64_t M, int64_t N, int64_t K, const float* sx,
                                 int32_t sx_per_row, const float* zx, const int32_t* wsum,
                                 const float* sw, const float* bias, void* out, int32_t out_dtype,
                                 int64_t ldo, int32_t* status, void* stream) {
  return lc_qlinear_i8_ex(a, a_unsigned, lda, b, ldb, M, N, K, sx, sx_per_row, zx, wsum, sw, bias, out,
                          out_dtype, ldo, status, 0, stream);
}

extern "C" int32_t lc_qlinear_i8_ex(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b,
                                    int64_t ldb, int64_t M, int64_t N, int64_t K, const float* sx,
                                    int32_t sx_per_row, const float* zx, const int32_t* wsum,
                                    const float* sw, const float* bias, void* out, int32_t out_dtype,
                                    int64_t ldo, int32_t* status, int32_t variant, void* stream) {
  void* outs[1] = {out};
  return lc_qlinear_i8_multi(a, a_unsigned, lda, b, ldb, M, N, K, sx, sx_per_row, zx, wsum, sw, bias, outs, 1,
                             out_dtype, ldo, status, variant, stream);
}

extern "C" int32_t lc_qlinear_i8_multi(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b,
                                       int64_t ldb, int64_t M, int64_t N, int64_t K, const float* sx,
                                       int32_t sx_per_row, const float* zx, const int32_t* wsum,
                                       const float* sw, const float* bias, void* const* host_outs,
                                       int32_t n_out, int32_t out_dtype, int64_t ldo, int32_t* status,
                                       int32_t variant, void* stream) {
  using namespace lc::gemm;
  if (!host_outs || n_out < 1 || n_out > 8)
    return fail(LC_ERR_INVALID_ARG, "qlinear_i8: between 1 and 8 output buffers are required");
  void* out = host_outs[0];
  for (int i = 0; i < n_out; ++i)
    if (!host_outs[i]) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: null output buffer %d", i);
  // bit 8 of `variant` is the wait test: the producer role issues no loads and every wait gives up
  // after a few thousand cycles, so the kernel records a code in `status` and returns
  const int wait_test = (variant & LC_QLINEAR_WAIT_TEST) ? 1 : 0;
  const int multicast = (variant & LC_QLINEAR_MULTICAST_OUT) ? 1 : 0;
  variant &= ~(LC_QLINEAR_WAIT_TEST | LC_QLINEAR_MULTICAST_OUT);
  if (wait_test && !status) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: the wait test needs a status word");
  if (multicast && (n_out != 1 || out_dtype != LC_F32 || N % 4 || (ldo * 4) % 16 || !aligned(host_outs[0], 16)))
    return fail(LC_ERR_UNSUPPORTED, "qlinear_i8: a multicast output needs one fp32 buffer, N a multiple of 4 and "
                                    "16-byte aligned rows");
  if (variant < 0 || variant > 2) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: variant must be 0, 1 or 2");
  if (M < 0 || N < 0 || K <= 0) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: bad shape");
  if (M == 0 || N == 0) return LC_OK;
  if (!a || !b || !out) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: null pointer");
  if (lda < K || ldb < K || ldo < N) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: leading dimension too small");
  if (lda % 16 || ldb % 16 || !aligned(a, 16) || !aligned(b, 16))
    return fail(LC_ERR_UNSUPPORTED,
                "qlinear_i8: operand rows must start on 16-byte boundaries (pad lda/ldb to 16)");
  if ((zx == nullptr) != (wsum == nullptr))
    return fail(LC_ERR_INVALID_ARG, "qlinear_i8: zx and wsum go together");
  if (out_dtype != LC_F32 && out_dtype != LC_BF16 && out_dtype != LC_S32)
    return fail(LC_ERR_UNSUPPORTED, "qlinear_i8: out_dtype %d not supported", out_dtype);
  if (out_dtype != LC_S32 && !sx) return fail(LC_ERR_INVALID_ARG, "qlinear_i8: sx is required");
  if (M > 0x7fffffffLL - BM || N > 0x7fffffffLL - BN || K > 0x7fffffffLL - BK)
    return fail(LC_ERR_UNSUPPORTED, "qlinear_i8: dimension exceeds the TMA coordinate range");

  // decode batches against a large weight: the weight-streaming GEMV-shaped kernel (identical results)
  if (n_out == 1 && !multicast && !wait_test && variant == 0 && qgemv_i8_applies(M, N, K, lda, ldb, a, b, out_dtype))
    return launch_qgemv_i8(a, a_unsigned, lda, b, ldb, M, N, K, sx, sx_per_row, zx, wsum, sw, bias, out, out_dtype, ldo,
                           status, as_stream(stream));

  Params p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.sx = sx;
  p.sx_per_row = sx_per_row;
  p.zx = zx;
  p.wsum = wsum;
  p.sw = sw;
  p.bias = bias;
  for (int i = 0; i < 8; ++i) p.outs[i] = i < n_out ? host_outs[i] : nullptr;
  p.n_out = n_out;
  p.out_dtype = out_dtype;
  p.ldo = ldo;
  const size_t esz = (out_dtype == LC_BF16) ? 2 : 4;
  p.out_vec = ((ldo * esz) % 16 == 0) ? 1 : 0;
  for (int i = 0; i < n_out; ++i)
    if (!aligned(host_outs[i], 16)) p.out_vec = 0;
  p.status = status;
  p.fast_f32 = (out_dtype == LC_F32 && sw && n_out == 1 && p.out_vec && !multicast) ? 1 + (zx ? 1 : 0) + (bias ? 2 : 0) : 0;
  p.multicast = multicast;

  p.wait_test = wait_test;
  p.rows_out = M;
  p.kb_wrap = 1;
  p.rowsum = nullptr;
  p.colcorr = nullptr;
  p.relu = 0;
  p.fq_scale = nullptr;
  p.fq_zp = nullptr;
  p.fq_min = p.fq_max = 0.0f;
  return launch_gemm<kModeI8>(a, K, lda, b, K, ldb, p, variant, make_idesc_pair(a_unsigned != 0), a_unsigned != 0,
                            N * K, as_stream(stream), "qlinear_i8");
}

// Status word of lc_qlinear_i8* / lc_wo_gemm_16 read back on the host.
extern "C" int32_t lc_qlinear_check_status(const int32_t* status, int32_t clear, void* stream) {
  if (!status) return fail(LC_ERR_INVALID_ARG, "qlinear_check_status: null pointer");
  cudaStream_t st = as_stream(stream);
  int32_t code = 0;
  cudaError_t err = cudaMemcpyAsync(&code, status, sizeof(code), cudaMemcpyDeviceToHost, st);
  if (err == cudaSuccess) err = cudaStreamSynchronize(st);
  if (err == cudaSuccess && clear && code != 0)
    err = cudaMemsetAsync(const_cast<int32_t*>(status), 0, sizeof(code), st);
  if (err != cudaSuccess) return fail(LC_ERR_CUDA, "qlinear_check_status: %s", cudaGetErrorString(err));
  if (code == 0) return LC_OK;
  static const char* const kRole[] = {"", "the TMA producer", "the MMA issuer", "an epilogue warp",
                                      "the barrier between ranks (a peer never arrived)"};
  return fail(LC_ERR_TIMEOUT, "a bounded device-side wait of %s ran out (status %d); the kernel returned early and "
                              "its output is incomplete", code >= 1 && code <= 4 ? kRole[code] : "a kernel role", code);
}

// Weight-only Linear on the tensor cores (see the header of this file).
extern "C" int32_t lc_wo_gemm_16(const void* a, int32_t a_dtype, int32_t n_terms, int64_t lda, const void* w16,
                                 int64_t ldw, int64_t M, int64_t N, int64_t K, const float* sw, const float* bias,
                                 const float* rowsum, const float* colcorr, int32_t relu, const float* out_scale,
                                 const float* out_zp, int32_t quant_min, int32_t quant_max, void* out,
                                 int32_t out_dtype, int64_t ldo, int32_t* status, int32_t variant, void* stream) {
  using namespace lc::gemm;
  if (M < 0 || N < 0 || K <= 0) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: bad shape");
  if (M == 0 || N == 0) return LC_OK;
  if (!a || !w16 || !out) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: null pointer");
  if (a_dtype != LC_BF16 && a_dtype != LC_F16)
    return fail(LC_ERR_UNSUPPORTED, "wo_gemm_16: operands must be bf16 or f16 (dtype %d)", a_dtype);
  if (n_terms < 1 || n_terms > 3) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: n_terms must be 1, 2 or 3");
  const int wait_test = (variant & LC_QLINEAR_WAIT_TEST) ? 1 : 0;
  variant &= ~LC_QLINEAR_WAIT_TEST;
  if (wait_test && !status) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: the wait test needs a status word");
  if (variant < 0 || variant > 2) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: variant must be 0, 1 or 2");
  // one K block = 64 elements = one 128-byte swizzle atom; with several terms every term starts
  // on a block boundary, so K must then be a whole number of blocks (the caller zero-pads)
  const int64_t kblocks = (K + 63) / 64;
  if (n_terms > 1 && K % 64) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: with several terms K must be a multiple of 64");
  if (lda < n_terms * K || ldw < K || ldo < N) return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: leading dimension too small");
  if (lda % 8 || ldw % 8 || K % 8 || !aligned(a, 16) || !aligned(w16, 16))
    return fail(LC_ERR_UNSUPPORTED, "wo_gemm_16: operand rows must start on 16-byte boundaries and K be a multiple of 8");
  if (out_dtype != LC_F32 && out_dtype != LC_BF16 && out_dtype != LC_F16)
    return fail(LC_ERR_UNSUPPORTED, "wo_gemm_16: out_dtype %d not supported", out_dtype);
  if ((rowsum == nullptr) != (colcorr == nullptr))
    return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: rowsum and colcorr go together");
  if ((out_scale == nullptr) != (out_zp == nullptr))
    return fail(LC_ERR_INVALID_ARG, "wo_gemm_16: out_scale and out_zp go together");
  if (M > 0x7fffffffLL - BM || N > 0x7fffffffLL - BN || n_terms * K * 2 > 0x7fffffffLL - BK)
    return fail(LC_ERR_UNSUPPORTED, "wo_gemm_16: dimension exceeds the TMA coordinate range");

  Params p;
  p.M = M;
  p.N = N;
  p.K = n_terms * kblocks * BK;  // bytes of K the main loop walks (A side)
  p.sx = nullptr;
  p.sx_per_row = 0;
  p.zx = nullptr;
  p.wsum = nullptr;
  p.sw = sw;
  p.bias = bias;
  for (int i = 0; i < 8; ++i) p.outs[i] = i == 0 ? out : nullptr;
  p.n_out = 1;
  p.out_dtype = out_dtype;
  p.ldo = ldo;
  const size_t esz = (out_dtype == LC_F32) ? 4 : 2;
  p.out_vec = ((ldo * esz) % 16 == 0 && aligned(out, 16)) ? 1 : 0;
  p.fast_f32 = 0;
  p.status = status;
  p.multicast = 0;
  p.wait_test = wait_test;
  p.rows_out = M;
  p.kb_wrap = static_cast<int>(kblocks);
  p.rowsum = rowsum;
  p.colcorr = colcorr;
  p.relu = relu ? 1 : 0;
  p.fq_scale = out_scale;
  p.fq_zp = out_zp;
  p.fq_min = static_cast<float>(quant_min);
  p.fq_max = static_cast<float>(quant_max);
  const bool bf16 = a_dtype == LC_BF16;
  return launch_gemm<kModeF16>(a, n_terms * K * 2, lda * 2, w16, K * 2, ldw * 2, p, variant,
                           make_idesc_f16(bf16, BN, 2 * BM), bf16, N * K * 2, as_stream(stream), "wo_gemm_16");
}

// Weight-only Linear for fp32 activations on exact integer arithmetic (see the header of this file).
extern "C" int32_t lc_wo_gemm_digits(const int8_t* digits, int64_t ldd, const float* row_scale, const int8_t* wq,
                                     int64_t ldw, int64_t M, int64_t N, int64_t K, const float* sw,
                                     const float* bias, const float* rowsum, const float* colcorr, int32_t relu,
                                     const float* out_scale, const float* out_zp, int32_t quant_min,
                                     int32_t quant_max, float* out, int64_t ldo, int32_t* status, int32_t variant,
                                     void* stream) {
  using namespace lc::gemm;
  if (M < 0 || N < 0 || K <= 0) return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: bad shape");
  if (M == 0 || N == 0) return LC_OK;
  if (!digits || !row_scale || !wq || !out) return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: null pointer");
  const int wait_test = (variant & LC_QLINEAR_WAIT_TEST) ? 1 : 0;
  variant &= ~LC_QLINEAR_WAIT_TEST;
  if (wait_test && !status) return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: the wait test needs a status word");
  if (variant < 0 || variant > 2) return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: variant must be 0, 1 or 2");
  if (ldd < K || ldw < K || ldo < N) return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: leading dimension too small");
  if (ldd % 16 || ldw % 16 || !aligned(digits, 16) || !aligned(wq, 16))
    return fail(LC_ERR_UNSUPPORTED, "wo_gemm_digits: operand rows must start on 16-byte boundaries (pad ldd/ldw to 16)");
  if ((rowsum == nullptr) != (colcorr == nullptr))
    return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: rowsum and colcorr go together");
  if ((out_scale == nullptr) != (out_zp == nullptr))
    return fail(LC_ERR_INVALID_ARG, "wo_gemm_digits: out_scale and out_zp go together");
  const int64_t plane_rows = lc_wo_digit_rows(M);
  if (plane_rows > 0x7fffffffLL - 2 * BM || N > 0x7fffffffLL - BN || K > 0x7fffffffLL - BK)
    return fail(LC_ERR_UNSUPPORTED, "wo_gemm_digits: dimension exceeds the TMA coordinate range");
  // |sum| <= K * 2^30 * 128 must stay inside the 64-bit recombination and each plane's int32 sum
  if (K > (int64_t{1} << 17)) return fail(LC_ERR_UNSUPPORTED, "wo_gemm_digits: K above 131072 could overflow int32");

  Params p;
  p.M = plane_rows;
  p.N = N;
  p.K = K;
  p.sx = row_scale;
  p.sx_per_row = 1;
  p.zx = nullptr;
  p.wsum = nullptr;
  p.sw = sw;
  p.bias = bias;
  for (int i = 0; i < 8; ++i) p.outs[i] = i == 0 ? out : nullptr;
  p.n_out = 1;
  p.out_dtype = LC_F32;
  p.ldo = ldo;
  p.out_vec = 0;
  p.fast_f32 = 0;
  p.status = status;
  p.multicast = 0;
  p.wait_test = wait_test;
  p.rows_out = M;
  p.kb_wrap = 1;
  p.rowsum = rowsum;
  p.colcorr = colcorr;
  p.relu = relu ? 1 : 0;
  p.fq_scale = out_scale;
  p.fq_zp = out_zp;
  p.fq_min = static_cast<float>(quant_min);
  p.fq_max = static_cast<float>(quant_max);
  return launch_gemm<kModeDigits>(digits, K, ldd, wq, K, ldw, p, variant, make_idesc_pair(false), false, N * K,
                                  as_stream(stream), "wo_gemm_digits");
}

// ---- the dynamic Linear forward as ONE call ------------------------------------------------------
// Activation quantization (per tensor or per row) and the GEMM, issued back to back on the stream from
// one entry point with one caller workspace: an eager framework pays the host cost of a call (argument
// marshalling, allocator, stream query) once per layer instead of three times.
namespace {
constexpr int64_t kDynAlign = 256;
inline int64_t dyn_round(int64_t v) { return (v + kDynAlign - 1) / kDynAlign * kDynAlign; }
inline int64_t dyn_pad16(int64_t k) { return (k + 15) / 16 * 16; }
}  // namespace

extern "C" int64_t lc_dynamic_linear_workspace_bytes(int64_t M, int64_t K) {
  if (M < 0 || K <= 0) return 0;
  // codes [M, pad16(K)], per-row scales and zero-points, {min, max}, scratch of the global-range kernel
  return dyn_round(M * dyn_pad16(K)) + 2 * dyn_round(M * 4 + 4) + dyn_round(16) +
         dyn_round(lc_observe_tensor_workspace_bytes());
}

extern "C" int32_t lc_dynamic_linear_f32(const float* x, int64_t ldx, int64_t M, int64_t K, int32_t act_scheme,
                                         int32_t quant_min, int32_t quant_max, int32_t is_signed, float eps,
                                         const int8_t* wq, int64_t ldw, int64_t N, const float* sw,
                                         const float* bias, const int32_t* wsum, void* out, int32_t out_dtype,
                                         int64_t ldo, void* workspace, int64_t workspace_bytes,
                                         int32_t workspace_is_fresh, int32_t* status, void* stream) {
  if (act_scheme < 0 || act_scheme > 2)
    return fail(LC_ERR_INVALID_ARG, "dynamic_linear: act_scheme must be 0 (tensor affine), 1 (tensor symmetric) or "
                                    "2 (token symmetric)");
  if (M < 0 || N < 0 || K <= 0 || ldx < K) return fail(LC_ERR_INVALID_ARG, "dynamic_linear: bad shape");
  if (M == 0 || N == 0) return LC_OK;
  if (!x || !wq || !out || !workspace) return fail(LC_ERR_INVALID_ARG, "dynamic_linear: null pointer");
  if (workspace_bytes < lc_dynamic_linear_workspace_bytes(M, K) || !aligned(workspace, 256))
    return fail(LC_ERR_WORKSPACE, "dynamic_linear: workspace of %lld bytes (256-byte aligned) required",
                (long long)lc_dynamic_linear_workspace_bytes(M, K));
  uint8_t* base = static_cast<uint8_t*>(workspace);
  const int64_t ldq = dyn_pad16(K);
  void* codes = base;
  float* scale = reinterpret_cast<float*>(base + dyn_round(M * ldq));
  float* zp = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scale) + dyn_round(M * 4 + 4));
  float* minmax = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(zp) + dyn_round(M * 4 + 4));
  void* observe_ws = reinterpret_cast<uint8_t*>(minmax) + dyn_round(16);
  const int64_t observe_bytes = lc_observe_tensor_workspace_bytes();
  const int code_dtype = is_signed ? LC_S8 : LC_U8;
  if (act_scheme == 2) {
    if (int32_t rc = lc_dynamic_quantize_rows_f32(x, M, K, ldx, 1, quant_min, quant_max, is_signed, eps, codes,
                                                  code_dtype, ldq, scale, zp, stream))
      return rc;
    return lc_qlinear_i8(codes, is_signed ? 0 : 1, ldq, wq, ldw, M, N, K, scale, 1, nullptr, nullptr, sw, bias, out,
                         out_dtype, ldo, status, stream);
  }
  // the global-range kernel wants its scratch zero-filled before its first use and leaves it zero
  if (workspace_is_fresh &&
      cudaMemsetAsync(observe_ws, 0, static_cast<size_t>(observe_bytes), as_stream(stream)) != cudaSuccess)
    return fail(LC_ERR_CUDA, "dynamic_linear: %s", cudaGetErrorString(cudaGetLastError()));
  const int symmetric = act_scheme == 1;
  if (int32_t rc = lc_dynamic_quantize_tensor_f32(x, M, K, ldx, symmetric, quant_min, quant_max, is_signed, eps,
                                                  codes, code_dtype, ldq, scale, zp, minmax, observe_ws,
                                                  observe_bytes, stream))
    return rc;
  const bool needs_zp = !(symmetric && is_signed);
  if (needs_zp && !wsum) return fail(LC_ERR_INVALID_ARG, "dynamic_linear: this activation grid needs wsum");
  return lc_qlinear_i8(codes, is_signed ? 0 : 1, ldq, wq, ldw, M, N, K, scale, 0, needs_zp ? zp : nullptr,
                       needs_zp ? wsum : nullptr, sw, bias, out, out_dtype, ldo, status, stream);
}
