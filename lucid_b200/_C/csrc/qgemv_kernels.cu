// GEMV-shaped int8 x int8 product for decode batches of the dynamically quantized Linear
// (lucid/nn/quantized/dynamic/linear.py:85-109: quantize the activations, multiply against the int8
// weight, rescale): out = f32(acc - zx * wsum[n]) * sx[m] * sw[n] + bias[n] for up to 16 rows of
// activation codes against a weight of 4 MB and more.
//
// The tensor-core GEMM serves such a batch with 128 x 32 tiles whose CTAs keep six 4 KB weight pieces
// in flight, which caps a long-K, narrow-N layer near 1.4 TB/s of weight bytes.  Here the weight is
// streamed once through a shared-memory ring like the weight-only layers' (16-row x 1024-byte TMA boxes,
// two half-size CTAs per SM, a producer thread and eight consumer warps that split a box row into
// 64-byte units), and the codes go to `mma.sync.m16n8k32` as they are: the int32 accumulator is exact,
// so results equal the GEMM's bit for bit.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace lc {
namespace {

namespace gv {
constexpr int KC = 1024;          // bytes of K per box row
constexpr int STAGE = 16 * KC;    // one box: a 16-row tile of one K chunk
constexpr int CW = 8;             // consumer warps
constexpr int THREADS = CW * 32 + 32;
constexpr int SMEM = 115584;      // two CTAs per SM
constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s
// (tm = row tiles per pass, nt = batch tiles of 8 rows)
__host__ __device__ constexpr int red_bytes(int nt, int tm) { return tm * CW * 16 * nt * 8 * 4; }
__host__ __device__ constexpr int stages(int nt, int tm) { return (SMEM - 256 - red_bytes(nt, tm)) / STAGE; }
}  // namespace gv

struct QgemvParams {
  const void* a;       // activation codes [M, lda]
  int64_t lda, M, N, K;
  const float* sx;     // per row or one value; null with int32 output
  int sx_per_row;
  const float* zx;     // device scalar or null
  const int32_t* wsum;
  const float* sw;
  const float* bias;
  void* out;           // fp32 or int32 [M, ldo]
  int64_t ldo;
  int out_s32;
  int32_t* status;     // optional: 1 = producer wait ran out, 2 = consumer wait ran out
  int tiles_per_cta;
};

__device__ __forceinline__ uint32_t gv_smem(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool gv_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  long long t0 = 0;
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
    else if (clock64() - t0 > gv::kWaitCycles)
      return false;
  }
}
__device__ __forceinline__ void gv_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gv_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gv_load_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 gv_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// weights (A, signed) x activation codes (B, signed or unsigned), int32 accumulation: exact
template <bool XU>
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  if constexpr (XU)
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// XU: activation codes are unsigned bytes.  NT: batch tiles of 8 rows (1, 2 or 4).  TMAX: row tiles per pass.
template <bool XU, int NT, int TMAX>
__global__ void __launch_bounds__(gv::THREADS, 2)
qgemv_i8_kernel(const __grid_constant__ CUtensorMap tmap_w, const QgemvParams p) {
  using namespace gv;
  constexpr int S = stages(NT, TMAX), COLS = NT * 8;
  static_assert(S >= 3, "ring too shallow");
  extern __shared__ uint8_t gv_smem_raw[];
  const uint32_t base = (gv_smem(gv_smem_raw) + 127u) & ~127u;
  const uint32_t red_base = base + S * STAGE;
  const uint32_t bar_base = red_base + red_bytes(NT, TMAX);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  int* red = reinterpret_cast<int*>(gv_smem_raw + (red_base - gv_smem(gv_smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == CW && lane == 0)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
  const int num_kc = static_cast<int>((p.K + KC - 1) / KC);
  const int64_t tiles = (p.N + 15) / 16;
  const int64_t tile_begin = static_cast<int64_t>(blockIdx.x) * p.tiles_per_cta;
  int64_t tile_end = tile_begin + p.tiles_per_cta;
  if (tile_end > tiles) tile_end = tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(CW) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == CW) {
    // ===================== producer: boxes in consumption order (pass, K chunk, tile) =====================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed_mask = 0, armed_parity = 0;
      bool ok = true;
      for (int64_t t0 = tile_begin; t0 < tile_end && ok; t0 += TMAX) {
        const int pass_tiles = static_cast<int>(tile_end - t0 < TMAX ? tile_end - t0 : TMAX);
        for (int kc = 0; kc < num_kc && ok; ++kc)
          for (int j = 0; j < pass_tiles; ++j) {
            if (!gv_wait(empty_bar(stage), phase ^ 1u)) {
              if (p.status) atomicCAS(p.status, 0, 1);
              ok = false;
              break;
            }
            gv_expect(full_bar(stage), STAGE);
            gv_load_box(base + stage * STAGE, &tmap_w, kc * (KC / 4), static_cast<int>((t0 + j) << 4), full_bar(stage));
            armed_mask |= 1u << stage;
            armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
            if (++stage == S) {
              stage = 0;
              phase ^= 1u;
            }
          }
      }
      // do not leave while one of this CTA's bulk copies may still be landing
      for (int s = 0; s < S; ++s)
        if (armed_mask & (1u << s)) gv_wait(full_bar(s), (armed_parity >> s) & 1u);
    }
    return;
  }

  // ===================== consumers =====================
  const int g = lane >> 2, t = lane & 3;
  const int kbase = warp * 128 + t * 16;  // this lane's 16 bytes of unit 0 of a box row; unit 1 lies 64 bytes further
  const uint8_t* xa = static_cast<const uint8_t*>(p.a);
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  const int zx_i = p.zx ? __float2int_rn(__ldg(p.zx)) : 0;
  for (int64_t t0 = tile_begin; t0 < tile_end; t0 += TMAX) {
    const int pass_tiles = static_cast<int>(tile_end - t0 < TMAX ? tile_end - t0 : TMAX);
    int acc[TMAX][NT][4];
#pragma unroll
    for (int j = 0; j < TMAX; ++j)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][nt][i] = 0;
    // activation codes of this lane: 16 bytes per unit and batch row nt * 8 + g, fetched D chunks ahead (a chunk
    // of a single-tile pass is one 16 KB box, shorter than a round trip to the L2)
    // (four batch tiles leave no registers for a second set: they load where the codes are needed)
    constexpr int D = NT == 1 ? 2 : (NT == 2 ? 1 : 0);
    uint4 xq[D > 0 ? D : 1][NT][2];
    auto load_x = [&](int kc, uint4 (&dst)[NT][2]) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int64_t k = static_cast<int64_t>(kc) * KC + kbase + 64 * u;
          const int b = nt * 8 + g;
          dst[nt][u] = (kc < num_kc && k < p.K && b < p.M)
                           ? __ldg(reinterpret_cast<const uint4*>(xa + static_cast<int64_t>(b) * p.lda + k))
                           : make_uint4(0u, 0u, 0u, 0u);
        }
    };
#pragma unroll
    for (int d = 0; d < D; ++d) load_x(d, xq[d]);
    for (int kc = 0; kc < num_kc; ++kc) {
      uint4 xc[NT][2];
      if constexpr (D == 0) {
        load_x(kc, xc);
      } else {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            xc[nt][u] = xq[0][nt][u];
#pragma unroll
            for (int d = 0; d + 1 < D; ++d) xq[d][nt][u] = xq[d + 1][nt][u];
          }
        load_x(kc + D, xq[D > 0 ? D - 1 : 0]);
      }
#pragma unroll
      for (int j = 0; j < TMAX; ++j) {
        if (j < pass_tiles && ok) {
          if (!gv_wait(full_bar(stage), phase)) {
            if (p.status) atomicCAS(p.status, 0, 2);
            ok = false;
          } else {
            const uint32_t src = base + stage * STAGE + g * KC + kbase;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const uint4 w0 = gv_lds128(src + 64 * u), w1 = gv_lds128(src + 64 * u + 8 * KC);  // rows g, g + 8
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                mma_s8<XU>(acc[j][nt], w0.x, w1.x, w0.y, w1.y, xc[nt][u].x, xc[nt][u].y);
                mma_s8<XU>(acc[j][nt], w0.z, w1.z, w0.w, w1.w, xc[nt][u].z, xc[nt][u].w);
              }
            }
            // the slot goes back to the copy engine (async proxy): order this warp's reads before that
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) gv_arrive(empty_bar(stage));
            if (++stage == S) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
    // ---- the eight K slices of the pass are added up (integers: any order) and finished ----
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");  // the previous pass has been read out
#pragma unroll
    for (int j = 0; j < TMAX; ++j)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        int* dst = red + ((j * CW + warp) * 16) * COLS + nt * 8 + 2 * t;
        dst[g * COLS] = acc[j][nt][0];
        dst[g * COLS + 1] = acc[j][nt][1];
        dst[(g + 8) * COLS] = acc[j][nt][2];
        dst[(g + 8) * COLS + 1] = acc[j][nt][3];
      }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    for (int e = threadIdx.x; e < pass_tiles * 16 * COLS; e += CW * 32) {
      const int j = e / (16 * COLS), r = (e / COLS) & 15, bcol = e % COLS;
      const int64_t n = ((t0 + j) << 4) + r;
      if (n >= p.N || bcol >= p.M || !ok) continue;
      int sum = 0;
#pragma unroll
      for (int w = 0; w < CW; ++w) sum += red[((j * CW + w) * 16 + r) * COLS + bcol];
      if (p.wsum) sum -= zx_i * __ldg(p.wsum + n);
      if (p.out_s32) {
        static_cast<int32_t*>(p.out)[static_cast<int64_t>(bcol) * p.ldo + n] = sum;
      } else {
        float f = __fmul_rn(static_cast<float>(sum), __ldg(p.sx + (p.sx_per_row ? bcol : 0)));
        if (p.sw) f = __fmul_rn(f, __ldg(p.sw + n));
        if (p.bias) f = __fadd_rn(f, __ldg(p.bias + n));
        static_cast<float*>(p.out)[static_cast<int64_t>(bcol) * p.ldo + n] = f;
      }
    }
  }
}

template <bool XU, int NT, int TMAX>
int32_t launch_qgemv_inst(const CUtensorMap& map, const QgemvParams& p, unsigned grid, cudaStream_t st) {
  auto kernel = qgemv_i8_kernel<XU, NT, TMAX>;
  static std::once_flag flags[64];
  static cudaError_t results[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(LC_ERR_CUDA, "no current CUDA device");
  std::call_once(flags[dev], [&]() {
    results[dev] = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gv::SMEM);
    if (results[dev] == cudaSuccess)
      results[dev] = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  });
  if (results[dev] != cudaSuccess)
    return fail(LC_ERR_CUDA, "qlinear_i8 (gemv): cannot reserve shared memory: %s", cudaGetErrorString(results[dev]));
  kernel<<<grid, gv::THREADS, gv::SMEM, st>>>(map, p);
  return check_launch("qlinear_i8 (gemv)");
}

}  // namespace

bool qgemv_i8_applies(int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, const void* a, const void* b,
                      int32_t out_dtype) {
  // 17..32 rows (four batch tiles, eight MMAs per unit: the consumer warps set the pace) are worth it against the
  // GEMM's 128 x 32 tiles only while N gives those few CTAs (measured at 32 rows, us: [4096, 14336] 22 against 52,
  // [4096, 4096] 10 against 14, but [14336, 4096] 24 against 20 and [28672, 4096] 43 against 25)
  if (!(M >= 1 && (M <= 16 || (M <= 32 && N < 8192)))) return false;
  return K % 16 == 0 && N * K >= (int64_t{4} << 20) && lda % 16 == 0 && ldb % 16 == 0 &&
         aligned(a, 16) && aligned(b, 16) && (out_dtype == LC_F32 || out_dtype == LC_S32) &&
         (N + 15) / 16 * ((K + gv::KC - 1) / gv::KC) < (int64_t{1} << 31);
}

int32_t launch_qgemv_i8(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b, int64_t ldb, int64_t M,
                        int64_t N, int64_t K, const float* sx, int32_t sx_per_row, const float* zx, const int32_t* wsum,
                        const float* sw, const float* bias, void* out, int32_t out_dtype, int64_t ldo, int32_t* status,
                        cudaStream_t st) {
  CUtensorMap map;
  if (int32_t rc = encode_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, b, static_cast<uint64_t>(K / 4),
                                        static_cast<uint64_t>(N), static_cast<uint64_t>(ldb), gv::KC / 4, 16,
                                        CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  const int64_t tiles = (N + 15) / 16, slots = static_cast<int64_t>(sm_count()) * 2;
  const int64_t per = (tiles + slots - 1) / slots;
  const unsigned grid = static_cast<unsigned>((tiles + per - 1) / per);
  const size_t esz = 4;  // fp32 and int32 outputs alike
  // up to 8 / 16 / 32 rows: one / two / four batch tiles per launch (the last with passes of two row tiles)
  const int64_t rows_per_launch = 32;
  for (int64_t m0 = 0; m0 < M; m0 += rows_per_launch) {
    QgemvParams p;
    p.a = static_cast<const uint8_t*>(a) + m0 * lda;
    p.lda = lda;
    p.M = M - m0 < rows_per_launch ? M - m0 : rows_per_launch;
    p.N = N;
    p.K = K;
    p.sx = sx ? sx + (sx_per_row ? m0 : 0) : nullptr;
    p.sx_per_row = sx_per_row;
    p.zx = zx;
    p.wsum = wsum;
    p.sw = sw;
    p.bias = bias;
    p.out = static_cast<uint8_t*>(out) + static_cast<size_t>(m0 * ldo) * esz;
    p.ldo = ldo;
    p.out_s32 = out_dtype == LC_S32 ? 1 : 0;
    p.status = status;
    p.tiles_per_cta = static_cast<int>(per);
    int32_t rc;
    if (p.M <= 8)
      rc = a_unsigned ? launch_qgemv_inst<true, 1, 4>(map, p, grid, st) : launch_qgemv_inst<false, 1, 4>(map, p, grid, st);
    else if (p.M <= 16)
      rc = a_unsigned ? launch_qgemv_inst<true, 2, 4>(map, p, grid, st) : launch_qgemv_inst<false, 2, 4>(map, p, grid, st);
    else
      rc = a_unsigned ? launch_qgemv_inst<true, 4, 2>(map, p, grid, st) : launch_qgemv_inst<false, 4, 2>(map, p, grid, st);
    if (rc) return rc;
  }
  return LC_OK;
}

}  // namespace lc
