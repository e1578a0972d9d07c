// Lookups in an int8 embedding table with per-row scale / zero-point: the forward of the
// quantized Embedding and EmbeddingBag (lucid/nn/quantized/sparse.py:140-143, 284-304).  The
// reference dequantizes the whole [V, D] table on every call and then gathers from the fp32
// copy; here only the looked-up rows are read, as int8, and decoded on the way out with the
// dequantize formula (lucid/quantization/_functional.py:281-293): (f32(q) - z[row]) * s[row].
// The bag pooling follows lucid/_C/backend/cpu/methods/Sequence.cpp:44-85: entries are added
// in index order starting from zero, entries equal to padding_idx are skipped, the mean divides
// by the number of entries kept, max starts from the lowest float and an empty bag gives zeros.
//
// HBM-bound: 1 byte read + 4 bytes written per looked-up element (bags: 1 byte per entry
// element, 4 bytes per bag element).  Lookup: a lane owns four adjacent columns, so a warp reads
// 128 contiguous bytes of a table row and writes 512 contiguous bytes per step.  Bags: a thread
// owns 16 adjacent columns of one bag (one 16-byte load per entry) and keeps several entries in
// flight, because a bag is a chain of dependent loads.
#include "common.cuh"

namespace lc {
namespace {

constexpr int kEmbThreads = 256;
constexpr int kEmbSeg = 1024;  // columns of one row handled by one warp (8 steps of 128)
constexpr int kErrIndex = 1;   // device status: an index outside [0, V)

__device__ __forceinline__ float4 decode4(uint32_t w, float z, float s) {
  const int a = static_cast<int8_t>(w & 0xff), b = static_cast<int8_t>((w >> 8) & 0xff);
  const int c = static_cast<int8_t>((w >> 16) & 0xff), d = static_cast<int8_t>(w >> 24);
  return make_float4(__fmul_rn(__fsub_rn(static_cast<float>(a), z), s), __fmul_rn(__fsub_rn(static_cast<float>(b), z), s),
                     __fmul_rn(__fsub_rn(static_cast<float>(c), z), s), __fmul_rn(__fsub_rn(static_cast<float>(d), z), s));
}

// out[i, :] = decode(table[idx[i], :]).  Work unit: (looked-up row, 1024-column segment); the
// warps of the grid stride over the units.  VEC: D % 4 == 0 and both buffers 16-byte aligned.
template <bool VEC>
__global__ void __launch_bounds__(kEmbThreads)
embedding_s8_kernel(const int8_t* __restrict__ table, const float* __restrict__ scale,
                    const float* __restrict__ zero_point, const int64_t* __restrict__ idx, int64_t n, int64_t V,
                    int64_t D, float* __restrict__ out, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t segs = (D + kEmbSeg - 1) / kEmbSeg;
  const int64_t units = n * segs;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (kEmbThreads / 32);
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * (kEmbThreads / 32) + (threadIdx.x >> 5); u < units; u += warps) {
    const int64_t i = u / segs, c0 = (u % segs) * kEmbSeg;
    const int64_t row = idx[i];
    const bool ok = row >= 0 && row < V;
    if (!ok && lane == 0 && status) atomicCAS(status, 0, kErrIndex);
    const float s = ok ? scale[row] : 0.f;
    const float z = ok && zero_point ? zero_point[row] : 0.f;
    const int8_t* src = table + (ok ? row : 0) * D;
    float* dst = out + i * D;
    const int64_t c1 = c0 + kEmbSeg < D ? c0 + kEmbSeg : D;
    if (VEC) {
      uint32_t w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t c = c0 + k * 128 + lane * 4;
        w[k] = (ok && c < c1) ? *reinterpret_cast<const uint32_t*>(src + c) : 0u;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t c = c0 + k * 128 + lane * 4;
        if (c < c1) __stcs(reinterpret_cast<float4*>(dst + c), ok ? decode4(w[k], z, s) : make_float4(0.f, 0.f, 0.f, 0.f));
      }
    } else {
      for (int64_t c = c0 + lane; c < c1; c += 32)
        dst[c] = ok ? __fmul_rn(__fsub_rn(static_cast<float>(src[c]), z), s) : 0.f;
    }
  }
}

struct BagSpec {
  int64_t n, bags, V, D;
  int mode;  // 0 sum, 1 mean, 2 max (the kernel is compiled per mode; kept for the record)
  int64_t padding_idx;  // negative: none
  int include_last_offset;
};

template <int MODE>
__device__ __forceinline__ float pool1(float acc, float v) {
  if (MODE == 2) return v > acc ? v : acc;
  return __fadd_rn(acc, v);
}

// out[b, :] = pool over the entries of bag b.  Work item of one thread: (bag, CW adjacent
// columns), items dealt to threads in order, so the threads of a warp read adjacent pieces of
// the same table rows (16 bytes each for CW = 16) and bags narrower than a warp share one.  A
// bag is a chain of dependent loads (index -> scale and row piece): DEPTH rows are fetched at a
// time and the indices of the next batch are requested before the current one is reduced.
// CW = 16 / 4 need embedding_dim % CW == 0 and a table aligned to CW bytes; CW = 1 takes anything.
template <int CW, int DEPTH, int MODE>
__global__ void __launch_bounds__(kEmbThreads, 4)
embedding_bag_s8_kernel(const int8_t* __restrict__ table, const float* __restrict__ scale,
                        const float* __restrict__ zero_point, const int64_t* __restrict__ idx,
                        const int64_t* __restrict__ offsets, const float* __restrict__ weights, const BagSpec sp,
                        float* __restrict__ out, int32_t* status) {
  constexpr int WORDS = CW >= 4 ? CW / 4 : 1;
  const int64_t chunks = sp.D / CW;
  const int64_t items = sp.bags * chunks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kEmbThreads;
  const float lowest = -3.402823466e+38f;
  for (int64_t it = static_cast<int64_t>(blockIdx.x) * kEmbThreads + threadIdx.x; it < items; it += stride) {
    const int64_t b = it / chunks, c = (it % chunks) * CW;
    int64_t j0 = offsets[b];
    int64_t j1 = (b + 1 < sp.bags || sp.include_last_offset) ? offsets[b + 1] : sp.n;
    if (j0 < 0) j0 = 0;
    if (j1 > sp.n) j1 = sp.n;
    float acc[CW];
#pragma unroll
    for (int e = 0; e < CW; ++e) acc[e] = MODE == 2 ? lowest : 0.f;
    int64_t count = 0;
    int64_t next[DEPTH];
#pragma unroll
    for (int k = 0; k < DEPTH; ++k) next[k] = j0 + k < j1 ? idx[j0 + k] : -1;
    for (int64_t j = j0; j < j1; j += DEPTH) {
      int64_t rows[DEPTH];
      float s[DEPTH], z[DEPTH], pw[DEPTH];
      uint32_t w[DEPTH][WORDS];
      bool use[DEPTH];
#pragma unroll
      for (int k = 0; k < DEPTH; ++k) {
        rows[k] = next[k];
        use[k] = j + k < j1 && !(sp.padding_idx >= 0 && rows[k] == sp.padding_idx);
        if (use[k] && (rows[k] < 0 || rows[k] >= sp.V)) {
          if (status) atomicCAS(status, 0, kErrIndex);
          use[k] = false;
        }
      }
#pragma unroll
      for (int k = 0; k < DEPTH; ++k) {
        s[k] = use[k] ? scale[rows[k]] : 0.f;
        z[k] = use[k] && zero_point ? zero_point[rows[k]] : 0.f;
        pw[k] = use[k] && weights ? weights[j + k] : 1.f;
#pragma unroll
        for (int q = 0; q < WORDS; ++q) w[k][q] = 0u;
        if (use[k]) {
          const int8_t* src = table + rows[k] * sp.D + c;
          if (CW == 16) {
            const uint4 v = *reinterpret_cast<const uint4*>(src);
            w[k][0] = v.x;
            w[k][WORDS > 1 ? 1 : 0] = v.y;
            w[k][WORDS > 2 ? 2 : 0] = v.z;
            w[k][WORDS > 3 ? 3 : 0] = v.w;
          } else if (CW == 4) {
            w[k][0] = *reinterpret_cast<const uint32_t*>(src);
          } else {
            w[k][0] = static_cast<uint32_t>(static_cast<uint8_t>(src[0]));
          }
        }
      }
#pragma unroll
      for (int k = 0; k < DEPTH; ++k) {
        const int64_t jn = j + DEPTH + k;
        next[k] = jn < j1 ? idx[jn] : -1;
      }
#pragma unroll
      for (int k = 0; k < DEPTH; ++k) {
        if (!use[k]) continue;
#pragma unroll
        for (int q = 0; q < WORDS; ++q) {
          const float4 v4 = decode4(w[k][q], z[k], s[k]);
          const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
          for (int e = 0; e < (CW >= 4 ? 4 : 1); ++e) {
            const float t = weights ? __fmul_rn(v[e], pw[k]) : v[e];
            acc[q * 4 + e] = pool1<MODE>(acc[q * 4 + e], t);
          }
        }
        ++count;
      }
    }
    const float cn = static_cast<float>(count);
#pragma unroll
    for (int e = 0; e < CW; ++e) {
      if (MODE == 2 && count == 0) acc[e] = 0.f;
      if (MODE == 1 && count > 0) acc[e] = __fdiv_rn(acc[e], cn);
    }
    float* dst = out + b * sp.D + c;
    if (CW >= 4) {
#pragma unroll
      for (int q = 0; q < WORDS; ++q)
        __stcs(reinterpret_cast<float4*>(dst) + q, make_float4(acc[q * 4], acc[q * 4 + 1], acc[q * 4 + 2], acc[q * 4 + 3]));
    } else {
      dst[0] = acc[0];
    }
  }
}

template <int CW, int DEPTH>
void launch_bag(int mode, unsigned grid, cudaStream_t st, const int8_t* table, const float* scale,
                const float* zero_point, const int64_t* idx, const int64_t* offsets, const float* weights,
                const BagSpec& sp, float* out, int32_t* status) {
  if (mode == 0)
    embedding_bag_s8_kernel<CW, DEPTH, 0><<<grid, kEmbThreads, 0, st>>>(table, scale, zero_point, idx, offsets, weights, sp, out, status);
  else if (mode == 1)
    embedding_bag_s8_kernel<CW, DEPTH, 1><<<grid, kEmbThreads, 0, st>>>(table, scale, zero_point, idx, offsets, weights, sp, out, status);
  else
    embedding_bag_s8_kernel<CW, DEPTH, 2><<<grid, kEmbThreads, 0, st>>>(table, scale, zero_point, idx, offsets, weights, sp, out, status);
}

unsigned grid_for(int64_t units) {
  const int64_t per_cta = kEmbThreads / 32;
  int64_t grid = (units + per_cta - 1) / per_cta;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (grid > cap) grid = cap;
  return static_cast<unsigned>(grid < 1 ? 1 : grid);
}

}  // namespace
}  // namespace lc

using namespace lc;

extern "C" int32_t lc_embedding_s8_f32(const int8_t* table, const float* scale, const float* zero_point,
                                       const int64_t* indices, int64_t n, int64_t num_embeddings,
                                       int64_t embedding_dim, float* out, int32_t* status, void* stream) {
  if (n < 0 || num_embeddings < 1 || embedding_dim < 1)
    return fail(LC_ERR_INVALID_ARG, "embedding: bad sizes n=%lld V=%lld D=%lld", (long long)n,
                (long long)num_embeddings, (long long)embedding_dim);
  if (n == 0) return LC_OK;
  if (!table || !scale || !indices || !out) return fail(LC_ERR_INVALID_ARG, "embedding: null pointer");
  const bool vec = embedding_dim % 4 == 0 && aligned(table, 4) && aligned(out, 16);
  const int64_t units = n * ((embedding_dim + kEmbSeg - 1) / kEmbSeg);
  const unsigned grid = grid_for(units);
  if (vec)
    embedding_s8_kernel<true><<<grid, kEmbThreads, 0, as_stream(stream)>>>(table, scale, zero_point, indices, n,
                                                                           num_embeddings, embedding_dim, out, status);
  else
    embedding_s8_kernel<false><<<grid, kEmbThreads, 0, as_stream(stream)>>>(table, scale, zero_point, indices, n,
                                                                            num_embeddings, embedding_dim, out, status);
  return check_launch("embedding_s8");
}

extern "C" int32_t lc_embedding_bag_s8_f32(const int8_t* table, const float* scale, const float* zero_point,
                                           const int64_t* indices, int64_t n, const int64_t* offsets, int64_t n_offsets,
                                           const float* per_sample_weights, int64_t num_embeddings,
                                           int64_t embedding_dim, int32_t mode, int64_t padding_idx,
                                           int32_t include_last_offset, float* out, int32_t* status, void* stream) {
  if (n < 0 || n_offsets < 0 || num_embeddings < 1 || embedding_dim < 1)
    return fail(LC_ERR_INVALID_ARG, "embedding_bag: bad sizes");
  if (mode < 0 || mode > 2) return fail(LC_ERR_INVALID_ARG, "embedding_bag: mode must be 0 (sum), 1 (mean) or 2 (max)");
  if (per_sample_weights && mode != 0)
    return fail(LC_ERR_INVALID_ARG, "embedding_bag: per_sample_weights needs mode sum");
  if (include_last_offset && n_offsets < 1)
    return fail(LC_ERR_INVALID_ARG, "embedding_bag: include_last_offset needs at least one offset");
  BagSpec sp;
  sp.n = n;
  sp.bags = include_last_offset ? n_offsets - 1 : n_offsets;
  sp.V = num_embeddings;
  sp.D = embedding_dim;
  sp.mode = mode;
  sp.padding_idx = padding_idx;
  sp.include_last_offset = include_last_offset ? 1 : 0;
  if (sp.bags == 0) return LC_OK;
  if (!table || !scale || !offsets || !out || (n > 0 && !indices))
    return fail(LC_ERR_INVALID_ARG, "embedding_bag: null pointer");
  int cw = (embedding_dim % 16 == 0 && aligned(table, 16) && aligned(out, 16)) ? 16
           : (embedding_dim % 4 == 0 && aligned(table, 4) && aligned(out, 16)) ? 4 : 1;
  // few, long bags: a bag is walked serially, so narrower pieces give four times the threads,
  // each with twice the entries in flight
  if (cw == 16 && sp.bags * (embedding_dim / 16) < static_cast<int64_t>(sm_count()) * 512) cw = 4;
  const int64_t items = sp.bags * (embedding_dim / cw);
  int64_t grid64 = (items + kEmbThreads - 1) / kEmbThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  const unsigned grid = static_cast<unsigned>(grid64 > cap ? cap : (grid64 < 1 ? 1 : grid64));
  cudaStream_t st = as_stream(stream);
  if (cw == 16)
    launch_bag<16, 4>(mode, grid, st, table, scale, zero_point, indices, offsets, per_sample_weights, sp, out, status);
  else if (cw == 4)
    launch_bag<4, 8>(mode, grid, st, table, scale, zero_point, indices, offsets, per_sample_weights, sp, out, status);
  else
    launch_bag<1, 8>(mode, grid, st, table, scale, zero_point, indices, offsets, per_sample_weights, sp, out, status);
  return check_launch("embedding_bag_s8");
}
