/*
 * lucid_cuda.h -- C ABI of liblucid_cuda.so, the sm_100a (B200) backend for the
 * int8 quantized-inference path of the `lucid` framework.
 *
 * The library replaces, for this path only, the reference's pybind11 engine
 * boundary `lucid._C.engine.quantized` (lucid/_C/bindings/bind_quantized.cpp:17-27,
 * registered at lucid/_C/bindings/bind.cpp:215-217) and the eager op chains the
 * Python layer builds on the engine for `lucid.quantization`
 * (lucid/quantization/_functional.py, _qparams.py, observer.py).
 *
 * Conventions
 *  - every pointer named in a signature is a DEVICE pointer unless the name
 *    starts with `host_`; the library allocates nothing, the caller owns all
 *    buffers (outputs and scratch included);
 *  - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it;
 *  - the return value is 0 on success and negative on failure (LC_ERR_*), with
 *    a thread-local message available from lc_last_error();
 *  - tensors are dense row-major; a "channel layout" is the triple
 *    (outer, channels, inner): element (o, c, i) lives at (o*channels + c)*inner + i,
 *    which covers ch_axis = 0 (outer = 1), a middle axis, and the last axis
 *    (inner = 1).  Per-tensor work uses outer = channels = 1;
 *  - there is no CPU fallback anywhere behind this interface.
 */
#ifndef LUCID_CUDA_H_
#define LUCID_CUDA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LC_OK 0
#define LC_ERR_INVALID_ARG (-1)
#define LC_ERR_UNSUPPORTED (-2)
#define LC_ERR_CUDA (-3)
#define LC_ERR_TIMEOUT (-4)
#define LC_ERR_WORKSPACE (-5)

/* element types understood by the entry points */
#define LC_F32 0
#define LC_BF16 1
#define LC_F16 2
#define LC_S8 3
#define LC_U8 4
#define LC_S16 5
#define LC_S32 6

/* ---- library / device ------------------------------------------------- */
int32_t lc_version(void);
/* copies the calling thread's last error text into buf (NUL terminated) */
int32_t lc_last_error(char* host_buf, int32_t n);
/* compute capability (major*10+minor) and SM count of `device` */
int32_t lc_device_info(int32_t device, int32_t* host_sm, int32_t* host_sm_count);
/* 0 when `stream` is not being captured into a CUDA graph, else the id of that capture (unique
 * per capture sequence).  Host code that reuses device results between calls keys them by it:
 * a kernel recorded in one capture has not run, and will not run with another graph. */
int32_t lc_stream_capture_id(void* stream, uint64_t* host_id);

/* ---- observers --------------------------------------------------------
 * MinMaxObserver.forward: running global min and max
 * (lucid/quantization/observer.py:408-414).  If accumulate != 0 the result is
 * merged into the values already in min_out/max_out (the running statistic),
 * otherwise it overwrites them.  Needs lc_observe_tensor_workspace_bytes()
 * bytes of scratch that must be zero-filled before its first use; the kernel
 * leaves it zero-filled again.  If scale_out is not NULL the last CTA also
 * evaluates calculate_qparams (lucid/quantization/_qparams.py:186-205) on the
 * merged range and writes one scale and one zero-point. */
int64_t lc_observe_tensor_workspace_bytes(void);
int32_t lc_observe_tensor_f32(const float* x, int64_t n, float* min_out, float* max_out,
                              int32_t accumulate, int32_t symmetric, int32_t quant_min,
                              int32_t quant_max, int32_t is_signed, float eps,
                              float* scale_out, float* zp_out, void* workspace,
                              int64_t workspace_bytes, void* stream);

/* lc_observe_tensor_f32 for callers that cannot give it scratch memory.
 * (This entry point has no counterpart in the reference.)
 * Some hosts of this library cannot allocate device memory at the point where they need
 * a global min/max: a serving process whose allocator took the whole GPU at start-up and
 * hands nothing to plug-ins, a binding written in a language runtime that has no CUDA
 * allocator of its own, or code that is already inside a region where cudaMalloc is not
 * allowed.  For them the kernel's scratch (a ticket and one partial min/max per CTA, about
 * 9.3 KB) is a static array inside the library; every GPU that loads the library holds it
 * until the process exits.  Nothing is allocated or freed by this call, the caller still
 * passes the input and the outputs, and results are identical to lc_observe_tensor_f32.
 * Limits and rules:
 *  - at most lc_observe_tensor_static_max_elems() (2^30) elements per call; larger inputs
 *    are rejected with LC_ERR_UNSUPPORTED -- use the workspace variant for those;
 *  - the first call on each device looks up the array's device address (with that device
 *    current); make that first call before starting any stream capture.  The address is cached
 *    while the device's primary context lives; after a context teardown (cudaDeviceReset) the
 *    next call notices the stale address and looks it up again;
 *  - all calls on a device share the one array: two calls whose kernels can overlap on the
 *    GPU (different streams, no dependency) race on it.  Serialise them. */
int64_t lc_observe_tensor_static_max_elems(void);
int32_t lc_observe_tensor_static_f32(const float* x, int64_t n, float* min_out, float* max_out,
                                     int32_t accumulate, int32_t symmetric, int32_t quant_min,
                                     int32_t quant_max, int32_t is_signed, float eps,
                                     float* scale_out, float* zp_out, void* stream);

/* lucid.histc as the histogram observer calls it (lucid/quantization/observer.py:852-870):
 * counts of x in `bins` equal-width bins over [lo, hi], lo < hi finite (the caller resolves
 * the lo == hi conventions of lucid/_ops/_adapters.py:1256-1279).  Bucketing in float64 like
 * the reference's CPU kernel (lucid/_C/backend/cpu/methods/Reduction.cpp:839-888): values
 * outside the range and NaN are skipped, bin = trunc((x - lo) / ((hi - lo) / bins)), the
 * right edge falls into the last bin; counts are exact integers converted to fp32 once
 * (lucid/_C/ops/composite/Stats.cpp:78-89).  accumulate != 0 adds the counts to `out`.
 * workspace: lc_histc_workspace_bytes(bins) bytes, 16-byte aligned, zero-filled once by the
 * caller; the kernel leaves it zero.  bins <= 16384. */
int64_t lc_histc_workspace_bytes(int32_t bins);
int32_t lc_histc_f32(const float* x, int64_t n, int32_t bins, double lo, double hi, float* out,
                     int32_t accumulate, void* workspace, int64_t workspace_bytes, void* stream);

/* PerChannelMinMaxObserver.forward: per-channel min and max over every other
 * axis (lucid/quantization/observer.py:672-686). */
int32_t lc_observe_channel_f32(const float* x, int64_t outer, int64_t channels, int64_t inner,
                               float* min_out, float* max_out, int32_t accumulate, void* stream);

/* calculate_qparams on n (min,max) pairs (lucid/quantization/_qparams.py:186-205):
 * range widened to include 0; symmetric: s = max(|min|,|max|)/((qmax-qmin)/2),
 * z = 0 (signed) or (qmax+qmin+1)/2; affine: s = (max-min)/(qmax-qmin),
 * z = clip(qmin - rint(min/s), qmin, qmax); s floored at eps.  IEEE fp32 per step. */
int32_t lc_calculate_qparams_f32(const float* min_val, const float* max_val, int64_t n,
                                 int32_t symmetric, int32_t quant_min, int32_t quant_max,
                                 int32_t is_signed, float eps, float* scale_out, float* zp_out,
                                 void* stream);

/* ---- quantize / dequantize / fake_quantize ----------------------------
 * quantize (lucid/quantization/_functional.py:59-69,179-197):
 *   q = cast(clip(rint(x * inv) + z, qmin, qmax)),  inv = 1/scale.
 * scale: device array of n_scale (1 or `channels`) floats, inverted on the
 * device with an IEEE fp32 division -- the reference's `1.0 / s` for a tensor
 * scale; or NULL, in which case host_inv_scale (the double-precision 1.0/s
 * rounded once to fp32, the reference's Python-float case) is used.
 * zero_point: device array of n_zp (1 or `channels`) floats, or NULL to use
 * host_zero_point.  out_dtype: LC_S8, LC_U8, LC_S16 or LC_S32 (the storage
 * dtypes of qint8/qint4, the GEMM's u8 operand, quint8, qint32). */
int32_t lc_quantize_f32(const float* x, int64_t outer, int64_t channels, int64_t inner,
                        const float* scale, int64_t n_scale, const float* zero_point,
                        int64_t n_zp, float host_inv_scale, float host_zero_point,
                        int32_t quant_min, int32_t quant_max, void* out, int32_t out_dtype,
                        void* stream);

/* dequantize (lucid/quantization/_functional.py:281-293): (f32(q) - z) * s.
 * q_dtype: LC_S8, LC_U8, LC_S16 or LC_S32.  out_dtype: LC_F32 (the reference's
 * result type) or LC_BF16. */
int32_t lc_dequantize(const void* q, int32_t q_dtype, int64_t outer, int64_t channels,
                      int64_t inner, const float* scale, int64_t n_scale,
                      const float* zero_point, int64_t n_zp, float host_scale,
                      float host_zero_point, void* out, int32_t out_dtype, void* stream);

/* forward of fake_quantize (lucid/quantization/_functional.py:304-333):
 *   out = (clip(rint(x*inv)+z, qmin, qmax) - z) * s
 * and, if mask_out is not NULL, the straight-through mask (1.0 where the
 * unclamped code is inside [qmin, qmax]). */
int32_t lc_fake_quantize_f32(const float* x, int64_t outer, int64_t channels, int64_t inner,
                             const float* scale, int64_t n_scale, const float* zero_point,
                             int64_t n_zp, float host_inv_scale, float host_scale,
                             float host_zero_point, int32_t quant_min, int32_t quant_max,
                             float* out, float* mask_out, void* stream);

/* fake_quantize of an element-wise merge in one pass: out = fq(a + b), fq(a * b) or
 * fq(relu(a + b)) on a per-tensor grid; b == NULL merges with host_scalar instead.  The
 * converted residual add of the reference (QFunctional.add / mul / add_relu / add_scalar /
 * mul_scalar, lucid/nn/quantized/functional_module.py:125-330, on _QuantizedGridModule._fake_quant,
 * lucid/nn/quantized/_utils.py:29-45), which runs the merge and the fake-quantize chain as
 * separate eager ops.  op: 0 add, 1 mul, 2 add + ReLU.  scale / zero_point: device scalars,
 * or NULL for the host values (as in lc_fake_quantize_f32). */
int32_t lc_fake_quantize_merge_f32(const float* a, const float* b, float host_scalar, int32_t op,
                                   int64_t n, const float* scale, const float* zero_point,
                                   float host_inv_scale, float host_scale, float host_zero_point,
                                   int32_t quant_min, int32_t quant_max, float* out, void* stream);

/* ---- fused dynamic activation quantization ---------------------------
 * One pass per row: observer + calculate_qparams + quantize for a [rows, cols]
 * fp32 matrix with row stride ldx (elements); writes codes with row stride ldq
 * (bytes == elements), one scale and one zero-point per row.  This is the
 * per-token form of the dynamic Linear's activation quantization
 * (lucid/nn/quantized/dynamic/linear.py:87-88 generalised to a per-row range)
 * and the fused form of PerChannelMinMaxObserver(ch_axis=0) + quantize. */
int32_t lc_dynamic_quantize_rows_f32(const float* x, int64_t rows, int64_t cols, int64_t ldx,
                                     int32_t symmetric, int32_t quant_min, int32_t quant_max,
                                     int32_t is_signed, float eps, void* q_out,
                                     int32_t out_dtype, int64_t ldq, float* scale_out,
                                     float* zp_out, void* stream);

/* Per-tensor dynamic quantization of a [rows, cols] matrix, the activation
 * step of the dynamic Linear (lucid/nn/quantized/dynamic/linear.py:87-88):
 * global min/max -> calculate_qparams -> quantize, scale and zero-point stay
 * on the device.  Two launches (the global range is a true dependency).
 * Scratch as for lc_observe_tensor_f32.  minmax_out receives {min, max}. */
int32_t lc_dynamic_quantize_tensor_f32(const float* x, int64_t rows, int64_t cols, int64_t ldx,
                                       int32_t symmetric, int32_t quant_min,
                                       int32_t quant_max, int32_t is_signed, float eps,
                                       void* q_out, int32_t out_dtype, int64_t ldq,
                                       float* scale_out, float* zp_out, float* minmax_out,
                                       void* workspace, int64_t workspace_bytes, void* stream);

/* ---- int8 Linear: tcgen05 kind::i8 GEMM with fused dequant epilogue ----
 * Integer form of the dynamic Linear forward
 * (lucid/nn/quantized/dynamic/linear.py:85-92; float GEMM it replaces:
 * lucid/_C/nn/Linear.cpp:74-136 -> backend/cpu/methods/Matmul.cpp:80-122):
 *   acc[m,n] = sum_k a[m,k] * b[n,k]                         (int32, exact)
 *   acc'     = acc - zx * wsum[n]            if zx and wsum are given
 *   out      = f32(acc') * sx[m or 0] * sw[n] + bias[n]      (out_dtype F32/BF16)
 *   out      = acc'                                          (out_dtype S32)
 * a: [M,K] int8 or uint8 codes (a_unsigned), row stride lda bytes;
 * b: [N,K] int8 codes (the reference's (out,in) weight layout), row stride ldb.
 * lda and ldb must be multiples of 16 and the bases 16-byte aligned (TMA).
 * sx: one float (sx_per_row = 0) or M floats; zx: one float holding an integer
 * value, or NULL; wsum[n] = sum_k b[n,k] as int32, or NULL; sw: N floats or
 * NULL (treated as 1); bias: N floats or NULL.  ldo in elements.
 * status: optional device int32 that receives a non-zero code if a bounded
 * device-side wait ran out (the output is then invalid). */
int32_t lc_qlinear_i8(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b,
                      int64_t ldb, int64_t M, int64_t N, int64_t K, const float* sx,
                      int32_t sx_per_row, const float* zx, const int32_t* wsum,
                      const float* sw, const float* bias, void* out, int32_t out_dtype,
                      int64_t ldo, int32_t* status, void* stream);

/* lc_qlinear_i8 with an explicit kernel choice: variant 0 = automatic (what lc_qlinear_i8
 * does), 1 = single-CTA tiles (128 x 256), 2 = CTA-pair tiles (tcgen05 cta_group::2,
 * 256 x 256 per 2-CTA cluster).  Results are identical; the variants exist for testing and
 * tuning.  Same reference counterpart as lc_qlinear_i8. */
int32_t lc_qlinear_i8_ex(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b,
                         int64_t ldb, int64_t M, int64_t N, int64_t K, const float* sx,
                         int32_t sx_per_row, const float* zx, const int32_t* wsum,
                         const float* sw, const float* bias, void* out, int32_t out_dtype,
                         int64_t ldo, int32_t* status, int32_t variant, void* stream);

/* lc_qlinear_i8_ex writing every output tile to n_out (1..8) buffers of identical shape and
 * leading dimension.  host_outs is a HOST array of device pointers: the first is normally
 * this GPU's buffer, the others may be peer GPUs' buffers mapped into this process (P2P or
 * symmetric memory).  With each rank passing `buffer + rank * N` of every rank's full
 * [M, P*N] result, the column-parallel Linear and the all-gather of its output shards
 * become one kernel: tiles cross NVLink as plain stores of whole 128-byte row segments
 * while the tensor cores work on the next tile.  No counterpart in the reference (it has
 * no multi-device path). */
int32_t lc_qlinear_i8_multi(const void* a, int32_t a_unsigned, int64_t lda, const int8_t* b,
                            int64_t ldb, int64_t M, int64_t N, int64_t K, const float* sx,
                            int32_t sx_per_row, const float* zx, const int32_t* wsum,
                            const float* sw, const float* bias, void* const* host_outs,
                            int32_t n_out, int32_t out_dtype, int64_t ldo, int32_t* status,
                            int32_t variant, void* stream);

/* Bit of `variant` (lc_qlinear_i8_ex, lc_qlinear_i8_multi, lc_wo_gemm_16) that turns a launch into
 * a test of the kernels' bounded waits: the producer role issues no loads and every wait gives up
 * after a few thousand cycles, so each role records its code in `status` (required), the CTAs free
 * their TMEM and the kernel returns without having written a valid output.  Nothing traps or
 * spins without a bound; the next ordinary launch is unaffected. */
#define LC_QLINEAR_WAIT_TEST 256

/* Bit of `variant` for lc_qlinear_i8_multi with n_out == 1: host_outs[0] is a MULTICAST address of
 * the result buffer (NVLink SHARP / NVLS: one virtual address bound to the same buffer on every
 * GPU of the group).  Every output segment then leaves the GPU once, as a multimem.st, and the
 * NVSwitch writes it into every GPU's copy, this GPU's included: the all-gather of a
 * column-parallel Linear with one store per tile instead of one per peer.  fp32 output only. */
#define LC_QLINEAR_MULTICAST_OUT 512

/* Reads the device status word of the kernels above on the host: synchronises `stream`, returns
 * LC_OK when the word is 0 and LC_ERR_TIMEOUT (with the role that gave up in lc_last_error) when a
 * bounded device-side wait ran out; clear != 0 resets the word.  The reference's engine reports
 * failures as exceptions from a synchronous call (lucid/_C/ops/quantized/QuantizedMatmul.cpp:42-45);
 * this is the asynchronous counterpart. */
int32_t lc_qlinear_check_status(const int32_t* status, int32_t clear, void* stream);

/* ---- multi-GPU plumbing of the column-parallel Linear (no counterpart in the reference) ----
 * Barrier between the `world` (<= 16) ranks of one node, one rank per GPU.  host_flags is a HOST
 * array of `world` device pointers: entry r is rank r's flag array (world x uint32, zero-filled
 * once, in memory every rank can store to: peer-mapped or symmetric memory) as mapped in this
 * process.  The kernel publishes `epoch` in this rank's slot of every rank's array after a
 * system-wide fence (so that output tiles this GPU stored into its peers' buffers are visible
 * first) and waits until every rank has published an epoch >= `epoch` in this rank's array.  Use a
 * new, larger epoch for every barrier.  The wait is BOUNDED: after wait_cycles SM cycles the kernel
 * writes 4 into *status (device int32, may be NULL) and returns, so a rank that died or never
 * joined cannot hang this GPU; lc_qlinear_check_status reports it as LC_ERR_TIMEOUT. */
int32_t lc_peer_barrier(void* const* host_flags, int32_t rank, int32_t world, uint32_t epoch,
                        int64_t wait_cycles, int32_t* status, void* stream);

/* rows x width_bytes from src (row pitch src_pitch bytes) to dst (row pitch dst_pitch), device to
 * device on the copy engines (cudaMemcpy2DAsync); either side may be a peer GPU's memory mapped
 * into this process.  Moves a rank's column block of a row-major result into a peer's copy. */
int32_t lc_copy_2d_async(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                         int64_t width_bytes, int64_t rows, void* stream);

/* The whole forward of the dynamic Linear (lucid/nn/quantized/dynamic/linear.py:85-92) from ONE call:
 * dynamic activation quantization of x [M, K] fp32 (act_scheme 0: per-tensor affine, the reference's
 * default with quint8; 1: per-tensor symmetric; 2: per-row symmetric) followed by lc_qlinear_i8
 * against wq / sw / bias (wsum = row sums of wq, needed whenever the grid has a zero-point).  Codes,
 * scales and the scratch of the range kernel live in `workspace` (lc_dynamic_linear_workspace_bytes,
 * 256-byte aligned, reusable by later calls of at most the same M and K on the same stream); pass
 * workspace_is_fresh != 0 the first time a buffer is used (its scratch part is then zero-filled).
 * Results are those of the separate calls; what this saves is host time per layer. */
int64_t lc_dynamic_linear_workspace_bytes(int64_t M, int64_t K);
int32_t lc_dynamic_linear_f32(const float* x, int64_t ldx, int64_t M, int64_t K, int32_t act_scheme,
                              int32_t quant_min, int32_t quant_max, int32_t is_signed, float eps,
                              const int8_t* wq, int64_t ldw, int64_t N, const float* sw, const float* bias,
                              const int32_t* wsum, void* out, int32_t out_dtype, int64_t ldo, void* workspace,
                              int64_t workspace_bytes, int32_t workspace_is_fresh, int32_t* status, void* stream);

/* row sums of an int8 matrix as int32 (the zero-point correction term) */
int32_t lc_rowsum_s8(const int8_t* b, int64_t rows, int64_t cols, int64_t ldb, int32_t* out,
                     void* stream);

/* ---- weight-only int8 Linear for decode batch sizes --------------------
 * Per-output-channel symmetric int8 weights, float activations, fp32
 * accumulation: y[b,n] = (sum_k x[b,k] * wq[n,k]) * sw[n] + bias[n].
 * Replaces the dequantize-then-F.linear forward of the quantized Linear at
 * small batch (lucid/nn/quantized/linear.py:206-214) and is the per-channel
 * counterpart of quantized_matmul_op (lucid/_C/ops/quantized/QuantizedMatmul.cpp:143-207).
 * x_dtype / y dtype: LC_F32, LC_BF16 or LC_F16.  bf16 / f16 activations run on the tensor cores
 * (weights of 4 MB and more streamed through shared memory once); LC_F32 activations are served by plain
 * FP32 multiply-adds, one warp per output row, meant for up to four rows of a small weight -- from five
 * rows on, or for weights of tens of MB, call lc_split_f32_digits + lc_wo_gemm_digits instead (exact,
 * tensor cores: [4096, 4096] at 32 rows 20 us against 557 us), as the host layer does.
 * flags: LC_WO_OVERLAP_PREVIOUS lets the kernel start while the kernel before it on the
 * stream is still draining (programmatic dependent launch): it prefetches weights into
 * shared memory and waits for that kernel before it reads x or writes y.  The caller asserts that wq, sw and bias were completely written before that
 * previous kernel started.  Ignored by the paths that do not stream weights through
 * shared memory. */
#define LC_WO_OVERLAP_PREVIOUS 1
int32_t lc_wo_linear_s8(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                        const int8_t* wq, int64_t ldw, int64_t N, const float* sw,
                        const float* bias, void* y, int64_t ldy, int32_t flags, void* stream);

/* lc_wo_linear_s8 followed, in the same kernel, by what the statically quantized Linear applies
 * to its output (lucid/nn/quantized/linear.py:206-214; LinearReLU, lucid/nn/quantized/intrinsic.py:40):
 * y = max(y, 0) if relu, then y = (clip(rint(y * (1/S)) + Z, quant_min, quant_max) - Z) * S with
 * the calibrated S = *out_scale, Z = *out_zp (device scalars; both NULL: no requantization). */
int32_t lc_wo_linear_s8_ex(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                           const int8_t* wq, int64_t ldw, int64_t N, const float* sw, const float* bias,
                           int32_t relu, const float* out_scale, const float* out_zp, int32_t quant_min,
                           int32_t quant_max, void* y, int64_t ldy, int32_t flags, void* workspace,
                           int64_t workspace_bytes, void* stream);

/* Scratch for the _ex weight-only entry points (may be NULL).  With it, the kernel that streams large
 * weights gives every SM the same number of bytes whatever the shape: work is cut into (16-row tile,
 * 1024-byte K chunk) units, every CTA takes an equal contiguous run of them, and a tile whose K range
 * two or more CTAs share is finished by the one that arrives last (each parks its raw sums in its own
 * slot of the scratch; the sums are added in CTA order, so results do not depend on timing).  Without
 * it every CTA takes whole tiles, which leaves CTA slots idle when the tiles do not divide evenly (a
 * [4096, 14336] matrix fills 256 of the 296 slots of two CTAs per SM).  Sums over a split K range are added in a different
 * order than in one pass, so the last bits of an output may differ between the two schedules.
 * Measured on B200 the shared tiles' ticketed finish costs more than the idle SMs it removes (decode
 * MLP 53 us against 41 us), so the host layer leaves the scratch out by default.
 * lc_wo_linear_workspace_bytes(N) bytes, 16-byte aligned, zero-filled once by the caller; the kernel
 * leaves it zero.  One scratch per stream: launches that can overlap on the GPU must not share it.
 * If lc_wo_linear_status reports a wait that ran out, zero the scratch again before reusing it. */
int64_t lc_wo_linear_workspace_bytes(int64_t N);

/* Gate and up projection of a SwiGLU MLP in one pass over the weights, with the activation
 * fused: wq is [N2 = 2F, K] with rows interleaved in blocks of 8 (rows 16t..16t+7 are gate
 * rows 8t..8t+7, rows 16t+8..16t+15 the matching up rows), sw / bias interleaved the same
 * way; y[b, h] = silu(gate_h) * up_h in the activation type (bf16 / f16), F columns.
 * The unfused form in the reference is two quantized Linears followed by eager silu and
 * multiply ops (lucid/nn/quantized/linear.py:206-214; fusion listed as a follow-up of the
 * quantized_matmul path, lucid/_C/ops/quantized/QuantizedMatmul.cpp:143-207).
 * flags as for lc_wo_linear_s8; batch <= 32. */
int32_t lc_wo_swiglu_s8(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                        const int8_t* wq, int64_t ldw, int64_t N2, const float* sw, const float* bias,
                        void* y, int64_t ldy, int32_t flags, void* stream);
/* the same with scratch for the balanced schedule (see lc_wo_linear_workspace_bytes; size it for N2) */
int32_t lc_wo_swiglu_s8_ex(const void* x, int32_t x_dtype, int64_t batch, int64_t K, int64_t ldx,
                           const int8_t* wq, int64_t ldw, int64_t N2, const float* sw, const float* bias,
                           void* y, int64_t ldy, int32_t flags, void* workspace, int64_t workspace_bytes,
                           void* stream);

/* ---- weight-only Linear on the tensor cores, for more rows than a GEMV handles ----
 * The statically quantized Linear's forward, dequantize(W) -> F.linear -> (ReLU) -> fake_quantize
 * (lucid/nn/quantized/linear.py:206-214, LinearReLU in lucid/nn/quantized/intrinsic.py:40), and
 * the weight-only product of quantized_matmul_op (lucid/_C/ops/quantized/QuantizedMatmul.cpp:143-207)
 * for per-channel int8 weights, as ONE tcgen05 kind::f16 GEMM with fp32 accumulation:
 *   acc[m,n] = sum_t sum_k a_t[m,k] * w16[n,k]
 *   y        = acc * sw[n] + rowsum[m] * colcorr[n] + bias[n]      (each step one fp32 operation)
 *   y        = max(y, 0)                                           if relu
 *   out      = (clip(rint(y * (1/S)) + Z, quant_min, quant_max) - Z) * S   if out_scale / out_zp
 * a: [M, n_terms * K] bf16 (or f16 with n_terms = 1): the n_terms addends of the activation side
 * by side, row stride lda elements.  A bf16 / f16 activation is its own single term.  An fp32
 * activation is the exact sum of three bf16 terms (lc_split_f32_bf16x3), so every product is exact;
 * the tensor core however truncates when it adds into the fp32 accumulator (error 2.3e-6 of the
 * output RMS at K = 512, growing linearly with K), so fp32 activations should use
 * lc_wo_gemm_digits below, which is exact and faster.  w16: [N, K] the int8 codes widened
 * exactly to a_dtype (lc_widen_s8), row stride ldw elements; no fp32 copy of the weight is ever
 * made.  lda, ldw and K are multiples of 8; with n_terms > 1, K is a multiple of 64 (zero-padded).
 * sw: N floats or NULL; bias: N floats or NULL; rowsum [M] and colcorr [N] (= -zw[n] * sw[n], the
 * weight zero-point term) both or neither; out_scale / out_zp: device scalars of the calibrated
 * output grid, both or neither.  out_dtype: LC_F32, LC_BF16 or LC_F16, ldo in elements.
 * status, variant: as for lc_qlinear_i8_ex. */
int32_t lc_wo_gemm_16(const void* a, int32_t a_dtype, int32_t n_terms, int64_t lda, const void* w16,
                      int64_t ldw, int64_t M, int64_t N, int64_t K, const float* sw, const float* bias,
                      const float* rowsum, const float* colcorr, int32_t relu, const float* out_scale,
                      const float* out_zp, int32_t quant_min, int32_t quant_max, void* out,
                      int32_t out_dtype, int64_t ldo, int32_t* status, int32_t variant, void* stream);

/* The same Linear for fp32 activations on EXACT integer arithmetic (tcgen05 kind::i8).  Every row of
 * x is scaled by a power of two so that its largest magnitude lies in [2^29, 2^30), rounded to an
 * integer X and cut into four signed base-256 digits (lc_split_f32_digits): entries within 2^-6 of
 * the row maximum keep all 24 bits, the absolute error of smaller ones is below 2^-30 of the row
 * maximum.  The four digit planes ride through one int8 GEMM with int32 accumulation and are put
 * back together in 64-bit integers in the epilogue, so sum_k X[m,k] * wq[n,k] is exact and
 *   y = f32(sum) * row_scale[m] * sw[n] + rowsum[m] * colcorr[n] + bias[n]
 * rounds the dot product once; ReLU and requantization as for lc_wo_gemm_16.  This is what the
 * statically quantized Linear runs for more than 32 rows; it is more accurate than the fp32 GEMM of
 * the reference (lucid/_C/nn/Linear.cpp:74-136), whose accumulation rounds at every step.
 * digits: [lc_wo_digit_rows(M), K] int8, row stride ldd (multiple of 16), laid out by
 * lc_split_f32_digits; row_scale: [M]; wq: [N, K] int8 codes, ldw a multiple of 16; out: fp32.
 * K <= 131072.  status, variant: as for lc_qlinear_i8_ex. */
int64_t lc_wo_digit_rows(int64_t rows);
int32_t lc_split_f32_digits(const float* x, int64_t rows, int64_t cols, int64_t ldx, int8_t* digits,
                            int64_t ldd, float* row_scale, float* rowsum, void* stream);
int32_t lc_wo_gemm_digits(const int8_t* digits, int64_t ldd, const float* row_scale, const int8_t* wq,
                          int64_t ldw, int64_t M, int64_t N, int64_t K, const float* sw, const float* bias,
                          const float* rowsum, const float* colcorr, int32_t relu, const float* out_scale,
                          const float* out_zp, int32_t quant_min, int32_t quant_max, float* out, int64_t ldo,
                          int32_t* status, int32_t variant, void* stream);

/* int8 codes [rows, cols] (row stride ld_in) -> the same integers as bf16 or f16 (exact for every
 * code), row stride ld_out >= cols elements, columns [cols, ld_out) zero-filled.  The operand
 * layout of lc_wo_gemm_16; made once per weight (the conversion step of
 * lucid/nn/quantized/linear.py:216-235 from_float, extended by one cached copy). */
int32_t lc_widen_s8(const int8_t* q, int64_t rows, int64_t cols, int64_t ld_in, void* out, int32_t out_dtype,
                    int64_t ld_out, void* stream);

/* x fp32 [rows, cols] (row stride ldx) -> terms bf16 [rows, 3 * kp]: x1 = bf16(x), x2 = bf16(x - x1),
 * x3 = bf16(x - x1 - x2) in columns [0, kp), [kp, 2kp), [2kp, 3kp), zero-filled beyond `cols`; x1 + x2 + x3
 * == x exactly for every normal fp32 value.  kp >= cols, a multiple of 64.  rowsum (may be NULL)
 * receives sum_k x[m,k] in fp32.  The activation operand of lc_wo_gemm_16 for fp32 inputs
 * (the reference feeds fp32 activations to its float GEMM, lucid/_C/nn/Linear.cpp:74-136). */
int32_t lc_split_f32_bf16x3(const float* x, int64_t rows, int64_t cols, int64_t ldx, void* terms, int64_t kp,
                            float* rowsum, void* stream);

/* Synchronises the device and reads the status word of the weight-only kernels on the
 * current device: 0, or the code of a bounded device-side wait that ran out (the
 * affected outputs are invalid).  clear != 0 resets it.  No counterpart in the
 * reference, whose engine reports errors as exceptions (QuantizedMatmul.cpp:42-45). */
int32_t lc_wo_linear_status(int32_t* host_code, int32_t clear);

/* ---- group-wise affine weight-only format ------------------------------
 * engine.quantized.{quantize,dequantize,quantized_matmul}
 * (lucid/_C/ops/quantized/QuantizedMatmul.cpp:111-121, 123-141, 143-207):
 * per (row, group of group_size columns): s = (max-min)/(2^bits-1), bias = min,
 * code = clip(rint((w-bias)/s), 0, 2^bits-1), 32/bits codes per 32-bit word,
 * first code in the low bits.  bits in {4, 8}; group_size in {32, 64, 128}. */
int32_t lc_group_quantize_f32(const float* w, int64_t N, int64_t K, int32_t group_size,
                              int32_t bits, int32_t* packed, float* scales, float* biases,
                              void* stream);
int32_t lc_group_dequantize(const int32_t* packed, const float* scales, const float* biases,
                            int64_t N, int64_t K, int32_t group_size, int32_t bits, float* out,
                            void* stream);
/* y[b,n] = sum_k x[b,k] * (code[n,k]*s[n,g] + bias[n,g]); x and y of x_dtype */
int32_t lc_group_matmul(const void* x, int32_t x_dtype, int64_t batch, int64_t K,
                        const int32_t* packed, const float* scales, const float* biases,
                        int64_t N, int32_t group_size, int32_t bits, void* y, void* stream);
/* lc_group_matmul with the flags and scratch of the weight-streaming kernel (LC_WO_OVERLAP_PREVIOUS;
 * lc_wo_linear_workspace_bytes(N), may be NULL).  Packed weights of 4 MB and more (smaller ones from five
 * rows on) -- 8-bit or 4-bit codes in groups of 64 or 128, K a multiple of four groups -- with bf16 / f16
 * activations are streamed through
 * shared memory once, like per-channel int8 weights (the packed words are the codes in K order, first
 * code in the low bits); every other case runs the direct kernel. */
/* flag of lc_group_matmul_ex: x is LC_BF16 and y receives fp32 (row pitch N floats).  For fp32 activations on
 * the streaming kernel: lc_split_f32_bf16x3 writes every fp32 row as three bf16 rows that add up to it exactly,
 * this call multiplies the 3 * batch rows, and the caller adds each row's three results.  Refused
 * (LC_ERR_UNSUPPORTED) where the streaming kernel does not apply. */
#define LC_GROUP_OUT_F32 2
int32_t lc_group_matmul_ex(const void* x, int32_t x_dtype, int64_t batch, int64_t K,
                           const int32_t* packed, const float* scales, const float* biases,
                           int64_t N, int32_t group_size, int32_t bits, void* y, int32_t flags,
                           void* workspace, int64_t workspace_bytes, void* stream);

/* ---- int8 embedding tables ---------------------------------------------
 * Forward of the quantized Embedding (lucid/nn/quantized/sparse.py:140-143): the reference
 * dequantizes the whole [V, D] table per call (lucid/quantization/_functional.py:281-293) and
 * gathers from the fp32 copy (F.embedding, lucid/nn/functional/sparse.py:70); here
 * out[i, :] = (f32(table[indices[i], :]) - zero_point[indices[i]]) * scale[indices[i]] for the
 * looked-up rows only.  zero_point may be NULL (symmetric table).  An index outside
 * [0, num_embeddings) yields a row of zeros and sets *status to 1 (status: device int32,
 * cleared by the caller, may be NULL); the reference refuses such an index on the host
 * (lucid/_C/backend/cpu/IndexBounds.h:89-93), which would need a device-to-host read here. */
int32_t lc_embedding_s8_f32(const int8_t* table, const float* scale, const float* zero_point,
                            const int64_t* indices, int64_t n, int64_t num_embeddings,
                            int64_t embedding_dim, float* out, int32_t* status, void* stream);

/* Forward of the quantized EmbeddingBag (lucid/nn/quantized/sparse.py:284-304) with the pooling
 * of lucid/_C/backend/cpu/methods/Sequence.cpp:44-85: bag b covers indices[offsets[b] ..
 * offsets[b+1]) (the last one runs to n unless include_last_offset, in which case offsets has
 * one entry more than there are bags); entries equal to padding_idx (>= 0) are skipped; rows are
 * decoded as above and added in index order starting from zero (mode 0), divided by the number
 * of entries kept (mode 1), or reduced with max starting from the lowest float (mode 2); an
 * empty bag gives zeros.  per_sample_weights (mode 0 only, may be NULL) multiplies each decoded
 * row before it is added.  out: [bags, embedding_dim] fp32. */
int32_t lc_embedding_bag_s8_f32(const int8_t* table, const float* scale, const float* zero_point,
                                const int64_t* indices, int64_t n, const int64_t* offsets,
                                int64_t n_offsets, const float* per_sample_weights,
                                int64_t num_embeddings, int64_t embedding_dim, int32_t mode,
                                int64_t padding_idx, int32_t include_last_offset, float* out,
                                int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LUCID_CUDA_H_ */
