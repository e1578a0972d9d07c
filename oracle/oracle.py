"""CPU oracle for the int8 quantized-inference path (TEST INFRASTRUCTURE ONLY).

This file restates, on NumPy, the arithmetic the reference framework performs
for ``lucid.quantization`` quantize / dequantize / fake_quantize, its range
observers, ``calculate_qparams`` and the three quantized ``Linear`` forwards.
It is the checker the CUDA kernels are compared against and the CPU baseline
``bench.py`` times; nothing in the shipped package imports it.

Every float step is rounded to fp32 on its own, as the reference does by
running one eager fp32 op per step (no FMA contraction, no double
intermediates).  ``np.rint`` is round-half-to-even, which is what the
reference's CPU ``round`` does (``lucid/_C/backend/cpu/Vforce.cpp:314``).

Pinning: the reference engine cannot be built or imported on Linux (it links
Apple Accelerate and a binary MLX wheel, ``setup.py:23-31``), so the oracle is
pinned against the known-answer tests of the reference's own test-suite
(``lucid/test/unit/quantization/test_functional.py``, ``test_observer.py``)
and against ``torch.quantize_per_tensor``, which the reference's parity test
declares array-equal to its ``quantize``
(``lucid/test/parity/quantization/test_functional_parity.py:20-26``).  See
``tests/test_oracle_golden.py``.  The group-wise weight-only functions follow
only the formulas the reference documents (``lucid/quantization/_qgemm.py:84-97``);
their bit-level behaviour lives inside MLX 0.32.3 and is **parity unpinned**.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# quantized dtypes (lucid/quantization/_qscheme.py:131-245)
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class QDtype:
    name: str
    bits: int
    signed: bool
    quant_min: int
    quant_max: int
    storage: str


qint8 = QDtype("qint8", 8, True, -128, 127, "int8")
quint8 = QDtype("quint8", 8, False, 0, 255, "int16")
qint32 = QDtype("qint32", 32, True, -(2**31), 2**31 - 1, "int32")
qint4 = QDtype("qint4", 4, True, -8, 7, "int8")
# narrow-range signed int8: scale = absmax / 127, clamp [-127, 127]
qint8_narrow = QDtype("qint8", 8, True, -127, 127, "int8")


def _f32(a) -> np.ndarray:
    return np.asarray(a, dtype=F32)


# --------------------------------------------------------------------------
# calculate_qparams (lucid/quantization/_qparams.py:93-205)
# --------------------------------------------------------------------------
def calculate_qparams(min_val, max_val, symmetric: bool, qdtype: QDtype, eps: float = 1e-8):
    """Scale / zero-point from an observed range; fp32 per step.

    Follows ``_qparams.py:186-205``: the range is widened to include 0, the
    symmetric scale is ``max(|min|,|max|) / ((qmax-qmin)/2.0)`` floored at
    ``eps`` and the affine zero-point uses a true division ``min / scale``.
    """
    mn = np.minimum(_f32(min_val), F32(0.0))
    mx = np.maximum(_f32(max_val), F32(0.0))
    eps_t = F32(eps)
    qmin, qmax = qdtype.quant_min, qdtype.quant_max
    if symmetric:
        max_abs = np.maximum(np.abs(mn), np.abs(mx))
        half = F32((qmax - qmin) / 2.0)
        scale = np.maximum((max_abs / half).astype(F32), eps_t)
        if qdtype.signed:
            zp = np.zeros_like(scale)
        else:
            zp = np.full_like(scale, float((qmax + qmin + 1) // 2))
    else:
        span = (mx - mn).astype(F32)
        scale = np.maximum((span / F32(qmax - qmin)).astype(F32), eps_t)
        r = np.rint((mn / scale).astype(F32)).astype(F32)
        zp = np.clip((F32(qmin) - r).astype(F32), F32(qmin), F32(qmax))
    return scale.astype(F32), zp.astype(F32)


# --------------------------------------------------------------------------
# observers (lucid/quantization/observer.py:408-418, 672-689)
# --------------------------------------------------------------------------
def minmax_tensor(x: np.ndarray):
    """Global min and max: two separate full passes, like ``x.min(); x.max()``."""
    x = _f32(x)
    return F32(x.min()), F32(x.max())


def minmax_channel(x: np.ndarray, ch_axis: int = 0):
    """Per-channel min/max: ``moveaxis(ch->0).reshape(C,-1)`` then amin/amax."""
    x = _f32(x)
    flat = np.moveaxis(x, ch_axis, 0).reshape(x.shape[ch_axis], -1)
    return flat.min(axis=1).astype(F32), flat.max(axis=1).astype(F32)


class MinMaxObserver:
    """Running range, seeded +inf/-inf (``observer.py:405-414``)."""

    def __init__(self, symmetric: bool = False, qdtype: QDtype = quint8, ch_axis: int | None = None):
        self.symmetric, self.qdtype, self.ch_axis = symmetric, qdtype, ch_axis
        self.min_val = F32(np.inf)
        self.max_val = F32(-np.inf)

    def __call__(self, x):
        if self.ch_axis is None:
            mn, mx = minmax_tensor(x)
        else:
            mn, mx = minmax_channel(x, self.ch_axis)
        self.min_val = np.minimum(self.min_val, mn)
        self.max_val = np.maximum(self.max_val, mx)
        return x

    def calculate_qparams(self):
        return calculate_qparams(self.min_val, self.max_val, self.symmetric, self.qdtype)


# --------------------------------------------------------------------------
# quantize / dequantize / fake_quantize (lucid/quantization/_functional.py)
# --------------------------------------------------------------------------
def _bcast(p, ch_axis, ndim):
    """``_reshape_for_channel`` (``_functional.py:47-56``)."""
    if ch_axis is None or np.ndim(p) == 0:
        return p
    shape = [1] * ndim
    shape[ch_axis] = -1
    return np.reshape(p, shape)


def _reciprocal(scale):
    """``1.0 / s``: fp32 IEEE division for an array scale, a double division
    rounded once to fp32 for a Python-float scale (``_dispatch.py:154-170``)."""
    if isinstance(scale, (float, int)):
        return F32(1.0 / float(scale))
    return (F32(1.0) / _f32(scale)).astype(F32)


def grid_code(x, scale, zero_point, ch_axis=None):
    """``round(x * (1/s)) + z`` (``_functional.py:59-69``), unclamped, fp32."""
    x = _f32(x)
    inv = _bcast(_reciprocal(scale), ch_axis, x.ndim)
    z = _bcast(_f32(zero_point), ch_axis, x.ndim)
    t = (x * inv).astype(F32)
    return (np.rint(t).astype(F32) + z).astype(F32)


def saturating_cast(codes: np.ndarray, storage: str) -> np.ndarray:
    """float -> int cast that saturates and maps NaN to 0
    (``lucid/_C/backend/cpu/methods/Factory.cpp:103-135``)."""
    info = np.iinfo(storage)
    c = np.where(np.isnan(codes), 0.0, np.asarray(codes, dtype=np.float64))
    c = np.clip(c, float(info.min), float(info.max))
    return np.trunc(c).astype(storage)


def quantize(x, scale, zero_point, qdtype: QDtype, ch_axis=None) -> np.ndarray:
    """``clip(round(x*(1/s))+z, qmin, qmax)`` cast to the storage dtype
    (``_functional.py:179-197``)."""
    code = grid_code(x, scale, zero_point, ch_axis)
    code = np.clip(code, F32(qdtype.quant_min), F32(qdtype.quant_max))
    return saturating_cast(code, qdtype.storage)


def dequantize(q, scale, zero_point, ch_axis=None) -> np.ndarray:
    """``(f32(q) - z) * s`` (``_functional.py:281-293``); always fp32."""
    q = np.asarray(q)
    s = _bcast(_f32(scale), ch_axis, q.ndim)
    z = _bcast(_f32(zero_point), ch_axis, q.ndim)
    return ((q.astype(F32) - z).astype(F32) * s).astype(F32)


def fake_quantize(x, scale, zero_point, quant_min: int, quant_max: int, ch_axis=None):
    """Forward of ``_FakeQuantizeAffine`` (``_functional.py:304-333``).

    Returns ``(dq, mask)``; ``mask`` is the straight-through-estimator mask
    (1 where the unclamped code is inside the grid).
    """
    x = _f32(x)
    pre = grid_code(x, scale, zero_point, ch_axis)
    q = np.clip(pre, F32(quant_min), F32(quant_max))
    s = _bcast(_f32(scale), ch_axis, x.ndim)
    z = _bcast(_f32(zero_point), ch_axis, x.ndim)
    dq = ((q - z).astype(F32) * s).astype(F32)
    mask = ((pre >= quant_min) & (pre <= quant_max)).astype(F32)
    return dq, mask


# --------------------------------------------------------------------------
# exact integer GEMM (lucid/_C/backend/cpu/methods/Matmul.cpp:8-20: the
# reference's CPU integer matmul is carried exactly through f64)
# --------------------------------------------------------------------------
def int_gemm_exact(aq: np.ndarray, bq: np.ndarray) -> np.ndarray:
    """``aq[M,K] @ bq[N,K]^T`` with exact int32 accumulation.

    |acc| <= 255*128*K stays far below 2**53 for any K this path accepts, so
    a float64 BLAS product is exact."""
    acc = np.asarray(aq, dtype=np.float64) @ np.asarray(bq, dtype=np.float64).T
    return acc.astype(np.int64).astype(np.int32)


# --------------------------------------------------------------------------
# quantized Linear forwards
# --------------------------------------------------------------------------
def quantize_weight_per_channel(w, qdtype: QDtype = qint8):
    """``nnqd.Linear.from_float`` (``nn/quantized/dynamic/linear.py:94-109``):
    per-output-row symmetric observer, then quantize with ``ch_axis=0``."""
    mn, mx = minmax_channel(w, 0)
    s, z = calculate_qparams(mn, mx, True, qdtype)
    return quantize(w, s, z, qdtype, ch_axis=0), s, z


def linear_f32(x, w, b=None):
    """``F.linear``: ``sgemm(x, w^T)`` then the bias loop
    (``lucid/_C/backend/cpu/methods/Matmul.cpp:80-122``)."""
    y = (_f32(x) @ _f32(w).T).astype(F32)
    if b is not None:
        y = (y + _f32(b)).astype(F32)
    return y


def dynamic_linear_reference(x, wq, sw, zw, bias, act_qdtype: QDtype = quint8):
    """The reference's dynamic Linear forward, float formulation
    (``nn/quantized/dynamic/linear.py:85-92``): per-tensor AFFINE fake-quant
    of ``x``, per-forward weight dequantize, fp32 GEMM + bias."""
    mn, mx = minmax_tensor(x)
    sx, zx = calculate_qparams(mn, mx, False, act_qdtype)
    xq, _ = fake_quantize(x, sx, zx, act_qdtype.quant_min, act_qdtype.quant_max)
    w = dequantize(wq, sw, zw, ch_axis=0)
    return linear_f32(xq, w, bias)


def dynamic_linear_float(x, wq, sw, zw, bias, mode: str = "tensor_affine", act_qdtype: QDtype = quint8):
    """The reference's float formulation with a selectable activation grid: the op
    sequence of ``dynamic/linear.py:85-92`` (fake-quantize ``x``, dequantize the whole
    weight, fp32 GEMM + bias) with per-tensor or per-row (per-token) activation qparams.
    This is what the CPU baseline times."""
    x2 = _f32(x).reshape(-1, np.shape(x)[-1])
    sx, zx = dynamic_act_qparams(x2, mode, act_qdtype)
    ch = 0 if mode == "token_symmetric" else None
    xq, _ = fake_quantize(x2, sx, zx, act_qdtype.quant_min, act_qdtype.quant_max, ch_axis=ch)
    w = dequantize(wq, sw, zw, ch_axis=0)
    return linear_f32(xq, w, bias)


def dynamic_act_qparams(x, mode: str, qdtype: QDtype):
    """Activation qparams for the integer formulation.

    ``mode``: ``"tensor_affine"`` (reference default, ``dynamic/linear.py:87``),
    ``"tensor_symmetric"`` or ``"token_symmetric"`` (one scale per row).
    """
    x = _f32(x)
    if mode == "tensor_affine":
        mn, mx = minmax_tensor(x)
        return calculate_qparams(mn, mx, False, qdtype)
    if mode == "tensor_symmetric":
        mn, mx = minmax_tensor(x)
        return calculate_qparams(mn, mx, True, qdtype)
    if mode == "token_symmetric":
        x2 = x.reshape(-1, x.shape[-1])
        mn, mx = minmax_channel(x2, 0)
        return calculate_qparams(mn, mx, True, qdtype)
    raise ValueError(mode)


def dynamic_linear_int(x, wq, sw, bias, mode: str = "tensor_affine", act_qdtype: QDtype = quint8, rows=None):
    """Integer formulation the CUDA path computes.

    ``acc[m,n] = sum_k (xq[m,k]-zx) * wq[n,k]`` exactly in int32, then
    ``y = f32(acc) * sx * sw[n] + b[n]`` evaluated in float64 and rounded once
    (the fp32 kernel result must be within rtol 1e-5 of this).  Returns
    ``(acc, y, xq, sx, zx)``.  ``rows`` (an index array) restricts the product to those
    rows of ``x``: the activation qparams still come from the whole tensor, ``xq`` and a
    per-row ``sx`` are returned whole, ``acc`` and ``y`` have ``len(rows)`` rows.
    """
    x2 = _f32(x).reshape(-1, np.shape(x)[-1])
    sx, zx = dynamic_act_qparams(x2, mode, act_qdtype)
    ch = 0 if mode == "token_symmetric" else None
    xq = quantize(x2, sx, zx, act_qdtype, ch_axis=ch)
    sel = slice(None) if rows is None else np.asarray(rows, dtype=np.int64)
    xi = xq[sel].astype(np.int64) - (zx.astype(np.int64).reshape(-1, 1)[sel] if ch == 0 else int(zx))
    acc = (xi.astype(np.float64) @ np.asarray(wq, dtype=np.float64).T).astype(np.int64).astype(np.int32)
    sx64 = sx.astype(np.float64).reshape(-1, 1)[sel] if ch == 0 else float(sx)
    y = acc.astype(np.float64) * sx64 * _f32(sw).astype(np.float64)[None, :]
    if bias is not None:
        y = y + _f32(bias).astype(np.float64)[None, :]
    return acc, y.astype(F32), xq, sx, zx


def static_linear_reference(x, wq, sw, zw, bias, out_scale, out_zp, out_qdtype: QDtype = quint8, relu: bool = False,
                            ch_axis: int = 0):
    """Static PTQ Linear forward (``nn/quantized/linear.py:206-214``):
    dequantize W, fp32 linear, fake-quantize the output onto the calibrated grid;
    ``relu`` inserts the activation of the fused ``LinearReLU`` (``nn/quantized/intrinsic.py:40``)
    between the linear and the fake-quantize."""
    w = dequantize(wq, sw, zw, ch_axis=None if np.ndim(sw) == 0 or np.size(sw) == 1 else ch_axis)
    y = linear_f32(x, w, bias)
    if relu:
        y = np.where(y < 0, F32(0), y).astype(F32)
    return fake_quantize(y, out_scale, out_zp, out_qdtype.quant_min, out_qdtype.quant_max)[0]


def weight_only_linear_perchannel(x, wq, sw, bias=None):
    """Weight-only per-channel int8 Linear with float activations:
    ``y = (x . wq^T) * sw + b`` evaluated in float64 (tolerance oracle)."""
    x64 = np.asarray(x, dtype=np.float64)
    y = (x64 @ np.asarray(wq, dtype=np.float64).T) * _f32(sw).astype(np.float64)[None, :]
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)[None, :]
    return y


# --------------------------------------------------------------------------
# group-wise affine weight-only format (documented formula only; parity
# unpinned: lucid/quantization/_qgemm.py:84-97,167-175,249-252)
# --------------------------------------------------------------------------
def group_quantize(w, group_size: int = 64, bits: int = 8):
    """Per (row, group of ``group_size`` input columns):
    ``s=(max-min)/(2^b-1)``, ``bias=min``, ``c=clip(round((w-bias)/s),0,2^b-1)``,
    ``32/bits`` codes per uint32 word, first code in the low bits (an
    assumption of this build; the reference leaves the order to MLX).
    A constant group gets ``s = 1`` replaced for the division only so that its
    codes are 0 and it decodes to ``bias`` exactly."""
    w = _f32(w)
    n, k = w.shape
    g = k // group_size
    wg = w.reshape(n, g, group_size)
    mn = wg.min(axis=2).astype(F32)
    mx = wg.max(axis=2).astype(F32)
    levels = F32(2**bits - 1)
    scale = ((mx - mn).astype(F32) / levels).astype(F32)
    safe = np.where(scale > 0, scale, F32(1.0)).astype(F32)
    t = ((wg - mn[:, :, None]).astype(F32) / safe[:, :, None]).astype(F32)
    codes = np.clip(np.rint(t), 0, float(levels)).astype(np.uint32).reshape(n, k)
    per = 32 // bits
    packed = np.zeros((n, k // per), dtype=np.uint32)
    for j in range(per):
        packed |= codes[:, j::per] << np.uint32(bits * j)
    return packed.view(np.int32), scale, mn


def group_unpack(packed, bits: int) -> np.ndarray:
    p = np.asarray(packed).view(np.uint32)
    per = 32 // bits
    n, words = p.shape
    codes = np.empty((n, words * per), dtype=np.uint32)
    mask = np.uint32(2**bits - 1)
    for j in range(per):
        codes[:, j::per] = (p >> np.uint32(bits * j)) & mask
    return codes


def group_dequantize(packed, scales, biases, group_size: int = 64, bits: int = 8) -> np.ndarray:
    """``w_hat = c * s + bias`` per group, fp32, rounded per step."""
    codes = group_unpack(packed, bits).astype(F32)
    n, k = codes.shape
    s = np.repeat(_f32(scales), group_size, axis=1)
    b = np.repeat(_f32(biases), group_size, axis=1)
    return ((codes * s).astype(F32) + b).astype(F32)


def group_matmul(x, packed, scales, biases, group_size: int = 64, bits: int = 8) -> np.ndarray:
    """``y = x . w_hat^T`` in float64 (tolerance oracle, transpose=True form)."""
    w = group_dequantize(packed, scales, biases, group_size, bits).astype(np.float64)
    return np.asarray(x, dtype=np.float64) @ w.T


# --------------------------------------------------------------------------
# int8 embedding tables (lucid/nn/quantized/sparse.py)
# --------------------------------------------------------------------------
def embedding_s8(table, scale, zero_point, indices) -> np.ndarray:
    """Quantized ``Embedding.forward`` (lucid/nn/quantized/sparse.py:140-143): dequantize the
    whole table per row (``ch_axis=0``), then gather the rows ``indices`` names."""
    w = dequantize(np.asarray(table), scale, zero_point, ch_axis=0)
    idx = np.asarray(indices, dtype=np.int64)
    if idx.size and (idx.min() < 0 or idx.max() >= w.shape[0]):
        raise IndexError("embedding: index out of range")
    return w[idx]


def embedding_bag_s8(table, scale, zero_point, indices, offsets, mode: str = "mean", padding_idx=None,
                     per_sample_weights=None, include_last_offset: bool = False) -> np.ndarray:
    """Quantized ``EmbeddingBag.forward`` (lucid/nn/quantized/sparse.py:284-304) with the CPU
    pooling loop of lucid/_C/backend/cpu/methods/Sequence.cpp:44-85: fp32 accumulation in index
    order from zero, ``padding_idx`` entries skipped, mean over the entries kept, max seeded with
    the lowest float, an empty bag gives zeros.  ``per_sample_weights`` (sum only) scales each
    looked-up row before it is added."""
    w = dequantize(np.asarray(table), scale, zero_point, ch_axis=0)
    idx = np.asarray(indices, dtype=np.int64).ravel()
    off = np.asarray(offsets, dtype=np.int64).ravel()
    bags = off.size - 1 if include_last_offset else off.size
    out = np.zeros((max(bags, 0), w.shape[1]), dtype=np.float32)
    psw = None if per_sample_weights is None else _f32(per_sample_weights).ravel()
    for b in range(bags):
        start = int(off[b])
        end = int(off[b + 1]) if (b + 1 < bags or include_last_offset) else idx.size
        acc = np.full(w.shape[1], np.finfo(np.float32).min if mode == "max" else 0, dtype=np.float32)
        count = 0
        for k in range(start, end):
            row = int(idx[k])
            if padding_idx is not None and padding_idx >= 0 and row == padding_idx:
                continue
            if row < 0 or row >= w.shape[0]:
                raise IndexError("embedding_bag: index out of range")
            v = w[row] if psw is None else (w[row] * psw[k]).astype(np.float32)
            acc = np.where(v > acc, v, acc) if mode == "max" else (acc + v).astype(np.float32)
            count += 1
        if mode == "max" and count == 0:
            acc[:] = 0
        if mode == "mean" and count > 0:
            acc = (acc / np.float32(count)).astype(np.float32)
        out[b] = acc
    return out


# --------------------------------------------------------------------------
# lucid.histc
# --------------------------------------------------------------------------
def histc(x, bins: int = 100, lo: float = 0.0, hi: float = 0.0) -> np.ndarray:
    """Counts of ``x`` in ``bins`` equal-width bins over ``[lo, hi]``, in ``x``'s dtype.

    Range handling of the Python adapter (lucid/_ops/_adapters.py:1256-1279): ``lo == hi``
    takes the range from the data, a range that is still one point widens to
    ``[v - 1, v + 1]``, a non-finite range is refused, NaN is sent below the range.
    Bucketing of the CPU kernel (lucid/_C/backend/cpu/methods/Reduction.cpp:839-888) in
    float64: ``step = (hi - lo) / bins``, values outside ``[lo, hi]`` are skipped,
    ``bin = trunc((v - lo) / step)`` with the right edge clamped into the last bin; counts
    are cast to the input dtype once (lucid/_C/ops/composite/Stats.cpp:78-89)."""
    x = np.asarray(x)
    lo, hi = float(lo), float(hi)
    if lo > hi:
        raise ValueError(f"histc: max must be at least min, got [{lo}, {hi}]")
    if lo == hi and x.size:
        lo, hi = float(x.min()), float(x.max())
    if not (np.isfinite(lo) and np.isfinite(hi)):
        raise ValueError(f"histc: range of [{lo}, {hi}] is not finite")
    if lo == hi:
        lo, hi = lo - 1.0, hi + 1.0
    v = x.astype(np.float64).ravel()
    v = np.where(np.isnan(v), -np.inf, v)
    step = (hi - lo) / float(bins)
    v = v[(v >= lo) & (v <= hi)]
    b = np.minimum(((v - lo) / step).astype(np.int64), bins - 1)
    return np.bincount(b, minlength=bins).astype(np.float64).astype(x.dtype if x.dtype.kind == "f" else np.float32)


# --------------------------------------------------------------------------
# seeded synthetic workloads (shapes and value distributions of the five
# benchmark configurations)
# --------------------------------------------------------------------------
def synth_config1(seed: int = 20260921):
    r = np.random.default_rng(seed)
    x = r.standard_normal((64, 1024), dtype=F32)
    w = (r.standard_normal((4096, 1024), dtype=F32) * F32(0.02)).astype(F32)
    b = (r.standard_normal(4096, dtype=F32) * F32(0.01)).astype(F32)
    return x, w, b


def synth_outlier_matrix(rows: int, cols: int, seed: int = 20260922):
    """N(0,1) with 0.1 % of the elements multiplied by 50."""
    r = np.random.default_rng(seed)
    x = r.standard_normal((rows, cols), dtype=F32)
    n_out = max(1, (rows * cols) // 1000)
    idx = r.integers(0, rows * cols, size=n_out)
    x.reshape(-1)[idx] *= F32(50.0)
    return x
