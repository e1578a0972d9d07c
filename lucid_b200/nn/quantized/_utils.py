"""Helpers shared by the quantized Linear layers: weight quantization at conversion
time (``lucid/nn/quantized/_utils.py:48-100``) and the int8 operand cache."""
from __future__ import annotations

import warnings

import torch

from lucid_b200 import _backend
from lucid_b200.quantization._functional import quantize


def quantize_weight(mod):
    """``(codes, scale, zero_point, ch_axis)`` of ``mod.weight`` using the module's QAT
    fake-quantizer if it has one, else a fresh weight observer from ``mod.qconfig``."""
    weight = _backend.on_cuda(mod.weight.detach())
    wfq = getattr(mod, "weight_fake_quant", None)
    if wfq is not None:
        wfq(weight)
        scale, zero_point = wfq.calculate_qparams()
        qdtype, ch_axis = wfq.qdtype, wfq.ch_axis
    else:
        obs = mod.qconfig.weight()
        obs(weight)
        scale, zero_point = obs.calculate_qparams()
        qdtype, ch_axis = obs.qdtype, obs.ch_axis
    codes = quantize(weight, scale, zero_point, qdtype, ch_axis=ch_axis)
    return codes, scale, zero_point, (ch_axis if ch_axis is not None else 0)


def activation_qparams(mod):
    """``(scale, zero_point, qdtype)`` of the calibrated output observer; warns when it
    never saw data (the quantized output would collapse onto a near-zero grid)."""
    obs = mod.activation_post_process
    min_val = getattr(obs, "min_val", None)
    if min_val is not None and bool(torch.isinf(min_val).any()):
        warnings.warn(
            f"Quantizing {type(mod).__name__} whose activation observer never saw data — run "
            "calibration through the prepared model before convert(), or the quantized output "
            "collapses to a near-zero grid.",
            stacklevel=3,
        )
    scale, zero_point = obs.calculate_qparams()
    return _backend.on_cuda(scale), _backend.on_cuda(zero_point), obs.qdtype


def ieee_fp32():
    """Context for a float library call (convolution, recurrent layer) that must compute in IEEE
    fp32 as the reference does: by default the CUDA library runs them on TF32 tensor cores
    (10-bit mantissa), which moves results across grid steps of a following requantization."""
    cudnn = torch.backends.cudnn
    return cudnn.flags(enabled=cudnn.enabled, benchmark=cudnn.benchmark, deterministic=cudnn.deterministic,
                       allow_tf32=False)


def wire_inner(mod):
    """The weighted layer carrying the qparams: a fused float module is a ``Sequential`` whose
    observer sits after the pair, so its qconfig and observer replace whatever ``mod[0]``
    carries (``lucid/nn/quantized/intrinsic.py:23-37``); any other module is returned as is."""
    if not isinstance(mod, torch.nn.Sequential):
        return mod
    inner = mod[0]
    inner.qconfig = mod.qconfig
    inner.activation_post_process = mod.activation_post_process
    return inner


class StaticWeightCache:
    """Launch-ready views of a statically quantized layer's weight buffers, rebuilt when one of
    them changes (new storage or in-place version): the scale as one value per output row, the
    zero-point term of the epilogue (``None`` for the usual symmetric weights; the one
    device-to-host read that decides this happens here, once per weight, never in a forward), and
    -- made on first use by a batch too large for the GEMV kernel -- the codes with rows on
    16-byte boundaries (the buffer itself when ``in_features`` is a multiple of 16)."""

    def __init__(self) -> None:
        self._key = None
        self._codes16 = None

    def get(self, codes: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, ch_axis: int):
        key = tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in (codes, scale, zero_point)) + (ch_axis,)
        if key != self._key:
            n, k = codes.shape
            scale = scale.reshape(-1).float()
            zero_point = zero_point.reshape(-1).float()
            self.col_scale = self.col_zp = None
            if scale.numel() == 1 or (ch_axis == 0 and scale.numel() == n):
                self.row_scale = scale.expand(n).contiguous()
                zp = zero_point.expand(n) if zero_point.numel() in (1, n) else None
                if zp is None:
                    raise ValueError("weight_zero_point does not match weight_scale")
                self.colcorr = (-(zp * self.row_scale)).contiguous() if bool((zp != 0).any()) else None
            elif ch_axis == 1 and scale.numel() == k:
                # per input column: the scale moves onto the activations, x' = x * s[k], and the
                # zero-point term becomes one value per row, sum_k x'[m,k] * z[k], subtracted from every column
                self.row_scale = None
                self.col_scale = scale.contiguous()
                self.col_zp = zero_point.expand(k).contiguous() if bool((zero_point != 0).any()) else None
                self.colcorr = None if self.col_zp is None else torch.full((n,), -1.0, device=codes.device)
            else:
                raise ValueError(f"weight_scale of {scale.numel()} entries does not fit a [{n}, {k}] weight "
                                 f"quantized along axis {ch_axis}")
            self.gemv_ok = self.col_scale is None and self.colcorr is None
            self._codes16 = None
            self._key = key
        return self

    def codes16(self, codes: torch.Tensor) -> torch.Tensor:
        if self._codes16 is None:
            self._codes16 = _backend.ops().pad_rows_to_16(codes)
        return self._codes16


class Int8WeightCache:
    """GEMM-ready views of a layer's int8 weight, rebuilt when the buffer changes:
    a copy whose rows start on 16-byte boundaries (what TMA needs; the buffer itself
    when ``in_features`` is already a multiple of 16) and the int32 row sums used by
    the zero-point correction ``acc - zx * sum_k w[n,k]``."""

    def __init__(self) -> None:
        self._key = None
        self.codes = None
        self.rowsum = None

    def get(self, weight_int8: torch.Tensor, weight_zero_point: torch.Tensor | None = None):
        key = (weight_int8.data_ptr(), weight_int8._version, weight_int8.device, tuple(weight_int8.shape),
               None if weight_zero_point is None else (weight_zero_point.data_ptr(), weight_zero_point._version))
        if key != self._key:
            # checked when the operand views are (re)built, never in an ordinary forward: the integer
            # GEMM computes sum_k xq * wq, which equals the reference's (q - z_w) * s_w form only for
            # symmetric weights (what from_float produces)
            if weight_zero_point is not None and bool((weight_zero_point != 0).any()):
                raise NotImplementedError(
                    "dynamic Linear: weight_zero_point is not all zero (weights quantized on an affine grid); "
                    "the int8 GEMM path takes symmetric per-row weights only -- re-quantize the float weights with "
                    "a symmetric weight observer (nnqd.Linear.from_float does)")
            self.codes = _backend.ops().pad_rows_to_16(weight_int8)
            self.rowsum = _backend.ops().rowsum_s8(self.codes)
            self._key = key
        return self.codes, self.rowsum
