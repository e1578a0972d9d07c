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


class Int8WeightCache:
    """GEMM-ready views of a layer's int8 weight, rebuilt when the buffer changes:
    a copy whose rows start on 16-byte boundaries (what TMA needs; the buffer itself
    when ``in_features`` is already a multiple of 16) and the int32 row sums used by
    the zero-point correction ``acc - zx * sum_k w[n,k]``."""

    def __init__(self) -> None:
        self._key = None
        self.codes = None
        self.rowsum = None

    def get(self, weight_int8: torch.Tensor):
        key = (weight_int8.data_ptr(), weight_int8._version, weight_int8.device, tuple(weight_int8.shape))
        if key != self._key:
            self.codes = _backend.ops().pad_rows_to_16(weight_int8)
            self.rowsum = _backend.ops().rowsum_s8(self.codes)
            self._key = key
        return self.codes, self.rowsum
