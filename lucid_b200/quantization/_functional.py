"""``quantize`` / ``dequantize`` / ``fake_quantize``
(API of ``lucid/quantization/_functional.py:72-463``).

One fused kernel each instead of the reference's 4-11 eager ops; the arithmetic
per element is the same sequence of fp32 roundings: ``round(x * (1/s)) + z``,
clip, cast; ``(q - z) * s``.  Inputs on the CPU are moved to the current CUDA
device and results are returned on the input's device.
"""
from __future__ import annotations

import torch

from lucid_b200 import _backend
from lucid_b200.quantization._qscheme import QDtype

_STORAGE = {"int8": torch.int8, "int16": torch.int16, "int32": torch.int32, "uint8": torch.uint8}


def _norm_axis(ch_axis, scale):
    """A channel axis only matters when the scale really is per-channel."""
    if ch_axis is None or not isinstance(scale, torch.Tensor) or scale.numel() <= 1:
        return None
    return ch_axis


def _back(result: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return result if like.is_cuda else result.to(like.device)


def quantize(x, scale, zero_point, qdtype: QDtype, ch_axis: int | None = None):
    """Integer codes ``clip(round(x/s) + z, qmin, qmax)`` in ``qdtype.storage``."""
    xd = _backend.on_cuda(x)
    q = _backend.ops().quantize(xd, scale, zero_point, qdtype.quant_min, qdtype.quant_max, _STORAGE[qdtype.storage],
                       _norm_axis(ch_axis, scale))
    return _back(q, x)


def dequantize(q, scale, zero_point, ch_axis: int | None = None):
    """``(q - z) * s`` as float32."""
    qd = _backend.on_cuda(q)
    return _back(_backend.ops().dequantize(qd, scale, zero_point, _norm_axis(ch_axis, scale)), q)


class _FakeQuantizeAffine(torch.autograd.Function):
    """Forward: encode + decode in one kernel.  Backward: straight-through, the
    gradient passes where the unclamped code lies inside ``[quant_min, quant_max]``."""

    @staticmethod
    def forward(ctx, x, scale, zero_point, quant_min, quant_max, ch_axis):
        xd = _backend.on_cuda(x)
        out, mask = _backend.ops().fake_quantize(xd, scale, zero_point, quant_min, quant_max, _norm_axis(ch_axis, scale),
                                        want_mask=x.requires_grad)
        if mask is not None:
            ctx.save_for_backward(_back(mask, x))
        return _back(out, x)

    @staticmethod
    def backward(ctx, grad_out):
        (mask,) = ctx.saved_tensors
        return grad_out * mask, None, None, None, None, None


def fake_quantize(x, scale, zero_point, quant_min: int, quant_max: int, ch_axis: int | None = None):
    """Quantize-then-dequantize in the float domain (differentiable through the STE)."""
    if isinstance(scale, torch.Tensor):
        scale = scale.detach()
    if isinstance(zero_point, torch.Tensor):
        zero_point = zero_point.detach()
    return _FakeQuantizeAffine.apply(x, scale, zero_point, quant_min, quant_max, ch_axis)
