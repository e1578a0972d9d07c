"""``calculate_qparams``: scale and zero-point from an observed range
(API of ``lucid/quantization/_qparams.py:23-205``), evaluated by the CUDA kernel
``lc_calculate_qparams_f32`` so that every step is an IEEE fp32 operation."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from lucid_b200 import _backend
from lucid_b200.quantization._qscheme import QDtype, QScheme


@dataclass(frozen=True)
class QParams:
    scale: torch.Tensor
    zero_point: torch.Tensor
    qscheme: QScheme
    qdtype: QDtype
    ch_axis: int | None = None


def _as_range_tensor(v) -> torch.Tensor:
    if isinstance(v, torch.Tensor):
        return _backend.on_cuda(v)
    return torch.tensor(float(v), dtype=torch.float32, device=_backend.cuda_device())


def calculate_qparams(min_val, max_val, qscheme: QScheme, qdtype: QDtype, eps: float = 1e-8):
    """Returns ``(scale, zero_point)`` as fp32 tensors shaped like the inputs.

    Symmetric: ``scale = max(|min|,|max|) / ((qmax-qmin)/2)`` (127.5 for qint8),
    zero-point 0 for a signed grid, the grid midpoint for an unsigned one.
    Affine: ``scale = (max-min)/(qmax-qmin)``, ``zp = clip(qmin - round(min/scale))``.
    The range is first widened to contain 0 and the scale floored at ``eps``.
    """
    mn, mx = _as_range_tensor(min_val), _as_range_tensor(max_val)
    shape = torch.broadcast_shapes(mn.shape, mx.shape)
    scale, zp = _backend.ops().calculate_qparams(mn.reshape(-1) if mn.shape == shape else mn.expand(shape).reshape(-1),
                                        mx.reshape(-1) if mx.shape == shape else mx.expand(shape).reshape(-1),
                                        qscheme.is_symmetric, qdtype.quant_min, qdtype.quant_max,
                                        qdtype.signed, eps)
    return scale.reshape(shape), zp.reshape(shape)
