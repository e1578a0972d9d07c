"""Quantizable element-wise merges (``lucid/nn/quantized/functional_module.py``): a model
calls ``FloatFunctional.add(x, y)`` instead of ``x + y`` so that ``prepare`` can observe the
merged activation; ``convert`` swaps it for ``QFunctional``, which snaps every merge onto the
one calibrated grid.  On CUDA the merge and the fake-quantize are one kernel
(``lc_fake_quantize_merge_f32``) instead of the reference's eager op chain."""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import activation_qparams
from lucid_b200.nn.quantized.modules import _QuantizedGridModule


class FloatFunctional(nn.Module):
    """Float merges whose result feeds the observer ``prepare`` attaches
    (``functional_module.py:99-122``); a plain passthrough before that."""

    def _obs(self, x: torch.Tensor) -> torch.Tensor:
        app = getattr(self, "activation_post_process", None)
        return app(x) if app is not None else x

    def add(self, x, y):
        return self._obs(x + y)

    def mul(self, x, y):
        return self._obs(x * y)

    def add_relu(self, x, y):
        return self._obs(torch.relu(x + y))

    def cat(self, tensors, dim: int = 0):
        return self._obs(torch.cat(list(tensors), dim=dim))

    def add_scalar(self, x, scalar: float):
        return self._obs(x + scalar)

    def mul_scalar(self, x, scalar: float):
        return self._obs(x * scalar)


class QFunctional(_QuantizedGridModule):
    """Each merge result fake-quantized to the calibrated ``(scale, zero_point)``
    (``functional_module.py:125-330``)."""

    def _merge(self, op: str, x: torch.Tensor, y) -> torch.Tensor:
        xd = _backend.on_cuda(x)
        if isinstance(y, torch.Tensor):
            yd = _backend.on_cuda(y)
            if yd.shape != xd.shape:  # broadcasting merges: eager merge, fused grid
                t = {"add": torch.add, "mul": torch.mul, "add_relu": lambda a, b: torch.relu(a + b)}[op](xd, yd)
                out = self._fake_quant(t)
                return out if x.is_cuda else out.to(x.device)
        else:
            yd = float(y)
        out = _backend.ops().fake_quantize_merge(xd, yd, op, self.scale, self.zero_point, self.qdtype.quant_min,
                                                 self.qdtype.quant_max)
        return out if x.is_cuda else out.to(x.device)

    def add(self, x, y):
        return self._merge("add", x, y)

    def mul(self, x, y):
        return self._merge("mul", x, y)

    def add_relu(self, x, y):
        return self._merge("add_relu", x, y)

    def cat(self, tensors, dim: int = 0):
        return self._fake_quant(torch.cat(list(tensors), dim=dim))

    def add_scalar(self, x, scalar: float):
        return self._merge("add", x, float(scalar))

    def mul_scalar(self, x, scalar: float):
        return self._merge("mul", x, float(scalar))

    @classmethod
    def from_float(cls, mod: nn.Module) -> "QFunctional":
        scale, zero_point, qdtype = activation_qparams(mod)
        return cls(scale, zero_point, qdtype)
