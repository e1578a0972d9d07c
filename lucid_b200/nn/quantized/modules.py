"""Boundary markers of the static PTQ workflow and their converted forms
(``lucid/nn/quantized/modules.py:28-412``): ``QuantStub`` / ``DeQuantStub`` mark where a
float model enters and leaves the quantized region, ``convert`` turns them into ``Quantize``
(fake-quantizes its input onto the calibrated grid, float-carried) and ``DeQuantize``
(identity); ``QuantWrapper`` puts a pair of stubs around a module."""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200.quantization._fake_quantize import FakeQuantize
from lucid_b200.quantization._functional import fake_quantize
from lucid_b200.quantization._qscheme import QDtype, quint8


class _QuantizedGridModule(nn.Module):
    """Carries one output grid ``(scale, zero_point, qdtype)``
    (``lucid/nn/quantized/_utils.py:29-45``)."""

    def __init__(self, scale: torch.Tensor, zero_point: torch.Tensor, qdtype: QDtype = quint8) -> None:
        super().__init__()
        self.register_buffer("scale", scale)
        self.register_buffer("zero_point", zero_point)
        self.qdtype = qdtype

    def _fake_quant(self, x: torch.Tensor) -> torch.Tensor:
        return fake_quantize(x, self.scale, self.zero_point, self.qdtype.quant_min, self.qdtype.quant_max)


class QuantStub(nn.Module):
    """Identity for PTQ (``prepare`` observes its output through a hook); under QAT the
    attached :class:`FakeQuantize` is applied (``modules.py:111-122``)."""

    def __init__(self, qconfig=None) -> None:
        super().__init__()
        if qconfig is not None:
            self.qconfig = qconfig

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        app = getattr(self, "activation_post_process", None)
        if isinstance(app, FakeQuantize) and x.is_floating_point():
            return app(x)
        return x


class DeQuantStub(nn.Module):
    def __init__(self, qconfig=None) -> None:
        super().__init__()
        if qconfig is not None:
            self.qconfig = qconfig

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x


class Quantize(_QuantizedGridModule):
    """Fake-quantizes real-valued inputs onto the calibrated grid; integer inputs (token
    indices) pass through (``modules.py:263-278``)."""

    def forward(self, X: torch.Tensor) -> torch.Tensor:  # noqa: N803 - the reference's argument name
        if not X.is_floating_point():
            return X
        return self._fake_quant(X)

    @classmethod
    def from_float(cls, stub: nn.Module) -> "Quantize":
        obs = stub.activation_post_process
        scale, zero_point = obs.calculate_qparams()
        return cls(scale, zero_point, obs.qdtype)


class DeQuantize(nn.Module):
    def forward(self, Xq: torch.Tensor) -> torch.Tensor:  # noqa: N803
        return Xq

    @classmethod
    def from_float(cls, stub: nn.Module) -> "DeQuantize":
        del stub
        return cls()


class QuantWrapper(nn.Module):
    def __init__(self, module: nn.Module) -> None:
        super().__init__()
        self.quant = QuantStub()
        self.module = module
        self.dequant = DeQuantStub()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dequant(self.module(self.quant(x)))
