"""Quantized activations (``lucid/nn/quantized/activation.py:20-475``): the float activation
followed by a fake-quantize onto the calibrated output grid.  ``convert`` swaps a calibrated
``nn.Sigmoid`` / ``nn.Hardswish`` / ... for these so a standalone activation inside a quantized
region is requantized rather than left at full precision.  The activation itself is torch's
elementwise op; the requantization is the ``lc_fake_quantize_f32`` kernel."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import activation_qparams
from lucid_b200.nn.quantized.modules import _QuantizedGridModule


class _QuantizedActivation(_QuantizedGridModule):
    def _act(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def _configure(self, mod: nn.Module) -> None:
        """Copies activation-specific parameters from the float module."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:  # noqa: A002 - the reference's argument name
        y = self._fake_quant(self._act(_backend.on_cuda(input).float()))
        return y if input.is_cuda else y.to(input.device)

    @classmethod
    def from_float(cls, mod: nn.Module):
        scale, zero_point, qdtype = activation_qparams(mod)
        obj = cls(scale, zero_point, qdtype)
        obj._configure(mod)
        return obj


class Sigmoid(_QuantizedActivation):
    def _act(self, x):
        return torch.sigmoid(x)


class Hardswish(_QuantizedActivation):
    def _act(self, x):
        return F.hardswish(x)


class Hardsigmoid(_QuantizedActivation):
    def _act(self, x):
        return F.hardsigmoid(x)


class Tanh(_QuantizedActivation):
    def _act(self, x):
        return torch.tanh(x)


class ELU(_QuantizedActivation):
    alpha: float = 1.0

    def _configure(self, mod: nn.Module) -> None:
        self.alpha = float(getattr(mod, "alpha", 1.0))

    def _act(self, x):
        return F.elu(x, self.alpha)


class LeakyReLU(_QuantizedActivation):
    negative_slope: float = 0.01

    def _configure(self, mod: nn.Module) -> None:
        self.negative_slope = float(getattr(mod, "negative_slope", 0.01))

    def _act(self, x):
        return F.leaky_relu(x, self.negative_slope)
