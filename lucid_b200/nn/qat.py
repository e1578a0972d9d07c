"""Quantization-aware-training layers (``lucid/nn/qat/{linear,conv,sparse}.py``): the float layer
with a trainable float weight, whose weight and output both pass through a
:class:`~lucid_b200.quantization.FakeQuantize` on every forward.  The rounding is this backend's
``lc_fake_quantize_f32`` kernel, which also writes the straight-through mask the backward
multiplies the incoming gradient with; the linear / convolution between the two fake-quantize
steps is the float library op.  ``prepare_qat`` installs these, ``convert`` turns them into the
int8 inference layers of ``lucid_b200.nn.quantized``."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F


def _attach(mod: nn.Module, qconfig, what: str, activation: bool = True) -> None:
    if qconfig is None:
        raise ValueError(f"qat.{what} requires a qconfig")
    mod.qconfig = qconfig
    mod.weight_fake_quant = qconfig.weight()
    if activation:
        mod.activation_post_process = qconfig.activation()


class Linear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, qconfig=None) -> None:
        super().__init__(in_features, out_features, bias)
        _attach(self, qconfig, "Linear")

    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.linear(x, self.weight_fake_quant(self.weight), self.bias)
        return self.activation_post_process(self._activation(y))

    @classmethod
    def from_float(cls, mod: nn.Module):
        """Shares the float layer's trained parameters (``prepare_qat`` works on a deep copy)."""
        qat = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, qconfig=mod.qconfig)
        qat.weight = mod.weight
        if mod.bias is not None:
            qat.bias = mod.bias
        return qat


class LinearReLU(Linear):
    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return torch.relu(y)

    @classmethod
    def from_float(cls, mod: nn.Module):
        inner = mod[0]
        inner.qconfig = mod.qconfig
        return super().from_float(inner)


class _ConvMixin:
    """Forward and construction shared by the three ranks."""

    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._conv_forward(x, self.weight_fake_quant(self.weight), self.bias)
        return self.activation_post_process(self._activation(y))

    @classmethod
    def from_float(cls, mod: nn.Module):
        if isinstance(mod, nn.Sequential):  # a fused [conv, relu] pair hands over its conv
            mod[0].qconfig = mod.qconfig
            mod = mod[0]
        qat = cls(mod.in_channels, mod.out_channels, mod.kernel_size, stride=mod.stride, padding=mod.padding,
                  dilation=mod.dilation, groups=mod.groups, bias=mod.bias is not None,
                  padding_mode=mod.padding_mode, qconfig=mod.qconfig)
        qat.weight = mod.weight
        if mod.bias is not None:
            qat.bias = mod.bias
        return qat


def _qat_conv(base: type, name: str, relu: bool) -> type:
    def __init__(self, *args, qconfig=None, **kwargs) -> None:
        base.__init__(self, *args, **kwargs)
        _attach(self, qconfig, name)

    body = {"__init__": __init__, "__doc__": f"QAT form of ``nn.{base.__name__}``" + (" with a fused ReLU." if relu else ".")}
    if relu:
        body["_activation"] = lambda self, y: torch.relu(y)
    return type(name, (_ConvMixin, base), body)


Conv1d = _qat_conv(nn.Conv1d, "Conv1d", False)
Conv2d = _qat_conv(nn.Conv2d, "Conv2d", False)
Conv3d = _qat_conv(nn.Conv3d, "Conv3d", False)
ConvReLU1d = _qat_conv(nn.Conv1d, "ConvReLU1d", True)
ConvReLU2d = _qat_conv(nn.Conv2d, "ConvReLU2d", True)
ConvReLU3d = _qat_conv(nn.Conv3d, "ConvReLU3d", True)


class Embedding(nn.Embedding):
    """Fake-quantizes the table, then looks up (``lucid/nn/qat/sparse.py``); weight-only, so
    there is no output fake-quantize."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None, *,
                 qconfig=None) -> None:
        super().__init__(num_embeddings, embedding_dim, padding_idx=padding_idx)
        _attach(self, qconfig, "Embedding", activation=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.embedding(x, self.weight_fake_quant(self.weight), self.padding_idx)

    @classmethod
    def from_float(cls, mod: nn.Module):
        qat = cls(mod.num_embeddings, mod.embedding_dim, padding_idx=mod.padding_idx, qconfig=mod.qconfig)
        qat.weight = mod.weight
        return qat


__all__ = ["Linear", "LinearReLU", "Conv1d", "Conv2d", "Conv3d", "ConvReLU1d", "ConvReLU2d", "ConvReLU3d", "Embedding"]
