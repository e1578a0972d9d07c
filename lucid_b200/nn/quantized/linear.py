"""Statically quantized Linear (API and buffers of ``lucid/nn/quantized/linear.py:37-242``):
int8 weights with a per-channel scale, float input, and the output fake-quantized onto
the calibrated activation grid.  The reference dequantizes the whole weight on every
forward and calls a float GEMM; here decode batches go through the weight-only GEMV
kernel (the weight is read once as int8) and larger batches decode the weight with
``lc_dequantize`` before a dense product.  The output requantization is one kernel.
"""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import activation_qparams, quantize_weight, wire_inner
from lucid_b200.quantization._functional import dequantize, fake_quantize
from lucid_b200.quantization._qscheme import QDtype, quint8

_GEMV_MAX_ROWS = 32


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight_ch_axis = 0
        self.out_qdtype: QDtype = quint8
        self.register_buffer("weight_int8", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features))
        self.register_buffer("weight_zero_point", torch.zeros(out_features))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))

    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return y

    def _weight_is_symmetric_per_row(self) -> bool:
        return self.weight_ch_axis == 0 and self.weight_scale.numel() == self.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xd = _backend.on_cuda(x)
        x2 = xd.reshape(-1, self.in_features)
        wq = _backend.on_cuda(self.weight_int8)
        bias = None if self.bias is None else _backend.on_cuda(self.bias)
        if 0 < x2.shape[0] <= _GEMV_MAX_ROWS and self._weight_is_symmetric_per_row():
            y = _backend.ops().wo_linear_s8(x2, wq, _backend.on_cuda(self.weight_scale), bias)
            # a non-zero weight zero-point (affine weight observers) shifts every output by
            # -z[n]*s[n]*sum_k x[m,k]
            wz = _backend.on_cuda(self.weight_zero_point)
            if bool((wz != 0).any()):
                y = y - (x2.float().sum(1, keepdim=True) * (wz * _backend.on_cuda(self.weight_scale))[None, :]).to(y.dtype)
        else:
            w = dequantize(wq, _backend.on_cuda(self.weight_scale), _backend.on_cuda(self.weight_zero_point),
                           ch_axis=self.weight_ch_axis)
            y = torch.nn.functional.linear(x2.to(w.dtype), w, bias)
        y = self._activation(y.reshape(*xd.shape[:-1], self.out_features))
        y = fake_quantize(y.float(), _backend.on_cuda(self.scale), _backend.on_cuda(self.zero_point), self.out_qdtype.quant_min,
                          self.out_qdtype.quant_max)
        return y if x.is_cuda else y.to(x.device)

    @classmethod
    def from_float(cls, mod: nn.Module) -> "Linear":
        qmod = cls(mod.in_features, mod.out_features, bias=mod.bias is not None)
        codes, w_scale, w_zp, ch_axis = quantize_weight(mod)
        qmod.register_buffer("weight_int8", codes)
        qmod.register_buffer("weight_scale", w_scale)
        qmod.register_buffer("weight_zero_point", w_zp)
        qmod.weight_ch_axis = ch_axis
        if mod.bias is not None:
            qmod.register_buffer("bias", _backend.on_cuda(mod.bias.detach()).clone())
        a_scale, a_zp, a_qdtype = activation_qparams(mod)
        qmod.register_buffer("scale", a_scale)
        qmod.register_buffer("zero_point", a_zp)
        qmod.out_qdtype = a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"qdtype={self.out_qdtype.name}")


class LinearReLU(Linear):
    """Static Linear with a ReLU applied before the output requantization
    (``lucid/nn/quantized/intrinsic.py``)."""

    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return torch.relu(y)

    @classmethod
    def from_float(cls, mod: nn.Module) -> "LinearReLU":
        return super().from_float(wire_inner(mod))
