"""Statically quantized Linear (API and buffers of ``lucid/nn/quantized/linear.py:37-242``):
int8 weights with a per-channel scale, float input, and the output fake-quantized onto
the calibrated activation grid.  The reference dequantizes the whole weight on every
forward, calls a float GEMM and then runs the fake-quantize chain
(``linear.py:206-214``); here the whole forward is one kernel: up to four rows of a
weight below 32 M elements go through the weight-only GEMV kernel (the weight is read
once as int8), everything else
through the tensor-core kernel on exact integer arithmetic (``lc_wo_gemm_digits``: the
fp32 activations as four int8 digit planes, int32 accumulation, one rounding), and in
both the scale, bias, ReLU and output requantization are the kernel's epilogue.  No
floating-point copy of the weight is made.
"""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import StaticWeightCache, activation_qparams, quantize_weight, wire_inner
from lucid_b200.nn.quantized.weight_only import fp32_rows_take_the_gemv
from lucid_b200.quantization._qscheme import QDtype, quint8



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
        self._weights = StaticWeightCache()

    _relu = False  # LinearReLU: a ReLU between the bias and the output requantization

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = _backend.ops()
        xd = _backend.on_cuda(x)
        x2 = xd.reshape(-1, self.in_features)
        if x2.dtype != torch.float32:  # the reference computes this layer in fp32
            x2 = x2.float()
        wq = _backend.on_cuda(self.weight_int8)
        bias = None if self.bias is None else _backend.on_cuda(self.bias)
        w = self._weights.get(wq, _backend.on_cuda(self.weight_scale), _backend.on_cuda(self.weight_zero_point),
                              self.weight_ch_axis)
        grid = dict(relu=self._relu, out_scale=_backend.on_cuda(self.scale), out_zp=_backend.on_cuda(self.zero_point),
                    quant_min=self.out_qdtype.quant_min, quant_max=self.out_qdtype.quant_max)
        rows = x2.shape[0]
        if rows == 0:
            y = torch.zeros((0, self.out_features), dtype=torch.float32, device=x2.device)
        elif w.gemv_ok and fp32_rows_take_the_gemv(rows, wq.numel()):
            y = ops.wo_linear_s8(x2, wq, w.row_scale, bias, **grid)
        else:
            rowsum = None
            if w.col_scale is not None:
                x2 = x2 * w.col_scale
                if w.col_zp is not None:
                    rowsum = (x2 * w.col_zp).sum(1)
            digits, row_scale, rs = ops.split_f32_digits(x2, want_rowsum=w.colcorr is not None and rowsum is None)
            y = ops.wo_gemm_digits(digits, row_scale, w.codes16(wq), sw=w.row_scale, bias=bias,
                                   rowsum=rowsum if rowsum is not None else rs, colcorr=w.colcorr, **grid)
        y = y.reshape(*xd.shape[:-1], self.out_features)
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

    _relu = True

    @classmethod
    def from_float(cls, mod: nn.Module) -> "LinearReLU":
        return super().from_float(wire_inner(mod))
