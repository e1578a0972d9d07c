"""Quantized convolutions (API and buffers of ``lucid/nn/quantized/conv.py:49-643``,
``conv_transpose.py:45-631`` and the fused ``ConvReLU*d`` of ``intrinsic.py:141-444``): int8
kernel with one scale / zero-point per output channel, float bias, and the output fake-quantized
onto the calibrated activation grid.  As in the reference the convolution itself runs in float:
the kernel is decoded with ``lc_dequantize`` on every forward (only the int8 codes are kept
resident), the convolution is the float library one, and the output requantization is the
``lc_fake_quantize_f32`` kernel."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import activation_qparams, ieee_fp32, quantize_weight, wire_inner
from lucid_b200.quantization._functional import dequantize, fake_quantize, quantize
from lucid_b200.quantization._qscheme import QDtype, per_channel_symmetric, qint8, quint8
from lucid_b200.quantization.observer import PerChannelMinMaxObserver

_FLOAT_CONV = {1: nn.Conv1d, 2: nn.Conv2d, 3: nn.Conv3d}
_CONV_TRANSPOSE = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}


def _as_tuple(value, rank: int) -> tuple[int, ...]:
    return (int(value),) * rank if isinstance(value, int) else tuple(int(v) for v in value)


class _QuantizedConvNd(nn.Module):
    _rank: int

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride, padding, dilation, groups: int,
                 bias: bool, padding_mode: str = "zeros") -> None:
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = padding
        self.dilation = dilation
        self.groups = groups
        self.padding_mode = padding_mode
        self.weight_ch_axis = 0
        self.out_qdtype: QDtype = quint8
        shape = (out_channels, in_channels // groups, *_as_tuple(kernel_size, self._rank))
        self.register_buffer("weight_int8", torch.zeros(shape, dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_channels))
        self.register_buffer("weight_zero_point", torch.zeros(out_channels))
        if bias:
            self.register_buffer("bias", torch.zeros(out_channels))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self._shell = None

    @property
    def padding_str(self) -> str | None:
        return self.padding if isinstance(self.padding, str) else None

    def _float_shell(self) -> nn.Module:
        """A float convolution of the same geometry without storage (meta device): its
        ``_conv_forward`` applies string padding and the padding mode exactly as the float
        layer this module was converted from did.  Kept out of the module registry."""
        if self._shell is None:
            shell = _FLOAT_CONV[self._rank](self.in_channels, self.out_channels, self.kernel_size, self.stride,
                                            self.padding, self.dilation, self.groups, False, self.padding_mode,
                                            device="meta")
            object.__setattr__(self, "_shell", shell)
        return self._shell

    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return y

    def forward(self, input: torch.Tensor) -> torch.Tensor:  # noqa: A002 - the reference's argument name
        x = _backend.on_cuda(input).float()
        weight = dequantize(_backend.on_cuda(self.weight_int8), _backend.on_cuda(self.weight_scale),
                            _backend.on_cuda(self.weight_zero_point), ch_axis=self.weight_ch_axis)
        bias = None if self.bias is None else _backend.on_cuda(self.bias)
        with ieee_fp32():
            y = self._activation(self._float_shell()._conv_forward(x, weight, bias))
        y = fake_quantize(y, _backend.on_cuda(self.scale), _backend.on_cuda(self.zero_point),
                          self.out_qdtype.quant_min, self.out_qdtype.quant_max)
        return y if input.is_cuda else y.to(input.device)

    @classmethod
    def from_float(cls, mod: nn.Module):
        inner = wire_inner(mod)
        qmod = cls(inner.in_channels, inner.out_channels, inner.kernel_size, inner.stride, inner.padding,
                   inner.dilation, inner.groups, inner.bias is not None, inner.padding_mode)
        codes, w_scale, w_zp, ch_axis = quantize_weight(inner)
        qmod.register_buffer("weight_int8", codes)
        qmod.register_buffer("weight_scale", w_scale)
        qmod.register_buffer("weight_zero_point", w_zp)
        qmod.weight_ch_axis = ch_axis
        if inner.bias is not None:
            qmod.register_buffer("bias", _backend.on_cuda(inner.bias.detach()).clone())
        a_scale, a_zp, a_qdtype = activation_qparams(inner)
        qmod.register_buffer("scale", a_scale)
        qmod.register_buffer("zero_point", a_zp)
        qmod.out_qdtype = a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride}, qdtype={self.out_qdtype.name}")


class Conv1d(_QuantizedConvNd):
    _rank = 1


class Conv2d(_QuantizedConvNd):
    _rank = 2


class Conv3d(_QuantizedConvNd):
    _rank = 3


class _ReLUBeforeRequant:
    """The ReLU of a fused pair runs before the output fake-quant, where calibration saw it."""

    def _activation(self, y: torch.Tensor) -> torch.Tensor:
        return torch.relu(y)


class ConvReLU1d(_ReLUBeforeRequant, Conv1d):
    pass


class ConvReLU2d(_ReLUBeforeRequant, Conv2d):
    pass


class ConvReLU3d(_ReLUBeforeRequant, Conv3d):
    pass


class _QuantizedConvTransposeNd(nn.Module):
    """Transposed convolution: weight ``(in, out / groups, *k)`` quantized per output channel on
    axis 1 (``conv_transpose.py:74-83``)."""

    _rank: int

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride, padding, output_padding, dilation,
                 groups: int, bias: bool) -> None:
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = padding
        self.output_padding = output_padding
        self.dilation = dilation
        self.groups = groups
        self.out_qdtype: QDtype = quint8
        self.weight_ch_axis = 1
        n_out = out_channels // groups
        shape = (in_channels, n_out, *_as_tuple(kernel_size, self._rank))
        self.register_buffer("weight_int8", torch.zeros(shape, dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(n_out))
        self.register_buffer("weight_zero_point", torch.zeros(n_out))
        if bias:
            self.register_buffer("bias", torch.zeros(out_channels))
        else:
            self.bias = None
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))

    def forward(self, input: torch.Tensor) -> torch.Tensor:  # noqa: A002
        x = _backend.on_cuda(input).float()
        weight = dequantize(_backend.on_cuda(self.weight_int8), _backend.on_cuda(self.weight_scale),
                            _backend.on_cuda(self.weight_zero_point), ch_axis=self.weight_ch_axis)
        bias = None if self.bias is None else _backend.on_cuda(self.bias)
        rank = self._rank
        with ieee_fp32():
            y = _CONV_TRANSPOSE[rank](x, weight, bias, _as_tuple(self.stride, rank), _as_tuple(self.padding, rank),
                                      _as_tuple(self.output_padding, rank), self.groups,
                                      _as_tuple(self.dilation, rank))
        y = fake_quantize(y, _backend.on_cuda(self.scale), _backend.on_cuda(self.zero_point),
                          self.out_qdtype.quant_min, self.out_qdtype.quant_max)
        return y if input.is_cuda else y.to(input.device)

    @classmethod
    def from_float(cls, mod: nn.Module):
        if isinstance(mod.padding, str):
            raise NotImplementedError("quantized conv_transpose: string padding is not supported yet")
        qmod = cls(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride, mod.padding, mod.output_padding,
                   mod.dilation, mod.groups, mod.bias is not None)
        weight = _backend.on_cuda(mod.weight.detach())
        wobs = PerChannelMinMaxObserver(ch_axis=1, qscheme=per_channel_symmetric, qdtype=qint8)
        wobs(weight)
        w_scale, w_zp = wobs.calculate_qparams()
        qmod.register_buffer("weight_int8", quantize(weight, w_scale, w_zp, qint8, ch_axis=1))
        qmod.register_buffer("weight_scale", w_scale)
        qmod.register_buffer("weight_zero_point", w_zp)
        if mod.bias is not None:
            qmod.register_buffer("bias", _backend.on_cuda(mod.bias.detach()).clone())
        a_scale, a_zp, a_qdtype = activation_qparams(mod)
        qmod.register_buffer("scale", a_scale)
        qmod.register_buffer("zero_point", a_zp)
        qmod.out_qdtype = a_qdtype
        return qmod

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride}, qdtype={self.out_qdtype.name}")


class ConvTranspose1d(_QuantizedConvTransposeNd):
    _rank = 1


class ConvTranspose2d(_QuantizedConvTransposeNd):
    _rank = 2


class ConvTranspose3d(_QuantizedConvTransposeNd):
    _rank = 3
