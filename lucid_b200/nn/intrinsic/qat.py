"""Trainable fused Conv + BatchNorm (+ ReLU) for QAT (``lucid/nn/intrinsic/qat/modules.py``).

A layer that folded BatchNorm into the convolution once would freeze the statistics; these
fold on every forward instead: the kernel is scaled by ``gamma / sqrt(running_var + eps)``,
fake-quantized (this backend's ``lc_fake_quantize_f32`` with its straight-through mask),
convolved, unscaled, and then the BatchNorm itself runs -- so it keeps training on batch
statistics while the weight already sees the folded int8 grid.  ``convert`` folds one last time
and bakes an int8 ``nn.quantized.Conv*d`` / ``ConvReLU*d``; no BatchNorm layer survives."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F
from torch.nn.utils.fusion import fuse_conv_bn_weights

from lucid_b200.nn.quantized._utils import ieee_fp32

_CONV_FNS = (F.conv1d, F.conv2d, F.conv3d)


class _ConvBnNd(nn.Module):
    _relu = False

    def __init__(self, conv: nn.Module, bn: nn.Module, relu: bool | None = None, qconfig=None) -> None:
        super().__init__()
        if qconfig is None:
            raise ValueError(f"{type(self).__name__} requires a qconfig")
        if not getattr(bn, "track_running_stats", False):
            raise ValueError(f"{type(self).__name__} requires a BatchNorm that tracks running statistics "
                             "(track_running_stats=True)")
        self.conv = conv
        self.bn = bn
        self.relu = self._relu if relu is None else bool(relu)
        self.qconfig = qconfig
        self.weight_fake_quant = qconfig.weight()
        self.activation_post_process = qconfig.activation()
        self.freeze_bn = False
        self.update_bn_stats()

    def _fold(self):
        """BatchNorm folded into the convolution's ``(weight, bias)`` with the running statistics."""
        conv, bn = self.conv, self.bn
        return fuse_conv_bn_weights(conv.weight, conv.bias, bn.running_mean, bn.running_var, bn.eps,
                                    bn.weight if bn.affine else None, bn.bias if bn.affine else None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        conv, bn = self.conv, self.bn
        running_std = (bn.running_var + bn.eps).sqrt()
        gamma = bn.weight if bn.affine else torch.ones_like(running_std)
        scale = gamma / running_std
        out_channels, ndim = conv.weight.shape[0], conv.weight.dim()
        w_q = self.weight_fake_quant(conv.weight * scale.reshape((out_channels,) + (1,) * (ndim - 1)))
        per_channel = (1, out_channels) + (1,) * (ndim - 2)
        with ieee_fp32():
            y = _CONV_FNS[ndim - 3](x, w_q, None, conv.stride, conv.padding, conv.dilation, conv.groups)
        y = y / scale.reshape(per_channel)
        if conv.bias is not None:
            y = y + conv.bias.reshape(per_channel)
        y = self.bn(y)
        if self.relu:
            y = torch.relu(y)
        return self.activation_post_process(y)

    def update_bn_stats(self):
        """``bn`` normalises with batch statistics and updates its running ones."""
        self.freeze_bn = False
        self.bn.training = True
        return self

    def freeze_bn_stats(self):
        """``bn`` normalises with its running statistics and stops updating them."""
        self.freeze_bn = True
        self.bn.training = False
        return self

    def train(self, mode: bool = True):
        super().train(mode)
        if self.freeze_bn:
            self.bn.training = False
        return self


class ConvBn1d(_ConvBnNd):
    pass


class ConvBn2d(_ConvBnNd):
    pass


class ConvBn3d(_ConvBnNd):
    pass


class ConvBnReLU1d(_ConvBnNd):
    _relu = True


class ConvBnReLU2d(_ConvBnNd):
    _relu = True


class ConvBnReLU3d(_ConvBnNd):
    _relu = True


def convbn_to_quantized(mod: nn.Module) -> nn.Module:
    """The int8 inference convolution of a trained fused layer: BatchNorm folded a last time, the
    folded kernel observed and quantized by the layer's own weight fake-quantizer."""
    import lucid_b200.nn.quantized as nnq
    from lucid_b200 import _backend
    from lucid_b200.quantization._functional import quantize

    with torch.no_grad():
        weight, bias = mod._fold()
        weight, bias = _backend.on_cuda(weight.detach()), _backend.on_cuda(bias.detach())
        wfq = mod.weight_fake_quant
        wfq(weight)
        w_scale, w_zp = wfq.calculate_qparams()
        ch_axis = wfq.ch_axis if wfq.ch_axis is not None else 0
        codes = quantize(weight, w_scale, w_zp, wfq.qdtype, ch_axis=wfq.ch_axis)
    conv = mod.conv
    rank = conv.weight.dim() - 2
    plain, fused = (nnq.Conv1d, nnq.Conv2d, nnq.Conv3d), (nnq.ConvReLU1d, nnq.ConvReLU2d, nnq.ConvReLU3d)
    q = (fused if mod.relu else plain)[rank - 1](conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride,
                                                 conv.padding, conv.dilation, conv.groups, True, conv.padding_mode)
    q.register_buffer("weight_int8", codes)
    q.register_buffer("weight_scale", w_scale)
    q.register_buffer("weight_zero_point", w_zp)
    q.weight_ch_axis = ch_axis
    q.register_buffer("bias", bias.clone())
    a_scale, a_zp = mod.activation_post_process.calculate_qparams()
    q.register_buffer("scale", _backend.on_cuda(a_scale))
    q.register_buffer("zero_point", _backend.on_cuda(a_zp))
    q.out_qdtype = mod.activation_post_process.qdtype
    return q


# names the reference uses for the same builder
_convbn_to_quantized = convbn_to_quantized
convbnrelu2d_to_quantized = convbn_to_quantized

__all__ = ["ConvBn1d", "ConvBn2d", "ConvBn3d", "ConvBnReLU1d", "ConvBnReLU2d", "ConvBnReLU3d"]
