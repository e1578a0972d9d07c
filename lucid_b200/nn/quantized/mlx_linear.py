"""``QuantizedLinearMLX``: weight-only group-wise int8 / int4 Linear (API and buffers of
``lucid/nn/quantized/mlx_linear.py:21-256``; the class keeps the reference's name so
converted checkpoints and routing code keep working).  The packed weight is stored under
an int32 tag, scales and biases per (row, group).  Device-transparent like the
reference: a CPU input is moved to the GPU and the result moved back."""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized.weight_only import _SettledBuffers
from lucid_b200.quantization._qgemm import quantize, quantized_matmul, wide_group_product


class QuantizedLinearMLX(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, bits: int = 8,
                 group_size: int = 64, relu: bool = False) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.bits = bits
        self.group_size = group_size
        self.relu = relu
        self.register_buffer("packed_weight", torch.zeros((out_features, in_features * bits // 32), dtype=torch.int32))
        self.register_buffer("scales", torch.zeros((out_features, in_features // group_size)))
        self.register_buffer("biases", torch.zeros((out_features, in_features // group_size)))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None
        self._wide_cache = {}
        self._settled = _SettledBuffers()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xd = _backend.on_cuda(x)
        rows = xd.numel() // max(self.in_features, 1)
        if rows > 32 and not (xd.requires_grad and torch.is_grad_enabled()):
            # compute-bound batches: the weight decoded once per module, bias and ReLU in the GEMM's epilogue
            y = wide_group_product(xd.reshape(-1, self.in_features), self.packed_weight, self.scales, self.biases,
                                   self.group_size, self.bits, cache=self._wide_cache,
                                   bias=None if self.bias is None else _backend.on_cuda(self.bias), relu=self.relu)
            y = y.reshape(*xd.shape[:-1], self.out_features)
            if y.dtype != x.dtype:
                y = y.to(x.dtype)
            return y if x.is_cuda else y.to(x.device)
        if (0 < rows <= 32 and xd.dtype in (torch.bfloat16, torch.float16) and self.packed_weight.is_cuda
                and not (xd.requires_grad and torch.is_grad_enabled())):
            # decode batches: the streaming kernel may fetch this layer's weights while the kernel before it on the
            # stream drains, once the buffers are known to have been complete before that kernel started
            x2 = xd.reshape(-1, self.in_features)
            y = _backend.ops().group_matmul(
                x2, self.packed_weight, self.scales, self.biases, self.group_size, self.bits,
                overlap_previous=self._settled(self.packed_weight, self.scales, self.biases))
            y = y.reshape(*xd.shape[:-1], self.out_features)
            if self.bias is not None:
                y = y + _backend.on_cuda(self.bias).to(y.dtype)
            if self.relu:
                y = torch.relu(y)
            return y if x.is_cuda else y.to(x.device)
        y = quantized_matmul(xd, self.packed_weight, self.scales, self.biases, transpose=True,
                             group_size=self.group_size, bits=self.bits)
        if self.bias is not None:
            y = y + _backend.on_cuda(self.bias).to(y.dtype)
        if self.relu:
            y = torch.relu(y)
        if y.dtype != x.dtype:
            y = y.to(x.dtype)
        return y if x.is_cuda else y.to(x.device)

    @classmethod
    def from_float(cls, mod: nn.Module, bits: int = 8, group_size: int = 64, relu: bool = False):
        m = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, bits=bits,
                group_size=group_size, relu=relu)
        packed, scales, biases = quantize(_backend.on_cuda(mod.weight.detach()), group_size=group_size, bits=bits)
        m.register_buffer("packed_weight", packed)
        m.register_buffer("scales", scales)
        m.register_buffer("biases", biases)
        if mod.bias is not None:
            m.register_buffer("bias", _backend.on_cuda(mod.bias.detach()).clone())
        return m

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"group_size={self.group_size}, relu={self.relu}, backend=cuda")
