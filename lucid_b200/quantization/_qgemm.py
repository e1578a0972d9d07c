"""Group-wise affine weight-only primitives, the Python face of the engine boundary
``lucid._C.engine.quantized`` (API of ``lucid/quantization/_qgemm.py:24-314``;
engine side ``lucid/_C/ops/quantized/QuantizedMatmul.cpp:111-207``), served here by
``lc_group_quantize_f32`` / ``lc_group_dequantize`` / ``lc_group_matmul``.

Format: per (row, group of ``group_size`` input columns) ``scale = (max-min)/(2^bits-1)``
and ``bias = min``; codes are unsigned, packed ``32/bits`` per 32-bit word (first code
in the low bits) and carried in an ``int32`` tensor as the reference does.
"""
from __future__ import annotations

import torch

from lucid_b200 import _backend

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def is_available() -> bool:
    try:
        _backend.ops()
    except ImportError:
        return False
    return torch.cuda.is_available()


def quantize(w, group_size: int = 64, bits: int = 8):
    """``(packed, scales, biases)`` of a 2-D weight ``[out, in]``."""
    return _backend.ops().group_quantize(_backend.on_cuda(w), group_size, bits)


def dequantize(wq, scales, biases, group_size: int = 64, bits: int = 8):
    """Dense float32 ``[out, in]`` reconstruction ``code * scale + bias``."""
    return _backend.ops().group_dequantize(_backend.on_cuda(wq), _backend.on_cuda(scales), _backend.on_cuda(biases), group_size, bits)


def wide_group_product(x2, wq, scales, biases, group_size: int, bits: int, cache=None, bias=None, relu: bool = False):
    """``relu(x2 @ w_hat.T + bias)`` for more rows than the streaming kernel takes.  The reference
    hands every shape to one engine call (``lucid/quantization/_qgemm.py:311-314``) and names the
    decode-then-multiply form as its exact counterpart (``_qgemm.py:289-291``); at these sizes the
    product, not the weight's bytes, is what costs, so the weight is decoded to the activation type
    and bf16 / f16 activations then run on the
    library's own tensor-core kernel (``lc_wo_gemm_16``, fp32 accumulation, bias and ReLU in its
    epilogue); fp32 activations take torch's fp32 product.  ``cache`` (a dict owned by the caller)
    keeps the decoded weight per (type, storages, in-place versions), so that a module decodes once."""
    ops = _backend.ops()
    key = (x2.dtype,) + tuple((t.data_ptr(), t._version) for t in (wq, scales, biases))
    if cache is not None and cache.get("key") == key:
        dense = cache["w"]
    else:
        dense = ops.group_dequantize(wq, scales, biases, group_size, bits).to(x2.dtype)
        if cache is not None:
            cache["key"], cache["w"] = key, dense
    if x2.dtype in (torch.bfloat16, torch.float16) and x2.shape[1] % 8 == 0:
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        return ops.wo_gemm_16(x2, 1, dense, bias=bias, relu=relu, out_dtype=x2.dtype)
    y = x2 @ dense.T
    if bias is not None:
        y = y + bias.to(y.dtype)
    return torch.relu(y) if relu else y


def _forward(xd, wq, scales, biases, transpose: bool, group_size: int, bits: int):
    lead = xd.shape[:-1]
    x2 = xd.reshape(-1, xd.shape[-1])
    if not transpose:
        dense = _backend.ops().group_dequantize(wq, scales, biases, group_size, bits).to(xd.dtype)
        return (x2 @ dense).reshape(*lead, dense.shape[1])
    if x2.shape[0] <= 32:
        y = _backend.ops().group_matmul(x2, wq, scales, biases, group_size, bits)
    else:  # compute-bound shapes
        y = wide_group_product(x2, wq, scales, biases, group_size, bits)
    return y.reshape(*lead, wq.shape[0])


class _QuantizedMatmul(torch.autograd.Function):
    """Differentiable in ``x`` only, like the engine's node: the backward decodes the packed
    weight and multiplies, ``dX = dY @ w_hat`` for the Linear form and ``dY @ w_hat.T``
    otherwise (``QuantizedMatmulBackward::apply``, ``lucid/_C/ops/quantized/QuantizedMatmul.cpp:73-90``).
    This is what a LoRA adapter on a frozen quantized base layer trains through
    (``lucid/peft/tuners/lora/_layer.py:988-1018``)."""

    @staticmethod
    def forward(ctx, xd, wq, scales, biases, transpose, group_size, bits):
        ctx.save_for_backward(wq, scales, biases)
        ctx.cfg = (transpose, group_size, bits)
        return _forward(xd, wq, scales, biases, transpose, group_size, bits)

    @staticmethod
    def backward(ctx, grad_out):
        wq, scales, biases = ctx.saved_tensors
        transpose, group_size, bits = ctx.cfg
        dense = _backend.ops().group_dequantize(wq, scales, biases, group_size, bits)
        if not transpose:
            dense = dense.T
        if dense.dtype != grad_out.dtype:
            dense = dense.to(grad_out.dtype)
        return grad_out @ dense, None, None, None, None, None, None


def quantized_matmul(x, wq, scales, biases, transpose: bool = True, group_size: int = 64, bits: int = 8):
    """``x @ w_hat.T`` (``transpose=True``, the Linear form) or ``x @ w_hat`` with the
    weight decoded inside the kernel; float activations, result in ``x``'s dtype.
    Differentiable with respect to ``x``."""
    if (transpose and x.is_cuda and wq.is_cuda and not (x.requires_grad and torch.is_grad_enabled())
            and x.dim() == 2 and x.shape[0] <= 32 and x.is_contiguous() and wq.is_contiguous()
            and scales.dtype is torch.float32 and scales.is_contiguous() and biases.dtype is torch.float32
            and biases.is_contiguous() and x.device == wq.device == scales.device == biases.device
            and x.device.index == torch.cuda.current_device() and x.dtype in _FLOATS
            and wq.shape[1] * 32 // bits == x.shape[1]
            and not (x.dtype is torch.float32 and wq.numel() >= (1 << 20))):  # (large weights, fp32 rows: see group_matmul)
        # decode-time dispatch: everything the general path would normalise is already in place
        lean = getattr(_backend.ops(), "group_matmul_lean", None)
        if lean is not None:
            return lean(x, wq, scales, biases, group_size, bits)
    xd = _backend.on_cuda(x)
    wq, scales, biases = _backend.on_cuda(wq), _backend.on_cuda(scales), _backend.on_cuda(biases)
    if xd.requires_grad and torch.is_grad_enabled():
        return _QuantizedMatmul.apply(xd, wq, scales, biases, transpose, group_size, bits)
    return _forward(xd, wq, scales, biases, transpose, group_size, bits)
