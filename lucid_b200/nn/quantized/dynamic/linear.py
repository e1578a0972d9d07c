"""Dynamically quantized Linear (API and buffers of
``lucid/nn/quantized/dynamic/linear.py:36-113``).

Weights are quantized once, per output row, symmetric int8.  The reference's forward
fake-quantizes ``x`` on a per-tensor affine ``quint8`` grid, dequantizes the weight and
runs a float GEMM; here the same quantities go through the integer form

    acc[m,n] = sum_k xq[m,k] * wq[n,k]           (u8 x s8 -> s32, tcgen05)
    y        = f32(acc - zx*rowsum(wq)[n]) * sx * sw[n] + b[n]

which equals the reference's result up to fp32 summation order.  ``act_scheme``
selects the activation grid: ``"tensor_affine"`` (reference default),
``"tensor_symmetric"`` or ``"token_symmetric"`` (one scale per row of ``x``).
Range, qparams and codes of the activations stay on the device: the forward contains
no host synchronisation.
"""
from __future__ import annotations

import contextlib
import threading
import weakref

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import Int8WeightCache
from lucid_b200.quantization._functional import quantize
from lucid_b200.quantization._qscheme import QDtype, per_channel_symmetric, qint8, quint8

_ACT_SCHEMES = ("tensor_affine", "tensor_symmetric", "token_symmetric")


class _SharedInputCodes:
    """Codes of the activation tensor quantized last inside a :func:`share_quantized_input` block,
    so that sibling layers fed the same tensor there (the q / k / v projections of an attention
    block, the gate and up projections of an MLP) quantize it once.  Sharing is OFF outside such a
    block: the only evidence that two calls see the same values is the tensor object and its
    in-place version counter, and writes that bypass the counter (a producer replayed from a CUDA
    graph, a peer GPU storing into the buffer, any raw-pointer kernel) would be missed.  Inside a
    block the caller vouches that the tensor is not rewritten between the sibling calls.  A hit
    needs the same tensor object (held weakly), version, shape, dtype, grid, CUDA stream and
    graph-capture id; the entry is dropped when the block ends."""

    def __init__(self) -> None:
        self._local = threading.local()

    @property
    def active(self) -> bool:
        return getattr(self._local, "depth", 0) > 0

    def enter(self) -> None:
        self._local.depth = getattr(self._local, "depth", 0) + 1

    def leave(self) -> None:
        self._local.depth -= 1
        if self._local.depth == 0:
            self._local.entry = None

    def get(self, x: torch.Tensor, key):
        entry = getattr(self._local, "entry", None)
        if entry is not None and entry[0]() is x and entry[1] == (x._version, tuple(x.shape), x.dtype, key):
            return entry[2]
        return None

    def put(self, x: torch.Tensor, key, val) -> None:
        self._local.entry = (weakref.ref(x), (x._version, tuple(x.shape), x.dtype, key), val)

    def clear(self) -> None:
        self._local.entry = None


_shared_input = _SharedInputCodes()


@contextlib.contextmanager
def share_quantized_input():
    """Within this block, dynamic Linears that are handed the SAME tensor object reuse its int8
    codes instead of quantizing it again::

        with share_quantized_input():
            q, k, v = self.q(x), self.k(x), self.v(x)

    The caller promises that ``x`` is not written to between those calls by anything torch's
    version counter cannot see (graph replays, peer stores, raw-pointer kernels)."""
    _shared_input.enter()
    try:
        yield
    finally:
        _shared_input.leave()


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight_ch_axis = 0
        self.act_qdtype: QDtype = quint8
        self.act_scheme = "tensor_affine"
        self.out_dtype = torch.float32
        self.register_buffer("weight_int8", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features))
        self.register_buffer("weight_zero_point", torch.zeros(out_features))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None
        self._cache = Int8WeightCache()
        self._scratches = {}

    def set_activation_scheme(self, scheme: str, qdtype: QDtype | None = None) -> "Linear":
        """Choose the activation grid; symmetric schemes default to ``qint8``."""
        if scheme not in _ACT_SCHEMES:
            raise ValueError(f"act_scheme must be one of {_ACT_SCHEMES}, got {scheme!r}")
        self.act_scheme = scheme
        self.act_qdtype = qdtype if qdtype is not None else (quint8 if scheme == "tensor_affine" else qint8)
        return self

    def _quantize_activations(self, x2: torch.Tensor):
        qd = self.act_qdtype
        code_dtype = torch.int8 if qd.signed else torch.uint8
        if self.act_scheme == "token_symmetric":
            xq, sx, _ = _backend.ops().dynamic_quantize_rows(x2, True, qd.quant_min, qd.quant_max, qd.signed, 1e-8,
                                                    code_dtype, pad_rows_to_16=True)
            return xq, sx, None
        symmetric = self.act_scheme == "tensor_symmetric"
        xq, sx, zx, _ = _backend.ops().dynamic_quantize_tensor(x2, symmetric, qd.quant_min, qd.quant_max, qd.signed, 1e-8,
                                                      code_dtype, pad_rows_to_16=True)
        needs_zp = not (symmetric and qd.signed)
        return xq, sx, (zx if needs_zp else None)

    def _scratch(self, rows: int, device: torch.device, stream: int):
        """Workspace of the single-call forward, one per (device, stream) this layer has been used
        on, grown when a larger batch arrives.  Returns ``(buffer, fresh)``."""
        key = (device, stream)
        have = self._scratches.get(key)
        if have is not None and have[0] >= rows:
            return have[1], False
        buf = _backend.ops().dynamic_linear_workspace(rows, self.in_features, device)
        self._scratches[key] = (rows, buf)
        return buf, True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = _backend.ops()
        if (x.is_cuda and x.dtype is torch.float32 and not _shared_input.active and x.is_contiguous()
                and self.weight_int8.device == x.device and x.numel() > 0 and hasattr(ops, "raw_stream")
                and torch.cuda.current_device() == x.device.index):
            # the common eager case in one library call: no intermediate tensors, one stream query
            x2 = x.view(-1, self.in_features)
            wq, wsum = self._cache.get(self.weight_int8, self.weight_zero_point)
            stream = ops.raw_stream(x.device)
            ws, fresh = self._scratch(x2.shape[0], x.device, stream)
            qd = self.act_qdtype
            y = ops.dynamic_linear(x2, self.act_scheme, qd.quant_min, qd.quant_max, qd.signed, wq, self.weight_scale,
                                   self.bias, wsum, ws, fresh, self.out_dtype, stream=stream)
            return y.view(*x.shape[:-1], self.out_features)
        if self.weight_zero_point.is_cuda and x.is_cuda and x.device != self.weight_int8.device:
            raise RuntimeError(f"input on {x.device} but weights on {self.weight_int8.device}")
        xd = _backend.on_cuda(x)
        x2 = xd.reshape(-1, self.in_features)
        if x2.dtype != torch.float32:
            x2 = x2.float()
        wq, wsum = self._cache.get(_backend.on_cuda(self.weight_int8), self.weight_zero_point)
        if x2.shape[0] == 0:
            y = torch.zeros((0, self.out_features), dtype=self.out_dtype, device=xd.device)
        else:
            hit = None
            if x.is_cuda and _shared_input.active:
                key = (self.act_scheme, self.act_qdtype.name, self.in_features, ops.capture_id(xd.device),
                       torch.cuda.current_stream(xd.device).cuda_stream)
                hit = _shared_input.get(x, key)
                if hit is None:
                    hit = self._quantize_activations(x2)
                    _shared_input.put(x, key, hit)
            if hit is None:
                hit = self._quantize_activations(x2)
            xq, sx, zx = hit
            y = ops.qlinear_i8(xq, wq, sx, _backend.on_cuda(self.weight_scale),
                               bias=None if self.bias is None else _backend.on_cuda(self.bias), zx=zx,
                               wsum=wsum if zx is not None else None, out_dtype=self.out_dtype)
        y = y.reshape(*xd.shape[:-1], self.out_features)
        return y if x.is_cuda else y.to(x.device)

    @classmethod
    def from_float(cls, mod: nn.Module, dtype: QDtype = qint8) -> "Linear":
        from lucid_b200.quantization.observer import PerChannelMinMaxObserver

        qmod = cls(mod.in_features, mod.out_features, bias=mod.bias is not None)
        weight = _backend.on_cuda(mod.weight.detach())
        obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=dtype)
        obs(weight)
        scale, zero_point = obs.calculate_qparams()
        qmod.register_buffer("weight_int8", quantize(weight, scale, zero_point, dtype, ch_axis=0))
        qmod.register_buffer("weight_scale", scale)
        qmod.register_buffer("weight_zero_point", zero_point)
        if mod.bias is not None:
            qmod.register_buffer("bias", _backend.on_cuda(mod.bias.detach()).clone())
        return qmod

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, dynamic=True"
