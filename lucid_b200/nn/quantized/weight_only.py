"""Weight-only int8 layers with per-output-channel symmetric scales and float activations
(W8A16): the decode-time counterpart of the dynamic Linear.  The reference's weight-only
layer is the group-wise ``QuantizedLinearMLX`` (``lucid/nn/quantized/mlx_linear.py:21-256``);
this is the per-channel layout of its sidecar modules (``weight_int8`` / ``weight_scale``
buffers as in ``lucid/nn/quantized/linear.py:189-199``) computed without dequantizing the
weight: up to 32 rows go through the GEMV-shaped kernel that reads the int8 weight once.
"""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.quantization._functional import quantize
from lucid_b200.quantization._qscheme import QDtype, per_channel_symmetric, qint8

_GEMV_MAX_ROWS = 32


def fp32_rows_take_the_gemv(rows: int, weight_elements: int) -> bool:
    """fp32 activations have no tensor-core form of their own: the GEMV-shaped entry point serves them with
    plain FP32 multiply-adds, one warp per output row, which is fine for up to four rows of a small weight and
    falls far behind from five rows on (measured on [4096, 4096]: 14 / 30 us at 1 / 4 rows, 121 / 557 us at
    5 / 32 rows) or when the weight is large ([14336, 4096]: 50 us at one row).  Everything else goes through the
    exact digit-plane product on the tensor cores (8-27 us for these shapes, whatever the row count)."""
    return rows <= 4 and weight_elements < (32 << 20)


class _SettledBuffers:
    """Tells when a module's constant buffers are known to have been complete before the
    previous kernel on the stream started, so that a decode kernel may prefetch them while
    that kernel drains.  True from the second consecutive forward that sees the same
    storages at the same in-place version: every write to them then precedes at least one
    whole kernel of this module, and launches on a stream start in order."""

    def __init__(self) -> None:
        self._seen = None

    def __call__(self, *tensors) -> bool:
        key = tuple((t.data_ptr(), t._version) for t in tensors if t is not None)
        settled = key == self._seen
        self._seen = key
        return settled


def wide_product(x2: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor, bias, cache: dict) -> torch.Tensor:
    """``x2 @ (codes * scale)^T + bias`` for more rows than the GEMV kernel takes, without a float copy
    of the weight: bf16 / f16 activations against the codes widened (exactly) to the same type on
    ``lc_wo_gemm_16``; fp32 activations as int8 digit planes on ``lc_wo_gemm_digits`` (exact).
    ``cache`` keeps the operand form of the weight per (kind, storage, version)."""
    ops = _backend.ops()
    k = x2.shape[1]
    halves = x2.dtype in (torch.bfloat16, torch.float16) and k % 8 == 0
    key = (x2.dtype if halves else "s8", codes.data_ptr(), codes._version)
    if cache.get("key") != key:
        cache["key"] = key
        cache["w"] = ops.widen_s8(codes, x2.dtype)[:, :k] if halves else ops.pad_rows_to_16(codes)
    if halves:
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        return ops.wo_gemm_16(x2, 1, cache["w"], sw=scale, bias=bias, out_dtype=x2.dtype)
    digits, row_scale, _ = ops.split_f32_digits(x2.float())
    return ops.wo_gemm_digits(digits, row_scale, cache["w"], sw=scale, bias=bias).to(x2.dtype)


def _quantize_rows(weight: torch.Tensor, dtype: QDtype):
    from lucid_b200.quantization.observer import PerChannelMinMaxObserver

    obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=dtype)
    obs(weight)
    scale, zero_point = obs.calculate_qparams()
    return quantize(weight, scale, zero_point, dtype, ch_axis=0), scale


class WeightOnlyLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight_int8", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_features))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features))
        else:
            self.bias = None
        self._settled = _SettledBuffers()
        self._wide_cache = {}

    @classmethod
    def from_float(cls, mod: nn.Module, dtype: QDtype = qint8) -> "WeightOnlyLinear":
        m = cls(mod.in_features, mod.out_features, bias=mod.bias is not None)
        codes, scale = _quantize_rows(_backend.on_cuda(mod.weight.detach().float()), dtype)
        m.register_buffer("weight_int8", codes)
        m.register_buffer("weight_scale", scale)
        if mod.bias is not None:
            m.register_buffer("bias", _backend.on_cuda(mod.bias.detach().float()).clone())
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xd = _backend.on_cuda(x)
        x2 = xd.reshape(-1, self.in_features)
        rows = x2.shape[0]
        # (16-bit activations reach the tensor-core GEMV kernels only with rows of K % 16 == 0; other K are served
        # by the same multiply-add kernel as fp32)
        on_tensor_cores = x2.dtype in (torch.bfloat16, torch.float16) and self.in_features % 16 == 0
        gemv = 0 < rows <= _GEMV_MAX_ROWS and (
            on_tensor_cores or fp32_rows_take_the_gemv(rows, self.weight_int8.numel()))
        if gemv:
            y = _backend.ops().wo_linear_s8(
                x2, self.weight_int8, self.weight_scale, self.bias,
                overlap_previous=self._settled(self.weight_int8, self.weight_scale, self.bias))
        elif x2.shape[0] == 0:
            y = x2.new_zeros((0, self.out_features))
        else:  # compute-bound batches: the tensor-core weight-only kernels
            y = self._wide(x2)
        y = y.reshape(*xd.shape[:-1], self.out_features)
        return y if x.is_cuda else y.to(x.device)

    def _wide(self, x2: torch.Tensor) -> torch.Tensor:
        return wide_product(x2, self.weight_int8, self.weight_scale, self.bias, self._wide_cache)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, weight_only=int8"


class WeightOnlySwiGLU(nn.Module):
    """``down(silu(gate(x)) * up(x))`` with int8 weights.  Gate and up rows are stored
    interleaved (blocks of 8) so that decode batches read both matrices in one pass whose
    epilogue applies the activation; the down projection is a :class:`WeightOnlyLinear`."""

    def __init__(self, hidden: int, intermediate: int) -> None:
        super().__init__()
        if intermediate % 8:
            raise ValueError("intermediate size must be a multiple of 8")
        self.hidden, self.intermediate = hidden, intermediate
        self.register_buffer("gate_up_int8", torch.zeros((2 * intermediate, hidden), dtype=torch.int8))
        self.register_buffer("gate_up_scale", torch.ones(2 * intermediate))
        self.down = WeightOnlyLinear(intermediate, hidden, bias=False)
        self._settled = _SettledBuffers()
        self._wide_cache = {}

    @classmethod
    def from_float(cls, gate: nn.Linear, up: nn.Linear, down: nn.Linear, dtype: QDtype = qint8) -> "WeightOnlySwiGLU":
        ops = _backend.ops()
        m = cls(gate.in_features, gate.out_features)
        (wg, sg), (wu, su) = (_quantize_rows(_backend.on_cuda(l.weight.detach().float()), dtype) for l in (gate, up))
        m.register_buffer("gate_up_int8", ops.interleave_gate_up(wg, wu))
        m.register_buffer("gate_up_scale", ops.interleave_gate_up(sg, su))
        m.down = WeightOnlyLinear.from_float(down, dtype)
        return m

    def _split(self, t: torch.Tensor):
        blocks = t.reshape(self.intermediate // 8, 16, *t.shape[1:])
        return blocks[:, :8].reshape(self.intermediate, *t.shape[1:]), blocks[:, 8:].reshape(self.intermediate, *t.shape[1:])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xd = _backend.on_cuda(x)
        x2 = xd.reshape(-1, self.hidden)
        fused_ok = (0 < x2.shape[0] <= _GEMV_MAX_ROWS and x2.dtype in (torch.bfloat16, torch.float16)
                    and self.hidden % 16 == 0)
        if fused_ok:
            h = _backend.ops().wo_swiglu_s8(
                x2, self.gate_up_int8, self.gate_up_scale,
                overlap_previous=self._settled(self.gate_up_int8, self.gate_up_scale))
        else:
            # one product against the interleaved weight; output columns come in blocks of 8 gate / 8 up
            gu = wide_product(x2, self.gate_up_int8, self.gate_up_scale, None, self._wide_cache)
            gu = gu.reshape(x2.shape[0], self.intermediate // 8, 2, 8)
            h = (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(x2.shape[0], self.intermediate)
        y = self.down(h).reshape(*xd.shape[:-1], self.hidden)
        return y if x.is_cuda else y.to(x.device)
