"""lucid_b200: the int8 quantized-inference path of the ``lucid`` framework on
NVIDIA B200 (sm_100a).

Only what that path needs lives here: ``lucid_b200.quantization`` (observers,
qparams, quantize / dequantize / fake_quantize, QConfig, prepare / convert /
quantize_dynamic, ``_qgemm``), ``lucid_b200.nn.quantized`` (the three quantized
``Linear`` layers), ``lucid_b200.backends.quantized``, the ``"cuda"`` device
module ``lucid_b200.cuda`` and the C-ABI kernel library under ``lucid_b200._C``.

The reference's tensor and module APIs are name-for-name PyTorch's, so tensors
are ``torch.Tensor`` and modules are ``torch.nn.Module``: torch provides device
memory, streams and the module system; the arithmetic of the quantized path is in
the library's own CUDA kernels.
"""
from __future__ import annotations

import torch as _torch

__version__ = "0.1.0"

# ---- tensor surface the path touches (lucid/_tensor, lucid/_factories, lucid/_dtype.py) ----
Tensor = _torch.Tensor
dtype = _torch.dtype
float32, float16, bfloat16, float64 = _torch.float32, _torch.float16, _torch.bfloat16, _torch.float64
int8, uint8, int16, int32, int64 = _torch.int8, _torch.uint8, _torch.int16, _torch.int32, _torch.int64
bool_ = _torch.bool
no_grad = _torch.no_grad
manual_seed = _torch.manual_seed


def device(spec="cpu", index=None):
    """``lucid.device``: ``"cpu"``, ``"cuda"`` or ``"cuda:i"``.  The reference's
    ``"metal"`` / ``"gpu"`` (``lucid/_device.py:21-22``) do not exist on this backend."""
    if isinstance(spec, _torch.device):
        return spec
    if isinstance(spec, str) and spec.split(":")[0] in ("metal", "gpu", "mps"):
        raise ValueError(f"device {spec!r} is Apple-only; this backend provides 'cpu' and 'cuda[:i]'")
    return _torch.device(spec) if index is None else _torch.device(spec, index)


def _factory(fn):
    def make(*args, device=None, **kwargs):  # noqa: A002 - mirrors the reference keyword
        if device is not None:
            kwargs["device"] = globals()["device"](device)
        return fn(*args, **kwargs)

    make.__name__ = fn.__name__
    make.__doc__ = f"``lucid.{fn.__name__}`` (thin view of ``torch.{fn.__name__}``)."
    return make


tensor = _factory(_torch.tensor)
zeros, ones, full, empty = (_factory(f) for f in (_torch.zeros, _torch.ones, _torch.full, _torch.empty))
zeros_like, ones_like, full_like = (_factory(f) for f in (_torch.zeros_like, _torch.ones_like, _torch.full_like))
randn, rand, arange = (_factory(f) for f in (_torch.randn, _torch.rand, _torch.arange))

# free functions used by observers / qparams / modules
round, clip, abs, maximum, minimum = _torch.round, _torch.clip, _torch.abs, _torch.maximum, _torch.minimum  # noqa: A001
amin, amax, moveaxis, isinf, where = _torch.amin, _torch.amax, _torch.moveaxis, _torch.isinf, _torch.where
scatter_add, stack, matmul = _torch.scatter_add, _torch.stack, _torch.matmul


def histc(input, bins=100, min=0.0, max=0.0):  # noqa: A002 - the reference's keywords
    """``lucid.histc``: counts over ``[min, max]`` in ``bins`` equal-width bins, in the input's
    dtype.  Range conventions of the reference's adapter (``lucid/_ops/_adapters.py:1256-1279``):
    ``min == max`` takes the range from the data, a single-point range widens to
    ``[v - 1, v + 1]``, a non-finite range is refused, NaN lies in no bin.  CUDA tensors are
    counted by the library's histogram kernel; CPU tensors by ``torch.histc``, whose results the
    reference's own tests pin it to (``lucid/test/unit/ops/test_adapter_index_stats.py:107-127``)."""
    import math

    lo, hi = float(min), float(max)
    if lo > hi:
        raise ValueError(f"histc: max must be at least min, got [{lo}, {hi}]")
    if not input.is_floating_point():
        raise NotImplementedError(f"histc: input must be a floating-point dtype, got {input.dtype}")
    if lo == hi and input.numel() > 0:
        lo, hi = float(input.min()), float(input.max())
    if not (math.isfinite(lo) and math.isfinite(hi)):
        raise ValueError(f"histc: range of [{lo}, {hi}] is not finite")
    if lo == hi:
        lo, hi = lo - 1.0, hi + 1.0
    if not input.is_cuda:
        return _torch.histc(input, bins=bins, min=lo, max=hi)
    from lucid_b200 import _backend

    return _backend.ops().histc(input.reshape(-1), int(bins), lo, hi).to(input.dtype)


from lucid_b200 import backends, cuda  # noqa: E402
from lucid_b200 import nn  # noqa: E402
from lucid_b200 import quantization  # noqa: E402
from lucid_b200 import serialization  # noqa: E402
from lucid_b200.serialization import load, save  # noqa: E402

__all__ = [
    "Tensor", "dtype", "device", "tensor", "zeros", "ones", "full", "empty", "zeros_like", "ones_like",
    "full_like", "randn", "rand", "arange", "histc", "no_grad", "manual_seed", "backends", "cuda", "nn", "quantization", "serialization", "save", "load",
]
