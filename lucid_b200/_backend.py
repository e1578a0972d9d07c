"""Access to the CUDA kernel front end (``lucid_b200._C.ops``) and device helpers.

The quantized path has exactly one implementation: the sm_100a kernels behind the
C ABI.  ``ops()`` imports the front end on first use and raises if the shared library
has not been built.  Callers reach these helpers as attributes of this module
(``_backend.ops()``, ``_backend.on_cuda(t)``).
"""
from __future__ import annotations

import torch

_OPS = None


def ops():
    global _OPS
    if _OPS is None:
        from lucid_b200._C import ops as _ops  # ImportError if liblucid_cuda.so is missing

        _OPS = _ops
    return _OPS


def cuda_device(index: int | None = None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError(
            "lucid_b200's quantized path runs on a CUDA device only (sm_100a kernels, no CPU fallback) "
            "and no CUDA device is available"
        )
    return torch.device("cuda", torch.cuda.current_device() if index is None else index)


def on_cuda(t: torch.Tensor) -> torch.Tensor:
    """The tensor itself if it already lives on a CUDA device, else a copy on the current one."""
    return t if t.is_cuda else t.to(cuda_device())
