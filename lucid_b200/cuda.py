"""``lucid.cuda``: the CUDA counterpart of the reference's ``lucid.metal`` device
module (``lucid/metal/__init__.py:39-524``): availability, synchronisation, memory
statistics, streams and events.  Thin views of torch.cuda, which owns the context."""
from __future__ import annotations

import torch

Stream = torch.cuda.Stream
Event = torch.cuda.Event


def is_available() -> bool:
    return torch.cuda.is_available()


def device_count() -> int:
    return torch.cuda.device_count()


def current_device() -> int:
    return torch.cuda.current_device()


def set_device(index: int) -> None:
    torch.cuda.set_device(index)


def get_device_name(index: int | None = None) -> str:
    return torch.cuda.get_device_name(index)


def synchronize(device=None) -> None:
    torch.cuda.synchronize(device)


def empty_cache() -> None:
    torch.cuda.empty_cache()


def memory_allocated(device=None) -> int:
    return torch.cuda.memory_allocated(device)


def max_memory_allocated(device=None) -> int:
    return torch.cuda.max_memory_allocated(device)


def reset_peak_memory_stats(device=None) -> None:
    torch.cuda.reset_peak_memory_stats(device)


def current_stream(device=None):
    return torch.cuda.current_stream(device)


def stream(s):
    return torch.cuda.stream(s)


def kernel_library_info() -> dict:
    """Version of liblucid_cuda and the compute capability / SM count of the current device."""
    import ctypes

    from lucid_b200 import _C

    sm, count = ctypes.c_int32(0), ctypes.c_int32(0)
    _C.check(_C.lib.lc_device_info(current_device(), ctypes.byref(sm), ctypes.byref(count)))
    return {"version": int(_C.lib.lc_version()), "sm": sm.value, "sm_count": count.value, "path": _C.LIB_PATH}
