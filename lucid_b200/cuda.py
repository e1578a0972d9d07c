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


class GraphedModule(torch.nn.Module):
    """``module`` with its forward captured in a CUDA graph for one input signature.

    The quantized layers launch a handful of short kernels per forward (observe, quantize,
    GEMM or GEMV); at decode and small-batch shapes the host spends longer preparing those
    launches than the GPU spends running them.  Nothing on the quantized path reads device
    values back on the host (dynamic scales stay on the device), so a forward is capturable:
    replaying the graph costs one launch.  Inputs are copied into the captured input buffers;
    the returned tensors are the captured output buffers (overwritten by the next call) unless
    ``clone_outputs`` is set.  Parameters and buffers of ``module`` are read in place at replay
    time, so weight updates that keep their storage are seen."""

    def __init__(self, module: torch.nn.Module, *example_inputs: torch.Tensor, warmup: int = 3,
                 clone_outputs: bool = False) -> None:
        super().__init__()
        if not example_inputs or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in example_inputs):
            raise ValueError("GraphedModule needs CUDA example inputs")
        self.module = module
        self._clone = clone_outputs
        self._inputs = [t.detach().clone() for t in example_inputs]
        side = torch.cuda.Stream(device=self._inputs[0].device)
        side.wait_stream(torch.cuda.current_stream(self._inputs[0].device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):  # first-use work (workspaces, padded weights) stays outside the graph
                module(*self._inputs)
            side.synchronize()
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph, stream=side):
                self._outputs = module(*self._inputs)
        torch.cuda.current_stream(self._inputs[0].device).wait_stream(side)

    def forward(self, *inputs: torch.Tensor):
        if len(inputs) != len(self._inputs):
            raise ValueError(f"captured for {len(self._inputs)} inputs, got {len(inputs)}")
        for dst, src in zip(self._inputs, inputs):
            if src.shape != dst.shape or src.dtype != dst.dtype:
                raise ValueError(f"captured for {tuple(dst.shape)} {dst.dtype}, got {tuple(src.shape)} {src.dtype}")
            dst.copy_(src, non_blocking=True)
        self._graph.replay()
        if not self._clone:
            return self._outputs
        return (self._outputs.clone() if isinstance(self._outputs, torch.Tensor)
                else type(self._outputs)(o.clone() for o in self._outputs))


def make_graphed(module: torch.nn.Module, *example_inputs: torch.Tensor, **kwargs) -> GraphedModule:
    """Capture ``module(*example_inputs)`` in a CUDA graph; see :class:`GraphedModule`."""
    return GraphedModule(module, *example_inputs, **kwargs)


def kernel_library_info() -> dict:
    """Version of liblucid_cuda and the compute capability / SM count of the current device."""
    import ctypes

    from lucid_b200 import _C

    sm, count = ctypes.c_int32(0), ctypes.c_int32(0)
    _C.check(_C.lib.lc_device_info(current_device(), ctypes.byref(sm), ctypes.byref(count)))
    return {"version": int(_C.lib.lc_version()), "sm": sm.value, "sm_count": count.value, "path": _C.LIB_PATH}
