"""``lucid_b200._C``: the C-ABI kernel library (``liblucid_cuda.so``, declared in
``include/lucid_cuda.h``) and its bindings.

Plays the role of the reference's ``lucid._C.engine.quantized`` submodule
(``lucid/_C/bindings/bind_quantized.cpp:17-27``) for the CUDA device.

* ``lucid_b200._C.build``   -- compiles the library with nvcc (no GPU needed);
* ``lucid_b200._C._loader`` -- ctypes loader: fails loudly if the library is missing;
* ``lucid_b200._C.ops``     -- torch-tensor front end of the entry points.

``lib``, ``check``, ``last_error``, ``LucidCudaError``, ``SIGNATURES``, ``LIB_PATH`` and the
``LC_*`` constants are served from the loader on first access, so that the build module
can be imported before the library exists.
"""
from __future__ import annotations


import importlib

_SUBMODULES = ("_loader", "ops", "build")


def __getattr__(name: str):
    if name.startswith("__") or name in _SUBMODULES:
        raise AttributeError(name)
    _loader = importlib.import_module("lucid_b200._C._loader")

    try:
        return getattr(_loader, name)
    except AttributeError:
        raise AttributeError(f"module 'lucid_b200._C' has no attribute {name!r}") from None
