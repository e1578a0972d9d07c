"""Import alias: makes ``import lucid`` / ``import lucid.quantization as Q`` /
``from lucid.quantization import _qgemm`` resolve to ``lucid_b200`` so code written
against the reference's module paths runs unchanged on the CUDA backend."""
import importlib
import sys

import lucid_b200 as _impl

_ALIASES = (
    "backends", "cuda", "nn", "nn.functional", "nn.quantized", "nn.quantized.dynamic", "quantization",
    "quantization._qgemm", "quantization.observer", "quantization.qconfig", "quantization._functional",
    "quantization._qparams", "quantization._qscheme", "_C",
)
for _name in _ALIASES:
    sys.modules[f"lucid.{_name}"] = importlib.import_module(f"lucid_b200.{_name}")
sys.modules["lucid"] = _impl
