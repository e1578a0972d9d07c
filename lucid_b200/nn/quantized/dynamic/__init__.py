"""Dynamically quantized layers (``lucid/nn/quantized/dynamic/__init__.py``)."""
from lucid_b200.nn.quantized.dynamic.linear import Linear

__all__ = ["Linear"]
