"""Fused float modules (``lucid/nn/intrinsic/modules.py``): plain ``Sequential`` pairs emitted
by :func:`lucid_b200.quantization.fuse_modules`.  They compute exactly what their members
compute; packaging them tells ``prepare`` to put one activation observer after the ReLU and
``convert`` to build the fused quantized layer."""
from torch import nn


class _FusedModule(nn.Sequential):
    """Tag for fused float modules."""


class LinearReLU(_FusedModule):
    def __init__(self, linear: nn.Linear, relu: nn.ReLU) -> None:
        super().__init__(linear, relu)


class ConvReLU1d(_FusedModule):
    def __init__(self, conv: nn.Conv1d, relu: nn.ReLU) -> None:
        super().__init__(conv, relu)


class ConvReLU2d(_FusedModule):
    def __init__(self, conv: nn.Conv2d, relu: nn.ReLU) -> None:
        super().__init__(conv, relu)


class ConvReLU3d(_FusedModule):
    def __init__(self, conv: nn.Conv3d, relu: nn.ReLU) -> None:
        super().__init__(conv, relu)


__all__ = ["LinearReLU", "ConvReLU1d", "ConvReLU2d", "ConvReLU3d"]

from lucid_b200.nn.intrinsic import qat  # noqa: E402,F401  (trainable Conv + BatchNorm fusion)
