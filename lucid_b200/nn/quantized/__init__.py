"""Quantized inference layers (``lucid/nn/quantized/__init__.py:26-54``): the three
Linear flavours of the int8 path.  Convolution, embedding, recurrent and activation
wrappers of the reference are float-compute composites outside this backend's scope."""
from lucid_b200.nn.quantized import dynamic
from lucid_b200.nn.quantized.linear import Linear, LinearReLU
from lucid_b200.nn.quantized.mlx_linear import QuantizedLinearMLX
from lucid_b200.nn.quantized.weight_only import WeightOnlyLinear, WeightOnlySwiGLU

__all__ = ["Linear", "LinearReLU", "QuantizedLinearMLX", "WeightOnlyLinear", "WeightOnlySwiGLU", "dynamic"]
