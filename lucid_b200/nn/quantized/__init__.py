"""Quantized inference layers (``lucid/nn/quantized/__init__.py:26-54``): the Linear
flavours of the int8 path, the stub / functional boundaries of the static workflow.
Convolution, embedding and activation wrappers of the reference are float-compute composites
outside this backend's scope."""
from lucid_b200.nn.quantized import dynamic
from lucid_b200.nn.quantized.functional_module import FloatFunctional, QFunctional
from lucid_b200.nn.quantized.linear import Linear, LinearReLU
from lucid_b200.nn.quantized.modules import DeQuantize, DeQuantStub, Quantize, QuantStub, QuantWrapper
from lucid_b200.nn.quantized.mlx_linear import QuantizedLinearMLX
from lucid_b200.nn.quantized.weight_only import WeightOnlyLinear, WeightOnlySwiGLU

__all__ = ["Linear", "LinearReLU", "QuantizedLinearMLX", "WeightOnlyLinear", "WeightOnlySwiGLU", "FloatFunctional",
           "QFunctional", "QuantStub", "DeQuantStub", "Quantize", "DeQuantize", "QuantWrapper", "dynamic"]
