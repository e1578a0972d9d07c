"""Quantized inference layers (``lucid/nn/quantized/__init__.py:15-54``): int8 weights with
``scale`` / ``zero_point`` buffers.  The Linear flavours run on this backend's int8 GEMM / GEMV
kernels and the embedding tables on its lookup kernels; convolutions and standalone
activations compute in float between a weight decode and an output requantization kernel, as
the reference's do.  ``QuantStub`` / ``DeQuantStub`` mark the boundaries of a quantized region
in a float model; ``Quantize`` / ``DeQuantize`` are their converted forms."""
from lucid_b200.nn.quantized import dynamic
from lucid_b200.nn.quantized.activation import ELU, Hardsigmoid, Hardswish, LeakyReLU, Sigmoid, Tanh
from lucid_b200.nn.quantized.conv import (Conv1d, Conv2d, Conv3d, ConvReLU1d, ConvReLU2d, ConvReLU3d,
                                          ConvTranspose1d, ConvTranspose2d, ConvTranspose3d)
from lucid_b200.nn.quantized.functional_module import FloatFunctional, QFunctional
from lucid_b200.nn.quantized.linear import Linear, LinearReLU
from lucid_b200.nn.quantized.mlx_linear import QuantizedLinearMLX
from lucid_b200.nn.quantized.modules import DeQuantize, DeQuantStub, Quantize, QuantStub, QuantWrapper
from lucid_b200.nn.quantized.sparse import Embedding, EmbeddingBag
from lucid_b200.nn.quantized.weight_only import WeightOnlyLinear, WeightOnlySwiGLU

__all__ = ["Linear", "QuantizedLinearMLX", "Conv1d", "Conv2d", "Conv3d", "ConvTranspose1d", "ConvTranspose2d",
           "ConvTranspose3d", "Embedding", "EmbeddingBag", "LinearReLU", "ConvReLU1d", "ConvReLU2d", "ConvReLU3d",
           "QuantStub", "DeQuantStub", "Quantize", "DeQuantize", "QuantWrapper", "FloatFunctional", "QFunctional",
           "Sigmoid", "Hardswish", "Hardsigmoid", "Tanh", "ELU", "LeakyReLU",
           "WeightOnlyLinear", "WeightOnlySwiGLU", "dynamic"]
