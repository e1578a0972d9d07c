"""``lucid.nn`` surface used by the quantized path.  The reference's module system is
name-for-name ``torch.nn`` (``lucid/nn/module.py:181-1447``): ``register_buffer``,
forward hooks, ``named_children``, ``state_dict`` and slot-preserving child replacement
by ``setattr`` all behave identically, so the float layers are torch's and only the
quantized layers (``lucid_b200.nn.quantized``) are this package's own."""
from torch.nn import (ELU, GELU, BatchNorm1d, BatchNorm2d, BatchNorm3d, Conv1d, Conv2d, Conv3d, ConvTranspose1d,
                      ConvTranspose2d, ConvTranspose3d, Embedding, EmbeddingBag, Hardsigmoid, Hardswish, Identity,
                      LayerNorm, LeakyReLU, Linear, Module, ModuleList, Parameter, ReLU, Sequential, Sigmoid, SiLU,
                      Softmax, Tanh)
from torch.nn import functional  # noqa: F401

from lucid_b200.nn import intrinsic, qat, quantized  # noqa: E402,F401

__all__ = ["Module", "Parameter", "Sequential", "ModuleList", "Linear", "Conv1d", "Conv2d", "Conv3d",
           "ConvTranspose1d", "ConvTranspose2d", "ConvTranspose3d", "BatchNorm1d", "BatchNorm2d", "BatchNorm3d",
           "Embedding", "EmbeddingBag", "ReLU", "GELU", "SiLU", "Sigmoid", "Tanh", "ELU", "LeakyReLU", "Hardswish",
           "Hardsigmoid", "LayerNorm", "Identity", "Softmax", "functional", "intrinsic", "qat", "quantized"]
