"""``lucid.nn`` surface used by the quantized path.  The reference's module system is
name-for-name ``torch.nn`` (``lucid/nn/module.py:181-1447``): ``register_buffer``,
forward hooks, ``named_children``, ``state_dict`` and slot-preserving child replacement
by ``setattr`` all behave identically, so the float layers are torch's and only the
quantized layers (``lucid_b200.nn.quantized``) are this package's own."""
from torch.nn import (GELU, Embedding, Identity, LayerNorm, Linear, Module, ModuleList, Parameter, ReLU,
                      Sequential, SiLU, Softmax)
from torch.nn import functional  # noqa: F401

from lucid_b200.nn import quantized  # noqa: E402,F401

__all__ = ["Module", "Parameter", "Sequential", "ModuleList", "Linear", "ReLU", "GELU", "SiLU", "LayerNorm",
           "Embedding", "Identity", "Softmax", "functional", "quantized"]
