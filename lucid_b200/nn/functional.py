"""``lucid.nn.functional`` (thin view of ``torch.nn.functional``)."""
from torch.nn.functional import *  # noqa: F401,F403
from torch.nn.functional import gelu, layer_norm, linear, relu, silu, softmax  # noqa: F401
