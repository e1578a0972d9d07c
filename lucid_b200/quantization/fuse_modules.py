"""``fuse_modules`` / ``fuse_modules_qat`` (``lucid/quantization/fuse_modules.py:86-247``): collapse named runs of
Conv (+ BatchNorm) (+ ReLU) or Linear + ReLU into one module before ``prepare``.  The first
member of a run is replaced by the fused module, the others by ``Identity``, each in its own
slot, so a hand-written ``forward`` keeps working.  BatchNorm is folded into the convolution's
weight with its frozen statistics (eval mode)."""
from __future__ import annotations

import copy
from collections.abc import Sequence

from torch import nn
from torch.nn.utils.fusion import fuse_conv_bn_eval

from lucid_b200.nn import intrinsic as nni

_CONV_TYPES = (nn.Conv1d, nn.Conv2d, nn.Conv3d)
_BN_TYPES = (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)
_CONV_RELU = {nn.Conv1d: nni.ConvReLU1d, nn.Conv2d: nni.ConvReLU2d, nn.Conv3d: nni.ConvReLU3d}


def _set_module(root: nn.Module, dotted: str, value: nn.Module) -> None:
    parent_path, _, name = dotted.rpartition(".")
    parent = root.get_submodule(parent_path) if parent_path else root
    setattr(parent, name, value)


def _kind(mod: nn.Module) -> str:
    """One letter per member of a run: C conv, B batch norm, R ReLU, L linear, ? anything else."""
    if isinstance(mod, _CONV_TYPES):
        return "C"
    if isinstance(mod, _BN_TYPES):
        return "B"
    if isinstance(mod, nn.ReLU):
        return "R"
    return "L" if isinstance(mod, nn.Linear) else "?"


# signature of a run -> the module that replaces its first member
_FUSED_HEAD = {
    "CB": lambda m: fuse_conv_bn_eval(m[0], m[1]),
    "CBR": lambda m: _CONV_RELU[type(m[0])](fuse_conv_bn_eval(m[0], m[1]), nn.ReLU()),
    "CR": lambda m: _CONV_RELU[type(m[0])](m[0], nn.ReLU()),
    "LR": lambda m: nni.LinearReLU(m[0], nn.ReLU()),
}


def _fuse_run(mods: Sequence[nn.Module]) -> list[nn.Module]:
    make_head = _FUSED_HEAD.get("".join(_kind(m) for m in mods))
    if make_head is None:
        raise ValueError(f"fuse_modules: unsupported fusion pattern {[type(m).__name__ for m in mods]}")
    return [make_head(mods)] + [nn.Identity() for _ in mods[1:]]


def fuse_modules(model: nn.Module, modules_to_fuse: Sequence[Sequence[str]], inplace: bool = False) -> nn.Module:
    """Supported runs: ``[Conv, BN]``, ``[Conv, BN, ReLU]``, ``[Conv, ReLU]``, ``[Linear, ReLU]``;
    anything else raises ``ValueError``.  Put the model in ``eval`` mode first."""
    model = model if inplace else copy.deepcopy(model)
    for group in modules_to_fuse:
        mods = [model.get_submodule(name) for name in group]
        for name, repl in zip(group, _fuse_run(mods), strict=True):
            _set_module(model, name, repl)
    return model


def _fuse_run_qat(mods: Sequence[nn.Module], qconfig) -> list[nn.Module]:
    from lucid_b200.nn.intrinsic import qat as nniqat

    signature = "".join(_kind(m) for m in mods)
    rank = _CONV_TYPES.index(type(mods[0])) if signature.startswith("C") else 0
    heads = {
        # a BatchNorm after the conv: the trainable layer that folds it on every forward
        "CB": lambda: (nniqat.ConvBn1d, nniqat.ConvBn2d, nniqat.ConvBn3d)[rank](mods[0], mods[1], qconfig=qconfig),
        "CBR": lambda: (nniqat.ConvBnReLU1d, nniqat.ConvBnReLU2d, nniqat.ConvBnReLU3d)[rank](mods[0], mods[1],
                                                                                           qconfig=qconfig),
        # no BatchNorm: the plain fused pair; prepare_qat makes it trainable
        "CR": lambda: _CONV_RELU[type(mods[0])](mods[0], nn.ReLU()),
        "C": lambda: mods[0],
        "LR": lambda: nni.LinearReLU(mods[0], nn.ReLU()),
    }
    if signature not in heads:
        raise ValueError(f"fuse_modules_qat: unsupported pattern {[type(m).__name__ for m in mods]}")
    return [heads[signature]()] + [nn.Identity() for _ in mods[1:]]


def fuse_modules_qat(model: nn.Module, modules_to_fuse: Sequence[Sequence[str]], qconfig, inplace: bool = False):
    """Fusion for quantization-aware training: a Conv followed by a BatchNorm becomes a trainable
    ``nn.intrinsic.qat.ConvBn*`` layer that folds the BatchNorm on every forward (run before
    ``prepare_qat``, which leaves those layers as they are)."""
    model = model if inplace else copy.deepcopy(model)
    for group in modules_to_fuse:
        mods = [model.get_submodule(name) for name in group]
        for name, repl in zip(group, _fuse_run_qat(mods, qconfig), strict=True):
            _set_module(model, name, repl)
    return model
