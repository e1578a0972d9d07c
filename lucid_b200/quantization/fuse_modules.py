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


def _fuse_run(mods: Sequence[nn.Module]) -> list[nn.Module]:
    ids: list[nn.Module] = [nn.Identity() for _ in range(len(mods) - 1)]
    first = mods[0]
    if isinstance(first, _CONV_TYPES):
        conv, rest = first, list(mods[1:])
        if rest and isinstance(rest[0], _BN_TYPES):
            conv = fuse_conv_bn_eval(first, rest.pop(0))
        if rest and isinstance(rest[0], nn.ReLU):
            rest.pop(0)
            if not rest:
                return [_CONV_RELU[type(first)](conv, nn.ReLU()), *ids]
        if not rest:
            return [conv, *ids]
    if isinstance(first, nn.Linear) and len(mods) == 2 and isinstance(mods[1], nn.ReLU):
        return [nni.LinearReLU(first, nn.ReLU()), *ids]
    raise ValueError(f"fuse_modules: unsupported fusion pattern {[type(m).__name__ for m in mods]}")


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

    ids: list[nn.Module] = [nn.Identity() for _ in range(len(mods) - 1)]
    first = mods[0]
    if isinstance(first, _CONV_TYPES):
        rank = _CONV_TYPES.index(type(first))
        rest = list(mods[1:])
        if rest and isinstance(rest[0], _BN_TYPES):
            bn = rest.pop(0)
            relu = bool(rest and isinstance(rest[0], nn.ReLU))
            cls = ((nniqat.ConvBnReLU1d, nniqat.ConvBnReLU2d, nniqat.ConvBnReLU3d) if relu
                   else (nniqat.ConvBn1d, nniqat.ConvBn2d, nniqat.ConvBn3d))[rank]
            return [cls(first, bn, qconfig=qconfig), *ids]
        if rest and isinstance(rest[0], nn.ReLU):  # no BatchNorm: the plain fused pair; prepare_qat makes it trainable
            return [_CONV_RELU[type(first)](first, nn.ReLU()), *ids]
        return [first, *ids]
    if isinstance(first, nn.Linear) and len(mods) == 2 and isinstance(mods[1], nn.ReLU):
        return [nni.LinearReLU(first, nn.ReLU()), *ids]
    raise ValueError(f"fuse_modules_qat: unsupported pattern {[type(m).__name__ for m in mods]}")


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
