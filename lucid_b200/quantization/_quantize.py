"""Eager-mode workflows: ``prepare`` -> calibrate -> ``convert`` (static PTQ) and
``quantize_dynamic`` (behaviour of ``lucid/quantization/_quantize.py:199-620``) for the
Linear layers this backend accelerates.  Children are replaced with ``setattr`` so they
keep their slot and order in the parent."""
from __future__ import annotations

import copy
import warnings

from torch import nn

from lucid_b200 import backends
from lucid_b200.quantization._propagate import (QConfigResolver, QConfigTable, clear_stamps, normalize_dynamic_spec,
                                                 weight_dtype)
from lucid_b200.quantization._qscheme import QDtype, qint8
from lucid_b200.quantization.qconfig import (get_default_qat_qconfig_mapping, get_default_qconfig_mapping)


def _observed_types() -> tuple[type, ...]:
    """Float module types whose output ``prepare`` observes (``_quantize.py:46-71``)."""
    import lucid_b200.nn.intrinsic as nni
    import lucid_b200.nn.quantized as nnq

    return (nn.Linear, nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.ConvTranspose1d, nn.ConvTranspose2d, nn.ConvTranspose3d,
            nni.ConvReLU1d, nni.ConvReLU2d, nni.ConvReLU3d, nni.LinearReLU, nn.Sigmoid, nn.Hardswish,
            nn.Hardsigmoid, nn.Tanh, nn.ELU, nn.LeakyReLU, nnq.QuantStub, nnq.FloatFunctional)


def _quant_mapping() -> dict:
    """Float module type -> ``from_float`` builder of its quantized form (``_quantize.py:74-121``)."""
    import lucid_b200.nn.intrinsic as nni
    import lucid_b200.nn.intrinsic.qat as nniqat
    import lucid_b200.nn.qat as nnqat
    import lucid_b200.nn.quantized as nnq

    return {
        nn.Linear: nnq.Linear.from_float,
        nn.Conv1d: nnq.Conv1d.from_float, nn.Conv2d: nnq.Conv2d.from_float, nn.Conv3d: nnq.Conv3d.from_float,
        nn.ConvTranspose1d: nnq.ConvTranspose1d.from_float, nn.ConvTranspose2d: nnq.ConvTranspose2d.from_float,
        nn.ConvTranspose3d: nnq.ConvTranspose3d.from_float,
        nn.Embedding: nnq.Embedding.from_float, nn.EmbeddingBag: nnq.EmbeddingBag.from_float,
        nn.Sigmoid: nnq.Sigmoid.from_float, nn.Hardswish: nnq.Hardswish.from_float,
        nn.Hardsigmoid: nnq.Hardsigmoid.from_float, nn.Tanh: nnq.Tanh.from_float, nn.ELU: nnq.ELU.from_float,
        nn.LeakyReLU: nnq.LeakyReLU.from_float,
        nni.ConvReLU1d: nnq.ConvReLU1d.from_float, nni.ConvReLU2d: nnq.ConvReLU2d.from_float,
        nni.ConvReLU3d: nnq.ConvReLU3d.from_float, nni.LinearReLU: nnq.LinearReLU.from_float,
        nnq.QuantStub: nnq.Quantize.from_float, nnq.DeQuantStub: nnq.DeQuantize.from_float,
        nnq.FloatFunctional: nnq.QFunctional.from_float,
        # trained QAT layers become the same inference layers
        nniqat.ConvBn1d: nniqat.convbn_to_quantized, nniqat.ConvBn2d: nniqat.convbn_to_quantized,
        nniqat.ConvBn3d: nniqat.convbn_to_quantized, nniqat.ConvBnReLU1d: nniqat.convbn_to_quantized,
        nniqat.ConvBnReLU2d: nniqat.convbn_to_quantized, nniqat.ConvBnReLU3d: nniqat.convbn_to_quantized,
        nnqat.Linear: nnq.Linear.from_float, nnqat.LinearReLU: nnq.LinearReLU.from_float,
        nnqat.Conv1d: nnq.Conv1d.from_float, nnqat.Conv2d: nnq.Conv2d.from_float, nnqat.Conv3d: nnq.Conv3d.from_float,
        nnqat.ConvReLU1d: nnq.ConvReLU1d.from_float, nnqat.ConvReLU2d: nnq.ConvReLU2d.from_float,
        nnqat.ConvReLU3d: nnq.ConvReLU3d.from_float, nnqat.Embedding: nnq.Embedding.from_float,
    }


# ---- group-wise (engine "mlx_group") builders --------------------------------
def _group_weight_bits(mod: nn.Module) -> int:
    qcfg = getattr(mod, "qconfig", None)
    if qcfg is not None:
        bits = getattr(getattr(qcfg.weight(), "qdtype", None), "bits", None)
        if isinstance(bits, int) and bits in (4, 8):
            return bits
    return 8


def _group_size_for(in_features: int):
    for gs in (64, 128, 32):
        if in_features % gs == 0:
            return gs
    return None


def _group_linear_builder(relu: bool = False):
    """Builder routing a (fused) Linear to the group-wise weight-only GEMM; a fused pair hands
    over its inner Linear with the ReLU folded into the kernel's epilogue (``_quantize.py:148-185``)."""

    def build(child: nn.Module) -> nn.Module:
        from lucid_b200.nn.quantized import Linear as QLinear
        from lucid_b200.nn.quantized import LinearReLU as QLinearReLU
        from lucid_b200.nn.quantized import QuantizedLinearMLX

        inner = child[0] if isinstance(child, nn.Sequential) else child
        gs = _group_size_for(inner.in_features)
        if gs is None:  # no group size divides in_features: keep the per-channel int8 module
            return (QLinearReLU if relu else QLinear).from_float(child)
        if inner is not child and getattr(inner, "qconfig", None) is None:
            inner.qconfig = getattr(child, "qconfig", None)
        return QuantizedLinearMLX.from_float(inner, bits=_group_weight_bits(inner), group_size=gs, relu=relu)

    return build


def _group_dynamic_builder(child: nn.Module, dtype: QDtype) -> nn.Module:
    import lucid_b200.nn.quantized.dynamic as nnqd
    from lucid_b200.nn.quantized import QuantizedLinearMLX

    gs = _group_size_for(child.in_features)
    if gs is None:
        return nnqd.Linear.from_float(child, dtype)
    return QuantizedLinearMLX.from_float(child, bits=dtype.bits, group_size=gs)


# ---- static PTQ ------------------------------------------------------------------
def _observer_hook(obs: nn.Module):
    def hook(_module, _args, output) -> None:
        obs(output)

    return hook


def prepare(model: nn.Module, qconfig=None, inplace: bool = False) -> nn.Module:
    """Attach an activation observer (as a forward hook) to every quantizable module the
    qconfig resolution selects; returns the model ready for calibration."""
    resolver = QConfigResolver.from_argument(qconfig, get_default_qconfig_mapping)
    model = model if inplace else copy.deepcopy(model)
    model.eval()
    observed = _observed_types()
    matched = 0
    for row in resolver.table(model).stamp():
        if row.qconfig is None or not isinstance(row.module, observed):
            continue
        obs = row.qconfig.activation()
        row.module.activation_post_process = obs
        row.module.register_forward_hook(_observer_hook(obs))
        matched += 1
    if matched == 0:
        warnings.warn("prepare(): the QConfigMapping matched no quantizable modules — convert() will "
                      "leave this model unchanged.", stacklevel=2)
    return model


def convert(model: nn.Module, inplace: bool = False) -> nn.Module:
    """Swap every calibrated module for its quantized counterpart and drop the
    ``qconfig`` stamps."""
    import lucid_b200.nn.quantized as nnq

    model = model if inplace else copy.deepcopy(model)
    import lucid_b200.nn.intrinsic as nni

    mapping = _quant_mapping()
    if backends.quantized.use_mlx():
        mapping[nn.Linear] = _group_linear_builder()
        mapping[nni.LinearReLU] = _group_linear_builder(relu=True)
    # the stub leaving the quantized region and embedding tables need no calibration
    _convert_children(model, mapping, always=(nnq.DeQuantStub, nn.Embedding, nn.EmbeddingBag))
    clear_stamps(model)
    model.eval()
    return model


def _convert_children(module: nn.Module, mapping, always: tuple[type, ...] = ()) -> None:
    """Swap calibrated children (and the ``always`` types, which carry no state to calibrate,
    unless ``prepare`` stamped them ``qconfig = None``) in their original slots."""
    for name, child in list(module.named_children()):
        build = mapping.get(type(child))
        stateless = isinstance(child, always) and getattr(child, "qconfig", True) is not None
        if build is not None and (hasattr(child, "activation_post_process") or stateless):
            child._forward_hooks.clear()
            setattr(module, name, build(child))
        else:
            _convert_children(child, mapping, always)


# ---- dynamic PTQ -------------------------------------------------------------------
def _dynamic_builders():
    import lucid_b200.nn.quantized.dynamic as nnqd

    builders = {nn.Linear: nnqd.Linear.from_float, nn.LSTM: nnqd.LSTM.from_float, nn.GRU: nnqd.GRU.from_float,
                nn.LSTMCell: nnqd.LSTMCell.from_float, nn.GRUCell: nnqd.GRUCell.from_float,
                nn.RNNCell: nnqd.RNNCell.from_float}
    if backends.quantized.use_mlx():
        builders[nn.Linear] = _group_dynamic_builder
    return builders


def quantize_dynamic(model: nn.Module, qconfig_spec=None, dtype: QDtype = qint8, inplace: bool = False):
    """Replace the targeted float layers by dynamically quantized ones; no calibration.

    ``qconfig_spec``: ``None`` (every supported type), a set of module types / dotted names,
    or a dict mapping those to a ``QConfig``, a ``QDtype`` or ``None`` (skip).

    Two phases: the whole tree is resolved first (which module gets which recipe), then the
    selected layers are swapped in their parents' slots.  Nothing is touched when the spec is
    malformed, because resolution happens before the first swap."""
    builders = _dynamic_builders()
    spec = normalize_dynamic_spec(qconfig_spec, dtype, tuple(builders))
    model = model if inplace else copy.deepcopy(model)
    model.eval()
    table = QConfigResolver(spec.mapping).table(model)

    def build(row):
        return builders[type(row.module)](row.module, weight_dtype(row.qconfig, dtype))

    root = table.root
    if root.qconfig is not None and type(root.module) in builders:  # the model is itself one bare layer
        out = build(root)
        clear_stamps(out)
        return out

    swapped_prefixes: list[str] = []   # subtrees that have been replaced as a whole
    stays_float: set[type] = set()     # asked for by a rule, but no dynamic form exists
    for row in table:
        if row.path == "" or row.qconfig is None:
            continue
        if any(row.path.startswith(prefix) for prefix in swapped_prefixes):
            continue
        if type(row.module) in builders:
            setattr(table.parent_module(row), row.name, build(row))
            swapped_prefixes.append(row.path + ".")
        elif row.by_rule and next(row.module.children(), None) is None:
            stays_float.add(type(row.module))
    if stays_float:
        left = ", ".join(sorted(t.__name__ for t in stays_float))
        have = ", ".join(sorted(t.__name__ for t in builders))
        warnings.warn(f"quantize_dynamic(): {left} has no dynamically quantized form and stays float; "
                      f"dynamic quantization covers {have}.", stacklevel=2)
    elif not swapped_prefixes:
        warnings.warn("quantize_dynamic(): no module of a targeted type "
                      f"({', '.join(spec.targets) or 'none'}) found — the model is returned unchanged.",
                      stacklevel=2)
    clear_stamps(model)
    return model


# ---- quantization-aware training ----------------------------------------------------------
def _qat_mapping() -> dict:
    """Float module type -> builder of its trainable fake-quantized form (``_quantize.py:622-640``)."""
    import lucid_b200.nn.intrinsic as nni
    import lucid_b200.nn.qat as nnqat

    return {nn.Linear: nnqat.Linear.from_float, nn.Conv1d: nnqat.Conv1d.from_float,
            nn.Conv2d: nnqat.Conv2d.from_float, nn.Conv3d: nnqat.Conv3d.from_float,
            nn.Embedding: nnqat.Embedding.from_float, nni.LinearReLU: nnqat.LinearReLU.from_float,
            nni.ConvReLU1d: nnqat.ConvReLU1d.from_float, nni.ConvReLU2d: nnqat.ConvReLU2d.from_float,
            nni.ConvReLU3d: nnqat.ConvReLU3d.from_float}


def prepare_qat(model: nn.Module, qconfig=None, inplace: bool = False) -> nn.Module:
    """Swap every weighted layer the qconfig resolution selects for its ``nn.qat`` form and
    give every ``QuantStub`` a fake-quantizer; the model is returned in ``train`` mode, ready
    to be fine-tuned and then handed to :func:`convert` (``_quantize.py:643-737``)."""
    import lucid_b200.nn.quantized as nnq
    from lucid_b200.nn.intrinsic.qat import _ConvBnNd

    resolver = QConfigResolver.from_argument(qconfig, get_default_qat_qconfig_mapping)
    model = model if inplace else copy.deepcopy(model)
    model.train()
    qat_map = _qat_mapping()
    table = resolver.table(model).stamp()
    closed: list[str] = []  # subtrees already made trainable as a whole: nothing below them is visited
    for row in table:
        if row.path == "" or any(row.path.startswith(prefix) for prefix in closed):
            continue
        child, build = row.module, qat_map.get(type(row.module))
        if isinstance(child, _ConvBnNd):
            closed.append(row.path + ".")  # fuse_modules_qat made it trainable; its conv runs through the fused forward
        elif row.qconfig is not None and build is not None:
            setattr(table.parent_module(row), row.name, build(child))
            closed.append(row.path + ".")
        elif row.qconfig is not None and isinstance(child, nnq.QuantStub):
            child.activation_post_process = row.qconfig.activation()
            closed.append(row.path + ".")
    return model
