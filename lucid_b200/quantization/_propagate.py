"""QConfig resolution over a module tree (behaviour of
``lucid/quantization/_propagate.py:50-278``).

Precedence for one module: its own ``qconfig`` attribute (``None`` = excluded) beats a
mapping rule for its name or type, which beats what its parent resolved to.
"""
from __future__ import annotations

from collections.abc import Collection, Mapping
from typing import Callable, Iterator, NamedTuple

from torch import nn

from lucid_b200.quantization._qscheme import QDtype, per_channel_symmetric, quint8
from lucid_b200.quantization.observer import PerChannelMinMaxObserver, PlaceholderObserver
from lucid_b200.quantization.qconfig import QConfig, QConfigMapping

_UNSET = object()


class Resolved(NamedTuple):
    name: str
    module: nn.Module
    path: str
    qconfig: QConfig | None


class QConfigResolver:
    def __init__(self, mapping: QConfigMapping, *, implicit: bool = False) -> None:
        self._mapping = mapping
        self._implicit = implicit  # mapping is a library default, not the caller's choice

    @classmethod
    def from_argument(cls, qconfig, default: Callable[[], QConfigMapping]) -> "QConfigResolver":
        if qconfig is None:
            return cls(default(), implicit=True)
        if isinstance(qconfig, QConfig):
            return cls(QConfigMapping().set_global(qconfig))
        if isinstance(qconfig, QConfigMapping):
            return cls(qconfig)
        raise TypeError(
            f"qconfig must be a QConfig, a QConfigMapping or None; got {type(qconfig).__name__}")

    def is_targeted(self, module: nn.Module, path: str) -> bool:
        return (self._mapping._has_rule(type(module), path)
                and self._mapping.get_qconfig(type(module), path) is not None)

    def resolve(self, module: nn.Module, path: str, inherited):
        own = getattr(module, "qconfig", _UNSET)
        if own is not _UNSET:
            if own is not None and not isinstance(own, QConfig):
                raise TypeError(f"{path or type(module).__name__}.qconfig must be a QConfig or None; "
                                f"got {type(own).__name__}")
            return own
        if self._mapping._has_rule(type(module), path):
            return self._mapping.get_qconfig(type(module), path)
        return inherited

    @staticmethod
    def stamp(entry: Resolved) -> Resolved:
        entry.module.qconfig = entry.qconfig
        return entry

    @staticmethod
    def strip(model: nn.Module) -> None:
        for m in model.modules():
            if "qconfig" in m.__dict__:
                del m.qconfig

    def root(self, model: nn.Module) -> Resolved:
        seed = self._mapping._fallback()
        # hand-placed qconfig attributes mean the caller chose what to quantize: a
        # library default must not then spread over the whole model
        if self._implicit and any(hasattr(m, "qconfig") for m in model.modules()):
            seed = None
        return Resolved("", model, "", self.resolve(model, "", seed))

    def children(self, module: nn.Module, path: str, qconfig) -> Iterator[Resolved]:
        for name, child in list(module.named_children()):
            child_path = f"{path}.{name}" if path else name
            yield Resolved(name, child, child_path, self.resolve(child, child_path, qconfig))

    def walk(self, model: nn.Module) -> Iterator[Resolved]:
        """Pre-order traversal, every module once (shared submodules are not revisited)."""
        seen: set[int] = set()
        pending = [self.root(model)]
        while pending:
            entry = pending.pop()
            if id(entry.module) in seen:
                continue
            seen.add(id(entry.module))
            yield entry
            pending.extend(reversed(list(self.children(entry.module, entry.path, entry.qconfig))))


def dynamic_qconfig(dtype: QDtype) -> QConfig:
    """Dynamic recipe: activations quantized at run time, weights per output row symmetric."""
    return QConfig(
        activation=PlaceholderObserver.with_args(qdtype=quint8),
        weight=PerChannelMinMaxObserver.with_args(ch_axis=0, qscheme=per_channel_symmetric, qdtype=dtype),
    )


def weight_dtype(qconfig: QConfig, fallback: QDtype) -> QDtype:
    found = getattr(qconfig.weight(), "qdtype", None)
    return found if isinstance(found, QDtype) else fallback


class DynamicSpec(NamedTuple):
    mapping: QConfigMapping
    targets: tuple[str, ...]


def _spec_value(key, value):
    if value is None or isinstance(value, QConfig):
        return value
    if isinstance(value, QDtype):
        return dynamic_qconfig(value)
    raise TypeError(f"qconfig_spec[{key!r}] must be a QConfig, a QDtype or None; got {type(value).__name__}")


def normalize_dynamic_spec(spec, dtype: QDtype, default_types: Collection[type]) -> DynamicSpec:
    """``None`` -> every type with a dynamic form; a set of types / names -> those, with the
    default recipe; a dict -> per-key QConfig, QDtype or ``None`` (skip)."""
    default = dynamic_qconfig(dtype)
    if spec is None:
        entries = dict.fromkeys(default_types, default)
    elif isinstance(spec, Mapping):
        entries = {k: _spec_value(k, v) for k, v in spec.items()}
    elif isinstance(spec, Collection) and not isinstance(spec, (str, type)):
        entries = dict.fromkeys(spec, default)
    else:
        raise TypeError("qconfig_spec must be a set of module types / names or a dict mapping them to a "
                        f"QConfig, a QDtype or None; got {type(spec).__name__}")
    mapping, targets = QConfigMapping(), []
    for key, qconfig in entries.items():
        if isinstance(key, str):
            mapping.set_module_name(key, qconfig)
            label = key
        elif isinstance(key, type) and issubclass(key, nn.Module):
            mapping.set_object_type(key, qconfig)
            label = key.__name__
        else:
            raise TypeError(f"qconfig_spec keys must be nn.Module subclasses or module names; got {key!r}")
        if qconfig is not None:
            targets.append(label)
    return DynamicSpec(mapping, tuple(sorted(targets)))
