"""Which ``QConfig`` every module of a tree gets (contract of
``lucid/quantization/_propagate.py:50-278`` as pinned by
``lucid/test/unit/quantization/test_qconfig_propagation.py``).

The tree is resolved in one flat pass into a :class:`QConfigTable` -- one row per module,
in ``named_modules`` order -- before anything is observed or swapped; ``prepare``,
``prepare_qat`` and ``quantize_dynamic`` then only read rows.  A row's qconfig is the first of

1. the module's own ``qconfig`` attribute (``None`` excludes the module and, through rule 3,
   what hangs below it),
2. a mapping rule for its dotted name, else for its type,
3. what its parent's row resolved to (for the root: the mapping's global entry).
"""
from __future__ import annotations

from collections.abc import Collection, Mapping
from dataclasses import dataclass
from typing import Callable, Iterator, NamedTuple

from torch import nn

from lucid_b200.quantization._qscheme import QDtype, per_channel_symmetric, quint8
from lucid_b200.quantization.observer import PerChannelMinMaxObserver, PlaceholderObserver
from lucid_b200.quantization.qconfig import QConfig, QConfigMapping

_NO_ATTRIBUTE = object()


@dataclass
class Row:
    """One module of the tree with its resolved qconfig."""

    path: str            # dotted name, "" for the root
    module: nn.Module
    qconfig: QConfig | None
    by_rule: bool        # a mapping rule with a qconfig (not None) names this module or its type

    @property
    def parent_path(self) -> str:
        return self.path.rpartition(".")[0]

    @property
    def name(self) -> str:
        return self.path.rpartition(".")[2]


class QConfigTable:
    """Rows in pre-order (parents before children); shared submodules appear once, under the
    first name they are reached by."""

    def __init__(self, rows: list[Row]) -> None:
        self._rows = {row.path: row for row in rows}

    def __iter__(self) -> Iterator[Row]:
        return iter(self._rows.values())

    def __getitem__(self, path: str) -> Row:
        return self._rows[path]

    @property
    def root(self) -> Row:
        return self._rows[""]

    def parent_module(self, row: Row) -> nn.Module:
        return self._rows[row.parent_path].module

    def stamp(self) -> "QConfigTable":
        """Write every row's qconfig onto its module (what ``convert`` and ``from_float`` read)."""
        for row in self:
            row.module.qconfig = row.qconfig
        return self

    def below(self, path: str) -> Callable[[Row], bool]:
        prefix = f"{path}." if path else ""
        return lambda row: row.path.startswith(prefix) and row.path != path


def clear_stamps(model: nn.Module) -> None:
    for module in model.modules():
        module.__dict__.pop("qconfig", None)


class QConfigResolver:
    """Resolves a model against one ``QConfigMapping``."""

    def __init__(self, mapping: QConfigMapping, *, library_default: bool = False) -> None:
        self.mapping = mapping
        # the mapping is this library's default recipe rather than something the caller passed
        self.library_default = library_default

    @classmethod
    def from_argument(cls, qconfig, default: Callable[[], QConfigMapping]) -> "QConfigResolver":
        """The ``qconfig`` argument of ``prepare`` / ``prepare_qat``: nothing, one recipe for the
        whole model, or a mapping."""
        if isinstance(qconfig, QConfigMapping):
            return cls(qconfig)
        if isinstance(qconfig, QConfig):
            return cls(QConfigMapping().set_global(qconfig))
        if qconfig is None:
            return cls(default(), library_default=True)
        raise TypeError(
            f"qconfig must be a QConfig, a QConfigMapping or None; got {type(qconfig).__name__}")

    def _own(self, module: nn.Module, path: str):
        own = getattr(module, "qconfig", _NO_ATTRIBUTE)
        if own is _NO_ATTRIBUTE or own is None or isinstance(own, QConfig):
            return own
        raise TypeError(f"{path or type(module).__name__}.qconfig must be a QConfig or None; "
                        f"got {type(own).__name__}")

    def table(self, model: nn.Module) -> QConfigTable:
        rows: dict[str, Row] = {}
        # A caller who placed qconfig attributes by hand has said what to quantize; the library's
        # default recipe must then not spread from the root over everything else.
        hand_placed = self.library_default and any(hasattr(m, "qconfig") for m in model.modules())
        for path, module in model.named_modules():
            kind = type(module)
            ruled = self.mapping._has_rule(kind, path)
            rule = self.mapping.get_qconfig(kind, path) if ruled else None
            own = self._own(module, path)
            if own is not _NO_ATTRIBUTE:
                resolved = own
            elif ruled:
                resolved = rule
            elif path == "":
                resolved = None if hand_placed else self.mapping._fallback()
            else:
                resolved = rows[path.rpartition(".")[0]].qconfig
            rows[path] = Row(path, module, resolved, ruled and rule is not None)
        return QConfigTable(list(rows.values()))


# ---- quantize_dynamic's spec argument ---------------------------------------------------
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
    targets: tuple[str, ...]   # labels of the entries that ask for quantization, for the warnings


def normalize_dynamic_spec(spec, dtype: QDtype, default_types: Collection[type]) -> DynamicSpec:
    """``None`` -> every type with a dynamic form; a set of types / names -> those, with the
    default recipe for ``dtype``; a dict -> per key a ``QConfig``, a ``QDtype`` (the default
    recipe at that width) or ``None`` (leave float)."""
    recipe = dynamic_qconfig(dtype)
    if spec is None:
        pairs = [(kind, recipe) for kind in default_types]
    elif isinstance(spec, Mapping):
        pairs = []
        for key, value in spec.items():
            if isinstance(value, QDtype):
                value = dynamic_qconfig(value)
            elif value is not None and not isinstance(value, QConfig):
                raise TypeError(f"qconfig_spec[{key!r}] must be a QConfig, a QDtype or None; "
                                f"got {type(value).__name__}")
            pairs.append((key, value))
    elif isinstance(spec, Collection) and not isinstance(spec, (str, type)):
        pairs = [(key, recipe) for key in spec]
    else:
        raise TypeError("qconfig_spec must be a set of module types / names or a dict mapping them to a "
                        f"QConfig, a QDtype or None; got {type(spec).__name__}")
    mapping = QConfigMapping()
    wanted: list[str] = []
    for key, qconfig in pairs:
        if isinstance(key, str):
            mapping.set_module_name(key, qconfig)
        elif isinstance(key, type) and issubclass(key, nn.Module):
            mapping.set_object_type(key, qconfig)
        else:
            raise TypeError(f"qconfig_spec keys must be nn.Module subclasses or module names; got {key!r}")
        if qconfig is not None:
            wanted.append(key if isinstance(key, str) else key.__name__)
    return DynamicSpec(mapping, tuple(sorted(wanted)))
