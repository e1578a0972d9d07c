"""``QConfig`` (activation / weight observer factories) and ``QConfigMapping``
(global -> by module type -> by module name resolution), API of
``lucid/quantization/qconfig.py:30-512``."""
from __future__ import annotations

from typing import Callable, NamedTuple

from torch import nn

from lucid_b200.quantization._fake_quantize import FakeQuantize
from lucid_b200.quantization._qscheme import per_channel_symmetric, per_tensor_affine, qint8, quint8
from lucid_b200.quantization.observer import (HistogramObserver, MovingAverageMinMaxObserver,
                                              PerChannelMinMaxObserver)

_Factory = Callable[..., nn.Module]


class QConfig(NamedTuple):
    activation: _Factory
    weight: _Factory


def get_default_qconfig() -> QConfig:
    """Static PTQ default: histogram-calibrated affine quint8 activations,
    per-output-channel symmetric qint8 weights."""
    return QConfig(
        activation=HistogramObserver.with_args(qscheme=per_tensor_affine, qdtype=quint8),
        weight=PerChannelMinMaxObserver.with_args(ch_axis=0, qscheme=per_channel_symmetric, qdtype=qint8),
    )


def get_default_qat_qconfig() -> QConfig:
    return QConfig(
        activation=FakeQuantize.with_args(observer=MovingAverageMinMaxObserver, qscheme=per_tensor_affine,
                                          qdtype=quint8),
        weight=FakeQuantize.with_args(observer=PerChannelMinMaxObserver, ch_axis=0,
                                      qscheme=per_channel_symmetric, qdtype=qint8),
    )


class QConfigMapping:
    """Most specific rule wins: module name, then module type, then the global default.
    A rule whose value is ``None`` excludes what it matches."""

    def __init__(self) -> None:
        self._global: QConfig | None = None
        self._object_type: dict[type, QConfig | None] = {}
        self._module_name: dict[str, QConfig | None] = {}

    def set_global(self, qconfig):
        self._global = qconfig
        return self

    def set_object_type(self, module_type: type, qconfig):
        self._object_type[module_type] = qconfig
        return self

    def set_module_name(self, name: str, qconfig):
        self._module_name[name] = qconfig
        return self

    def get_qconfig(self, module_type: type, module_name: str):
        if module_name in self._module_name:
            return self._module_name[module_name]
        if module_type in self._object_type:
            return self._object_type[module_type]
        return self._global

    def _has_rule(self, module_type: type, module_name: str) -> bool:
        return module_name in self._module_name or module_type in self._object_type

    def _fallback(self):
        return self._global


def get_default_qconfig_mapping() -> QConfigMapping:
    return QConfigMapping().set_global(get_default_qconfig())


def get_default_qat_qconfig_mapping() -> QConfigMapping:
    return QConfigMapping().set_global(get_default_qat_qconfig())
