"""Quantization schemes and integer grids.

Same names, fields and values as ``lucid/quantization/_qscheme.py:25-245``:
``quint8`` is stored in ``int16`` and ``qint4`` unpacked in ``int8``, as there.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass


class QScheme(enum.Enum):
    PER_TENSOR_AFFINE = "per_tensor_affine"
    PER_TENSOR_SYMMETRIC = "per_tensor_symmetric"
    PER_CHANNEL_AFFINE = "per_channel_affine"
    PER_CHANNEL_SYMMETRIC = "per_channel_symmetric"

    @property
    def is_per_channel(self) -> bool:
        return self.value.startswith("per_channel")

    @property
    def is_symmetric(self) -> bool:
        return self.value.endswith("symmetric")


per_tensor_affine = QScheme.PER_TENSOR_AFFINE
per_tensor_symmetric = QScheme.PER_TENSOR_SYMMETRIC
per_channel_affine = QScheme.PER_CHANNEL_AFFINE
per_channel_symmetric = QScheme.PER_CHANNEL_SYMMETRIC


@dataclass(frozen=True)
class QDtype:
    """An integer grid: bit width, signedness, inclusive code range, storage dtype name."""

    name: str
    bits: int
    signed: bool
    quant_min: int
    quant_max: int
    storage: str

    def __repr__(self) -> str:
        return f"lucid.quantization.{self.name}"


qint8 = QDtype("qint8", 8, True, -128, 127, "int8")
quint8 = QDtype("quint8", 8, False, 0, 255, "int16")
qint32 = QDtype("qint32", 32, True, -(2**31), 2**31 - 1, "int32")
qint4 = QDtype("qint4", 4, True, -8, 7, "int8")
