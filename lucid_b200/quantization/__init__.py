"""``lucid.quantization`` on the CUDA backend: the reference's public names
(``lucid/quantization/__init__.py:74-125``) with the hot path on sm_100a kernels.

Graph mode (``prepare_fx`` / ``convert_fx``) is a tracing front end over the reference's own
graph capture; the names are exported for compatibility and raise ``NotImplementedError``.
"""
from lucid_b200.quantization import _qgemm, observer, qconfig  # noqa: F401
from lucid_b200.quantization._fake_quantize import FakeQuantize
from lucid_b200.quantization._functional import dequantize, fake_quantize, quantize
from lucid_b200.quantization._qparams import QParams, calculate_qparams
from lucid_b200.quantization._qscheme import (QDtype, QScheme, per_channel_affine, per_channel_symmetric,
                                              per_tensor_affine, per_tensor_symmetric, qint4, qint8, qint32,
                                              quint8)
from lucid_b200.quantization._quantize import convert, prepare, prepare_qat, quantize_dynamic
from lucid_b200.quantization.fuse_modules import fuse_modules, fuse_modules_qat
from lucid_b200.quantization.observer import (FixedQParamsObserver, HistogramObserver, MinMaxObserver,
                                              MovingAverageMinMaxObserver,
                                              MovingAveragePerChannelMinMaxObserver, NoopObserver, ObserverBase,
                                              PerChannelMinMaxObserver, PlaceholderObserver)
from lucid_b200.quantization.qconfig import (QConfig, QConfigMapping, get_default_qat_qconfig,
                                             get_default_qat_qconfig_mapping, get_default_qconfig,
                                             get_default_qconfig_mapping)


def _not_on_this_backend(name: str):
    def stub(*_args, **_kwargs):
        raise NotImplementedError(
            f"{name} is a tracing / training front end with no kernels; it is not part of the CUDA "
            "inference backend")

    stub.__name__ = name
    return stub


prepare_fx = _not_on_this_backend("prepare_fx")
convert_fx = _not_on_this_backend("convert_fx")

__all__ = [
    "QScheme", "per_tensor_affine", "per_tensor_symmetric", "per_channel_affine", "per_channel_symmetric",
    "QDtype", "qint8", "quint8", "qint32", "qint4",
    "QParams", "calculate_qparams",
    "quantize", "dequantize", "fake_quantize",
    "ObserverBase", "MinMaxObserver", "MovingAverageMinMaxObserver", "PerChannelMinMaxObserver",
    "MovingAveragePerChannelMinMaxObserver", "HistogramObserver", "FixedQParamsObserver",
    "PlaceholderObserver", "NoopObserver",
    "FakeQuantize",
    "QConfig", "QConfigMapping", "get_default_qconfig", "get_default_qat_qconfig",
    "get_default_qconfig_mapping", "get_default_qat_qconfig_mapping",
    "prepare", "convert", "fuse_modules", "fuse_modules_qat",
    "quantize_dynamic", "prepare_qat", "prepare_fx", "convert_fx",
]
