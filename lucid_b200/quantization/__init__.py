"""``lucid.quantization`` on the CUDA backend: the reference's public names
(``lucid/quantization/__init__.py:74-125``) with the hot path on sm_100a kernels.

Graph mode (``prepare_fx`` / ``convert_fx``) wraps the model in its quantization boundaries and
runs the eager flow underneath, as the reference's does.
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


def prepare_fx(model, qconfig_mapping=None, example_inputs=None, inplace: bool = False):
    """Graph-mode entry of static PTQ (``lucid/quantization/_quantize_fx.py:30-109``): no hand-placed
    stubs -- the model is wrapped in a :class:`~lucid_b200.nn.quantized.QuantWrapper` (input quantized,
    output dequantized) and then prepared like the eager flow.  Calibrate the result, then
    :func:`convert_fx`.  ``example_inputs`` is accepted for signature compatibility; nothing is traced
    (the reference reaches graph mode by compiling the converted module-level composites, and a model
    converted here is captured whole by ``lucid_b200.cuda.make_graphed``)."""
    import copy

    from lucid_b200.nn.quantized import QuantWrapper

    del example_inputs
    return prepare(QuantWrapper(model if inplace else copy.deepcopy(model)), qconfig_mapping, inplace=True)


def convert_fx(model, inplace: bool = False):
    """Graph-mode convert (``_quantize_fx.py:112-170``): the eager :func:`convert` of a model that
    :func:`prepare_fx` produced."""
    return convert(model, inplace=inplace)


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
