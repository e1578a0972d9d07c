"""``FakeQuantize``: an observer plus a fake-quantize step, the building block of QAT
configs (API of ``lucid/quantization/_fake_quantize.py:33-245``)."""
from __future__ import annotations

import functools

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.quantization._functional import fake_quantize
from lucid_b200.quantization.observer import MovingAverageMinMaxObserver, ObserverBase


class FakeQuantize(nn.Module):
    def __init__(self, observer: type[ObserverBase] = MovingAverageMinMaxObserver, **observer_kwargs) -> None:
        super().__init__()
        self.activation_post_process = observer(**observer_kwargs)
        self.qdtype = self.activation_post_process.qdtype
        self.qscheme = self.activation_post_process.qscheme
        self.ch_axis = self.activation_post_process.ch_axis
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self._observer_enabled = True
        self._fake_quant_enabled = True

    def forward(self, x):
        if self._observer_enabled:
            with torch.no_grad():
                self.activation_post_process(x)
                scale, zero_point = self.activation_post_process.calculate_qparams()
                for name, value in (("scale", scale), ("zero_point", zero_point)):
                    buf = getattr(self, name)
                    if buf.shape == value.shape and buf.device == value.device:
                        buf.copy_(value)
                    else:
                        self.register_buffer(name, value.detach().clone())
        if self._fake_quant_enabled:
            scale = self.scale if self.scale.is_cuda else _backend.on_cuda(self.scale)
            return fake_quantize(x, scale, self.zero_point, self.qdtype.quant_min, self.qdtype.quant_max, self.ch_axis)
        return x

    def enable_observer(self, enabled: bool = True):
        self._observer_enabled = enabled
        return self

    def disable_observer(self):
        return self.enable_observer(False)

    def enable_fake_quant(self, enabled: bool = True):
        self._fake_quant_enabled = enabled
        return self

    def disable_fake_quant(self):
        return self.enable_fake_quant(False)

    def calculate_qparams(self):
        return self.activation_post_process.calculate_qparams()

    @classmethod
    def with_args(cls, **kwargs):
        return functools.partial(cls, **kwargs)
