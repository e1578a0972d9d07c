"""Dynamically quantized recurrent layers: ``LSTM``, ``GRU`` and the cells
(``lucid/nn/quantized/dynamic/rnn.py:45-264``).  The weight matrices are stored as int8 with
per-row symmetric scales, biases stay float; a float module of the same kind (the *shell*,
kept out of the module registry so that its weights never reach ``state_dict``) runs the
recurrence after its weights have been overwritten with the dequantized values, which is one
``lc_dequantize`` launch per matrix and forward.  Activations inside the cell are not
quantized, as in the reference."""
from __future__ import annotations

import copy

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import ieee_fp32
from lucid_b200.quantization._functional import dequantize, quantize
from lucid_b200.quantization._qscheme import QDtype, per_channel_symmetric, qint8


def _buffer_key(name: str) -> str:
    """Flat buffer name of shell parameter ``name`` (a buffer name cannot hold a dot):
    ``cell_l0.weight_ih`` -> ``weight_ih_l0``; torch's recurrent modules already use flat names."""
    owner, _, leaf = name.rpartition(".")
    return f"{leaf}_{owner.removeprefix('cell_')}" if owner else leaf


def _is_weight(name: str) -> bool:
    return name.rpartition(".")[2].startswith("weight")


class _DynamicRecurrent(nn.Module):
    _FLOAT: type = nn.Module

    def __init__(self, shell: nn.Module) -> None:
        super().__init__()
        object.__setattr__(self, "_shell", shell)
        named = [n for n, _ in shell.named_parameters()]
        self._weight_names = [(n, _buffer_key(n)) for n in named if _is_weight(n)]
        self._bias_names = [(n, _buffer_key(n)) for n in named if not _is_weight(n)]

    def _buffer(self, key: str) -> torch.Tensor:
        value = self._buffers[key]
        if value is None:
            raise RuntimeError(f"{type(self).__name__}: buffer '{key}' is unset")
        return value

    @torch.no_grad()
    def _loaded(self) -> nn.Module:
        """The shell with its weights replaced by the dequantized int8 buffers.  The values are
        written into the shell's own parameter storage, which keeps the fused weight layout of
        the recurrent kernels intact."""
        shell = object.__getattribute__(self, "_shell")
        first = self._buffer(self._weight_names[0][1] + "_int8")
        dev = first.device if first.is_cuda else _backend.cuda_device()
        if next(shell.parameters()).device != dev:
            shell.to(dev)
        if getattr(self, "_flat_for", None) != id(shell):  # a moved or deep-copied shell lost its fused layout
            if dev.type == "cuda" and hasattr(shell, "flatten_parameters"):
                shell.flatten_parameters()
            object.__setattr__(self, "_flat_for", id(shell))
        for path, key in self._weight_names:
            deq = dequantize(self._buffer(key + "_int8"), self._buffer(key + "_scale"), 0.0, ch_axis=0)
            shell.get_parameter(path).copy_(deq)
        for path, key in self._bias_names:
            shell.get_parameter(path).copy_(self._buffer(key))
        return shell

    @classmethod
    def from_float(cls, mod: nn.Module, dtype: QDtype = qint8):
        from lucid_b200.quantization.observer import PerChannelMinMaxObserver

        if not isinstance(mod, cls._FLOAT):
            raise TypeError(f"dynamic {cls.__name__}.from_float expects an nn.{cls._FLOAT.__name__}, "
                            f"got {type(mod).__name__}")
        shell = copy.deepcopy(mod).requires_grad_(False)  # the caller's float module stays as given
        qmod = cls(shell)
        for name, param in shell.named_parameters():
            key = _buffer_key(name)
            if _is_weight(name):
                obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=dtype)
                w = _backend.on_cuda(param.detach().float())
                obs(w)
                scale, zero_point = obs.calculate_qparams()
                qmod.register_buffer(key + "_int8", quantize(w, scale, zero_point, dtype, ch_axis=0))
                qmod.register_buffer(key + "_scale", scale)
            else:
                qmod.register_buffer(key, _backend.on_cuda(param.detach().float()).clone())
        return qmod

    def _run(self, x, *rest):
        if isinstance(x, torch.Tensor):
            xd = _backend.on_cuda(x)
            rest = tuple(None if r is None else (tuple(_backend.on_cuda(t) for t in r) if isinstance(r, tuple)
                                                  else _backend.on_cuda(r)) for r in rest)
            with ieee_fp32():
                return self._loaded()(xd, *rest)
        with ieee_fp32():
            return self._loaded()(x, *rest)  # a PackedSequence goes straight to the shell

    def extra_repr(self) -> str:
        return f"{object.__getattribute__(self, '_shell').extra_repr()}, dynamic=True"


class LSTM(_DynamicRecurrent):
    _FLOAT = nn.LSTM

    def forward(self, input, hx=None):  # noqa: A002 - the reference's argument name
        return self._run(input, hx)


class GRU(_DynamicRecurrent):
    _FLOAT = nn.GRU

    def forward(self, input, hx=None):  # noqa: A002
        return self._run(input, hx)


class LSTMCell(_DynamicRecurrent):
    _FLOAT = nn.LSTMCell

    def forward(self, input, hx=None):  # noqa: A002
        return self._run(input, hx)


class GRUCell(_DynamicRecurrent):
    _FLOAT = nn.GRUCell

    def forward(self, input, hx=None):  # noqa: A002
        return self._run(input, hx)


class RNNCell(_DynamicRecurrent):
    _FLOAT = nn.RNNCell

    def forward(self, input, hx=None):  # noqa: A002
        return self._run(input, hx)
