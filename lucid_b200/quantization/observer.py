"""Range observers (API of ``lucid/quantization/observer.py:91-1322``).

An observer is an identity module that records statistics of what flows through
it and turns them into ``(scale, zero_point)``.  The min/max reductions run in
the CUDA kernels ``lc_observe_tensor_f32`` / ``lc_observe_channel_f32``, which
merge straight into the running buffers (one pass over the data instead of the
reference's separate ``min`` and ``max`` passes); the statistics never visit the
host, so a calibration forward contains no synchronisation.  The histogram
observer is calibration-time only and stays on torch ops, as in the reference
its search runs in Python.
"""
from __future__ import annotations

import functools

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.quantization._qparams import calculate_qparams
from lucid_b200.quantization._qscheme import (QDtype, QScheme, per_channel_symmetric, per_tensor_affine, qint8,
                                              quint8)

_INF = float("inf")


class ObserverBase(nn.Module):
    """Common state: scheme, grid, channel axis (kept only for per-channel schemes), eps."""

    def __init__(self, qscheme: QScheme, qdtype: QDtype, ch_axis: int | None = None, eps: float = 1e-8) -> None:
        super().__init__()
        self.qscheme = qscheme
        self.qdtype = qdtype
        self.ch_axis = ch_axis if qscheme.is_per_channel else None
        self.eps = eps

    # -- running buffers ---------------------------------------------------------
    def _stat_shape(self, x: torch.Tensor) -> tuple[int, ...]:
        if self.ch_axis is not None and x.dim() > 0:
            return (x.shape[self.ch_axis],)
        return ()

    def _align_running_buffers(self, x: torch.Tensor) -> None:
        """Bring every local buffer to ``x``'s device; grow a scalar seed to one
        entry per channel the first time a per-channel observer sees data."""
        want = self._stat_shape(x)
        for name, buf in list(self.named_buffers(recurse=False)):
            shape = want if (want and buf.dim() == 0) else tuple(buf.shape)
            if buf.device != x.device or tuple(buf.shape) != shape:
                moved = buf.to(x.device)
                if tuple(moved.shape) != shape:
                    moved = moved.expand(shape).contiguous()
                self.register_buffer(name, moved)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        # a checkpoint of a calibrated per-channel observer holds (C,) statistics
        # while a fresh observer holds scalars: adopt the saved shape before loading
        for name, current in list(self.named_buffers(recurse=False)):
            saved = state_dict.get(prefix + name)
            if saved is not None and tuple(saved.shape) != tuple(current.shape):
                self.register_buffer(name, saved.detach().clone().to(current.device))
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    def _observed(self, x: torch.Tensor) -> torch.Tensor:
        xd = _backend.on_cuda(x.detach())
        if xd.dtype != torch.float32:
            xd = xd.float()
        self._align_running_buffers(xd)
        return xd

    def calculate_qparams(self):
        raise NotImplementedError

    @classmethod
    def with_args(cls, **kwargs):
        return functools.partial(cls, **kwargs)


class MinMaxObserver(ObserverBase):
    """Running global min / max, seeded with +inf / -inf."""

    def __init__(self, qscheme: QScheme = per_tensor_affine, qdtype: QDtype = quint8, eps: float = 1e-8) -> None:
        super().__init__(qscheme, qdtype, None, eps)
        self.register_buffer("min_val", torch.tensor(_INF))
        self.register_buffer("max_val", torch.tensor(-_INF))

    @torch.no_grad()
    def forward(self, x):
        xd = self._observed(x)
        if xd.numel():
            _backend.ops().observe_tensor(xd, self.min_val, self.max_val, accumulate=True)
        return x

    def calculate_qparams(self):
        return calculate_qparams(self.min_val, self.max_val, self.qscheme, self.qdtype, self.eps)


class MovingAverageMinMaxObserver(MinMaxObserver):
    """Exponential moving average of the per-batch min / max; the first batch seeds it."""

    def __init__(self, qscheme: QScheme = per_tensor_affine, qdtype: QDtype = quint8,
                 averaging_constant: float = 0.01, eps: float = 1e-8) -> None:
        super().__init__(qscheme, qdtype, eps)
        self.averaging_constant = averaging_constant

    @torch.no_grad()
    def forward(self, x):
        xd = self._observed(x)
        if not xd.numel():
            return x
        cur_min, cur_max = torch.empty_like(self.min_val), torch.empty_like(self.max_val)
        _backend.ops().observe_tensor(xd, cur_min, cur_max, accumulate=False)
        c = self.averaging_constant
        unseeded = torch.isinf(self.min_val)
        self.min_val.copy_(torch.where(unseeded, cur_min, self.min_val + c * (cur_min - self.min_val)))
        self.max_val.copy_(torch.where(unseeded, cur_max, self.max_val + c * (cur_max - self.max_val)))
        return x


class PerChannelMinMaxObserver(ObserverBase):
    """Running min / max per index of ``ch_axis``, reduced over every other axis."""

    def __init__(self, ch_axis: int = 0, qscheme: QScheme = per_channel_symmetric, qdtype: QDtype = qint8,
                 eps: float = 1e-8) -> None:
        super().__init__(qscheme, qdtype, ch_axis, eps)
        self.register_buffer("min_val", torch.tensor(_INF))
        self.register_buffer("max_val", torch.tensor(-_INF))

    def _axis(self) -> int:
        return self.ch_axis if self.ch_axis is not None else 0

    def _align_running_buffers(self, x):
        # a per-tensor scheme given to this class still tracks one range per channel
        saved, self.ch_axis = self.ch_axis, self._axis()
        try:
            super()._align_running_buffers(x)
        finally:
            self.ch_axis = saved

    @torch.no_grad()
    def forward(self, x):
        xd = self._observed(x)
        if xd.numel():
            _backend.ops().observe_channel(xd, self._axis(), self.min_val, self.max_val, accumulate=True)
        return x

    def calculate_qparams(self):
        return calculate_qparams(self.min_val, self.max_val, self.qscheme, self.qdtype, self.eps)


class MovingAveragePerChannelMinMaxObserver(PerChannelMinMaxObserver):
    def __init__(self, ch_axis: int = 0, qscheme: QScheme = per_channel_symmetric, qdtype: QDtype = qint8,
                 averaging_constant: float = 0.01, eps: float = 1e-8) -> None:
        super().__init__(ch_axis, qscheme, qdtype, eps)
        self.averaging_constant = averaging_constant

    @torch.no_grad()
    def forward(self, x):
        xd = self._observed(x)
        if not xd.numel():
            return x
        cur_min, cur_max = torch.empty_like(self.min_val), torch.empty_like(self.max_val)
        _backend.ops().observe_channel(xd, self._axis(), cur_min, cur_max, accumulate=False)
        c = self.averaging_constant
        # the reference seeds when *every* channel is still unseeded
        unseeded = torch.isinf(self.min_val).all()
        self.min_val.copy_(torch.where(unseeded, cur_min, self.min_val + c * (cur_min - self.min_val)))
        self.max_val.copy_(torch.where(unseeded, cur_max, self.max_val + c * (cur_max - self.max_val)))
        return x


class HistogramObserver(ObserverBase):
    """Histogram of the activations plus a clip-range search that minimises the
    expected squared quantization error over a few candidate tail fractions."""

    _TAILS = (0.0, 1e-5, 1e-4, 1e-3, 5e-3, 1e-2)

    def __init__(self, bins: int = 2048, qscheme: QScheme = per_tensor_affine, qdtype: QDtype = quint8,
                 eps: float = 1e-8) -> None:
        super().__init__(qscheme, qdtype, None, eps)
        self.bins = bins
        self.register_buffer("min_val", torch.tensor(_INF))
        self.register_buffer("max_val", torch.tensor(-_INF))
        self.register_buffer("histogram", torch.zeros(bins))

    def _rebin(self, hist, old_lo, old_hi, new_lo, new_hi):
        """Move every old bin's mass to the new bin that contains its centre."""
        old_w, new_w = (old_hi - old_lo) / self.bins, (new_hi - new_lo) / self.bins
        centres = old_lo + (torch.arange(self.bins, device=hist.device, dtype=torch.float32) + 0.5) * old_w
        dst = torch.clip((centres - new_lo) / new_w, 0.0, float(self.bins - 1)).to(torch.int64)
        return torch.zeros(self.bins, device=hist.device).scatter_add(0, dst, hist)

    def _count(self, xd, lo: float, hi: float):
        """``lucid.histc(x, bins, lo, hi)`` of the batch (``observer.py:861,864`` in the reference)."""
        if lo == hi:  # the adapter's single-point convention
            lo, hi = lo - 1.0, hi + 1.0
        return _backend.ops().histc(xd.reshape(-1), self.bins, lo, hi)

    @torch.no_grad()
    def forward(self, x):
        xd = self._observed(x)
        if not xd.numel():
            return x
        # the running range decides the bins, so it is read back (a sanctioned host round trip,
        # lucid/quantization/observer.py:855-856); one fused min/max pass instead of two
        mn = torch.empty((), dtype=torch.float32, device=xd.device)
        mx = torch.empty((), dtype=torch.float32, device=xd.device)
        _backend.ops().observe_tensor(xd, mn, mx, accumulate=False)
        lo, hi = float(mn), float(mx)
        old_lo, old_hi = float(self.min_val), float(self.max_val)
        if old_lo == _INF:
            new_lo, new_hi = lo, hi
            hist = self._count(xd, new_lo, new_hi)
        else:
            new_lo, new_hi = min(old_lo, lo), max(old_hi, hi)
            hist = self._count(xd, new_lo, new_hi)
            if (new_lo, new_hi) == (old_lo, old_hi):
                hist = hist + self.histogram
            else:
                hist = hist + self._rebin(self.histogram, old_lo, old_hi, new_lo, new_hi)
        self.min_val.fill_(new_lo)
        self.max_val.fill_(new_hi)
        self.histogram.copy_(hist)
        return x

    def _search_clip_range(self) -> tuple[float, float]:
        lo, hi = float(self.min_val), float(self.max_val)
        counts = self.histogram.double().cpu()
        total = float(counts.sum())
        if total <= 0.0 or hi <= lo:
            return lo, hi
        width = (hi - lo) / self.bins
        centres = lo + (torch.arange(self.bins, dtype=torch.float64) + 0.5) * width
        cum = torch.cumsum(counts, 0)
        levels = max(self.qdtype.quant_max - self.qdtype.quant_min, 1)

        def quantile(q: float) -> float:
            idx = int(torch.searchsorted(cum, torch.tensor(q * total, dtype=torch.float64)))
            return float(centres[min(idx, self.bins - 1)])

        best_err, best = _INF, (lo, hi)
        for tail in self._TAILS:
            cmin, cmax = quantile(tail), quantile(1.0 - tail)
            if cmax <= cmin:
                continue
            step = (cmax - cmin) / levels
            clipped = centres.clamp(cmin, cmax)
            err = float((counts * ((centres - clipped) ** 2 + step * step / 12.0))[counts > 0].sum())
            if err < best_err:
                best_err, best = err, (cmin, cmax)
        return best

    def calculate_qparams(self):
        lo, hi = self._search_clip_range()
        return calculate_qparams(float(lo), float(hi), self.qscheme, self.qdtype, self.eps)


class FixedQParamsObserver(ObserverBase):
    """Returns the qparams it was built with (for outputs of known range, e.g. sigmoid)."""

    def __init__(self, scale: float, zero_point: int, qscheme: QScheme = per_tensor_affine,
                 qdtype: QDtype = quint8, eps: float = 1e-8) -> None:
        super().__init__(qscheme, qdtype, None, eps)
        self.register_buffer("scale", torch.tensor(float(scale)))
        self.register_buffer("zero_point", torch.tensor(float(zero_point)))

    def forward(self, x):
        return x

    def calculate_qparams(self):
        return self.scale, self.zero_point


class PlaceholderObserver(ObserverBase):
    """Marks a tensor whose qparams are computed at run time (dynamic quantization)."""

    def __init__(self, qscheme: QScheme = per_tensor_affine, qdtype: QDtype = quint8, eps: float = 1e-8) -> None:
        super().__init__(qscheme, qdtype, None, eps)

    def forward(self, x):
        return x

    def calculate_qparams(self):
        raise RuntimeError(
            f"{type(self).__name__} collects no statistics; qparams are computed at runtime "
            "(dynamic quantization) or supplied elsewhere."
        )


class NoopObserver(PlaceholderObserver):
    pass
