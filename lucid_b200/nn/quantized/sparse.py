"""Quantized embedding tables (API and buffers of ``lucid/nn/quantized/sparse.py:28-337``):
an int8 ``[num_embeddings, embedding_dim]`` table with one scale / zero-point per row.  The
reference dequantizes the whole table on every forward and gathers from the float copy; here
the lookup kernel reads only the rows the indices name, as int8, and decodes them on the way
out (``lc_embedding_s8_f32`` / ``lc_embedding_bag_s8_f32``) -- same values, a fraction of the
traffic.  Out-of-range indices read as rows of zeros (the reference's host-side refusal
would cost a device-to-host read per forward)."""
from __future__ import annotations

import torch
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized._utils import quantize_weight
from lucid_b200.quantization._functional import quantize
from lucid_b200.quantization._qscheme import per_channel_symmetric, qint8
from lucid_b200.quantization.observer import PerChannelMinMaxObserver


def _quantize_table(mod: nn.Module):
    """Per-row int8 codes of ``mod.weight``: the module's own qconfig when it has one, else
    the symmetric per-row default (``sparse.py:146-170``)."""
    if getattr(mod, "qconfig", None) is not None:
        codes, scale, zero_point, _ = quantize_weight(mod)
        return codes, scale, zero_point
    weight = _backend.on_cuda(mod.weight.detach())
    obs = PerChannelMinMaxObserver(ch_axis=0, qscheme=per_channel_symmetric, qdtype=qint8)
    obs(weight)
    scale, zero_point = obs.calculate_qparams()
    return quantize(weight, scale, zero_point, qint8, ch_axis=0), scale, zero_point


class _QuantizedTable(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None) -> None:
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.padding_idx = padding_idx
        self.weight_ch_axis = 0
        self.register_buffer("weight_int8", torch.zeros((num_embeddings, embedding_dim), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(num_embeddings))
        self.register_buffer("weight_zero_point", torch.zeros(num_embeddings))

    def _table(self):
        return (_backend.on_cuda(self.weight_int8), _backend.on_cuda(self.weight_scale),
                _backend.on_cuda(self.weight_zero_point))

    def _status_word(self, device) -> torch.Tensor:
        """Device int32 the lookup kernels set to 1 when they meet an index outside the table (the
        row they write for it is all zeros; the table is never read out of bounds).  Kept across
        forwards and read only by :meth:`check_indices`, so the forward itself never waits for the GPU."""
        word = self.__dict__.get("_index_status")
        if word is None or word.device != device:
            word = torch.zeros(1, dtype=torch.int32, device=device)
            self.__dict__["_index_status"] = word
        return word

    def check_indices(self) -> None:
        """Raise ``IndexError`` if any forward since the last check saw an index outside
        ``[0, num_embeddings)`` (the reference refuses such an index at once, on the host,
        ``lucid/_C/backend/cpu/IndexBounds.h:89-93``); synchronises the device and clears the record.
        With ``validate = True`` every forward ends with this check."""
        word = self.__dict__.get("_index_status")
        if word is not None and int(word.item()) != 0:
            word.zero_()
            raise IndexError(f"{type(self).__name__}: an index outside [0, {self.num_embeddings}) was looked up "
                             "(its output rows are zeros)")

    validate = False

    def _fill(self, mod: nn.Module) -> None:
        codes, scale, zero_point = _quantize_table(mod)
        self.register_buffer("weight_int8", codes)
        self.register_buffer("weight_scale", scale)
        self.register_buffer("weight_zero_point", zero_point)


class Embedding(_QuantizedTable):
    """``forward(indices)`` -> ``indices.shape + (embedding_dim,)`` fp32 rows
    (``sparse.py:140-143``); ``padding_idx`` only matters to a gradient and is kept as an
    attribute."""

    def forward(self, indices: torch.Tensor) -> torch.Tensor:
        if indices.is_floating_point():
            raise TypeError("quantized.Embedding: indices must be an integer tensor")
        table, scale, zero_point = self._table()
        out = _backend.ops().embedding_s8(table, scale, zero_point, _backend.on_cuda(indices),
                                          status=self._status_word(table.device))
        if self.validate:
            self.check_indices()
        return out if indices.is_cuda else out.to(indices.device)

    @classmethod
    def from_float(cls, mod: nn.Module) -> "Embedding":
        qmod = cls(mod.num_embeddings, mod.embedding_dim, padding_idx=mod.padding_idx)
        qmod._fill(mod)
        return qmod

    def extra_repr(self) -> str:
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}"


class EmbeddingBag(_QuantizedTable):
    """Pooled lookups (``sparse.py:284-304``): 1-D ``indices`` with ``offsets`` naming where each
    bag starts, or 2-D ``indices`` with one bag per row; ``mode`` sum / mean / max;
    ``per_sample_weights`` with sum only; entries equal to ``padding_idx`` are left out."""

    def __init__(self, num_embeddings: int, embedding_dim: int, mode: str = "mean",
                 padding_idx: int | None = None, include_last_offset: bool = False) -> None:
        super().__init__(num_embeddings, embedding_dim, padding_idx)
        if mode not in ("sum", "mean", "max"):
            raise ValueError(f"quantized.EmbeddingBag: mode must be sum / mean / max, got {mode!r}")
        self.mode = mode
        self.include_last_offset = include_last_offset

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor | None = None,
                per_sample_weights: torch.Tensor | None = None,
                compressed_indices_mapping: torch.Tensor | None = None) -> torch.Tensor:
        if compressed_indices_mapping is not None:
            raise NotImplementedError("quantized.EmbeddingBag: compressed_indices_mapping is not supported")
        idx = _backend.on_cuda(indices)
        include_last = self.include_last_offset
        if idx.dim() == 2:
            if offsets is not None:
                raise ValueError("quantized.EmbeddingBag: offsets must be None for 2-D indices")
            rows, width = idx.shape
            off = torch.arange(0, rows * width, width, dtype=torch.int64, device=idx.device)
            include_last = False
        elif idx.dim() == 1:
            if offsets is None:
                raise ValueError("quantized.EmbeddingBag: offsets required for 1-D input")
            off = _backend.on_cuda(offsets)
        else:
            raise ValueError(f"quantized.EmbeddingBag: indices must be 1-D or 2-D, got {idx.dim()}-D")
        psw = None if per_sample_weights is None else _backend.on_cuda(per_sample_weights).reshape(-1)
        table, scale, zero_point = self._table()
        out = _backend.ops().embedding_bag_s8(table, scale, zero_point, idx.reshape(-1), off, self.mode,
                                              self.padding_idx, psw, include_last,
                                              status=self._status_word(table.device))
        if self.validate:
            self.check_indices()
        return out if indices.is_cuda else out.to(indices.device)

    @classmethod
    def from_float(cls, mod: nn.Module) -> "EmbeddingBag":
        qmod = cls(mod.num_embeddings, mod.embedding_dim, mode=getattr(mod, "mode", "mean"),
                   padding_idx=getattr(mod, "padding_idx", None),
                   include_last_offset=bool(getattr(mod, "include_last_offset", False)))
        qmod._fill(mod)
        return qmod

    def extra_repr(self) -> str:
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}, mode={self.mode}"
