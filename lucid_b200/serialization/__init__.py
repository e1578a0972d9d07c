"""Checkpoint I/O for quantized ``state_dict``s in the SafeTensors format, written the way the
reference writes it (``lucid/serialization/__init__.py:833-921``, ``_safetensors.py:29-135``) so
that files travel both ways: insertion-ordered tensors, a JSON header padded with spaces to a
multiple of 8 bytes, zero-rank tensors stored with shape ``(1,)`` and listed in the metadata
entry ``__lucid_scalar_keys__`` (a JSON list; a comma-joined list in older files), unsigned
integer tensors widened on load to the next signed width (``U8 -> int16``, ``U16 -> int32``,
``U32`` / ``U64 -> int64``).  The packed words of the group-wise format are uint32 bit patterns
carried in ``int32`` tensors (``lucid/_C/ops/quantized/QuantizedMatmul.cpp:60-66``) and are
stored as ``I32``, so their bits survive the round trip unchanged.

``save`` / ``load`` write and read ``.safetensors`` paths with the functions above; other
paths use ``torch.save`` / ``torch.load(weights_only=True)`` (the reference's ``.lucid`` pickle
stream is tied to its tensor engine and is not reproduced)."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

_ST_CODES = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.bool: "BOOL",
    torch.complex64: "C64",
}
_ST_TORCH = {code: dt for dt, code in _ST_CODES.items()}
# stored unsigned width -> (numpy type it is stored as, signed torch type it widens to)
_ST_UNSIGNED = {"U8": (np.uint8, torch.int16), "U16": (np.uint16, torch.int32), "U32": (np.uint32, torch.int64),
                "U64": (np.uint64, torch.int64)}
_ITEMSIZE = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "BOOL": 1, "C64": 8,
             "U8": 1, "U16": 2, "U32": 4, "U64": 8}
_METADATA_KEY = "__metadata__"
SCALAR_KEYS_KEY = "__lucid_scalar_keys__"
_INT64_MAX = 2**63 - 1


def _decode_scalar_keys(text: str) -> frozenset[str]:
    try:
        parsed = json.loads(text)
    except ValueError:
        parsed = None
    if isinstance(parsed, list) and all(isinstance(k, str) for k in parsed):
        return frozenset(parsed)
    return frozenset(k for k in text.split(",") if k)


def _host_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.dtype is torch.bfloat16:
        t = t.view(torch.int16)
    elif t.dtype is torch.complex64:
        t = torch.view_as_real(t).contiguous()
    return t.numpy().tobytes()


def save_safetensors(state_dict, path, metadata=None) -> None:
    """Write a flat ``name -> Tensor`` mapping; ``metadata`` maps strings to strings."""
    meta: dict[str, str] = {}
    for key, value in (metadata or {}).items():
        if not isinstance(value, str):
            raise TypeError(f"save_safetensors: metadata maps strings to strings, got {key!r}: {value!r}")
        meta[key] = value
    if SCALAR_KEYS_KEY in meta:
        raise ValueError(f"save_safetensors: metadata key {SCALAR_KEYS_KEY!r} is reserved")
    header: dict[str, object] = {}
    blobs: list[bytes] = []
    scalar_keys: list[str] = []
    offset = 0
    for name, value in state_dict.items():
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"save_safetensors: state_dict[{name!r}] is {type(value).__name__}, expected Tensor")
        code = _ST_CODES.get(value.dtype)
        if code is None:
            raise TypeError(f"save_safetensors: tensor {name!r} has dtype {value.dtype}, which SafeTensors cannot store")
        shape = [int(d) for d in value.shape]
        if not shape:
            shape = [1]  # readers without zero-rank support still load it; tagged below
            scalar_keys.append(name)
        blob = _host_bytes(value)
        header[name] = {"dtype": code, "shape": shape, "data_offsets": [offset, offset + len(blob)]}
        blobs.append(blob)
        offset += len(blob)
    if scalar_keys:
        meta[SCALAR_KEYS_KEY] = json.dumps(scalar_keys, separators=(",", ":"))
    if meta:
        header[_METADATA_KEY] = meta
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)  # the data section starts 8-aligned
    with open(os.fspath(path), "wb") as fh:
        fh.write(struct.pack("<Q", len(encoded)))
        fh.write(encoded)
        for blob in blobs:
            fh.write(blob)


class safe_open:  # noqa: N801 - the reference's (and the format's) name
    """Lazy reader: ``keys()``, ``get_tensor(name)``, ``metadata()``; a context manager."""

    def __init__(self, path, device="cpu") -> None:
        self._path = os.fspath(path)
        self._device = device
        with open(self._path, "rb") as fh:
            raw = fh.read(8)
            if len(raw) != 8:
                raise ValueError(f"{self._path}: not a SafeTensors file (shorter than its length prefix)")
            (n,) = struct.unpack("<Q", raw)
            size = os.path.getsize(self._path)
            if n > size - 8:
                raise ValueError(f"{self._path}: header length {n} exceeds the file")
            header = json.loads(fh.read(n).decode("utf-8"))
        if not isinstance(header, dict):
            raise ValueError(f"{self._path}: the header is not a JSON object")
        self._data_start = 8 + n
        self._data_size = size - self._data_start
        meta = header.pop(_METADATA_KEY, None) or {}
        self._scalars = _decode_scalar_keys(meta.pop(SCALAR_KEYS_KEY, "")) if isinstance(meta, dict) else frozenset()
        self._metadata = dict(meta) if meta else None
        self._entries = header
        for name, e in header.items():
            code, shape, (start, end) = e["dtype"], e["shape"], e["data_offsets"]
            if code not in _ITEMSIZE:
                raise TypeError(f"{self._path}: tensor {name!r} has dtype {code}, which this build does not hold")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if not (0 <= start <= end <= self._data_size) or end - start != count * _ITEMSIZE[code]:
                raise ValueError(f"{self._path}: tensor {name!r} has inconsistent offsets or shape")

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        return None

    def keys(self):
        return list(self._entries)

    def metadata(self):
        return None if self._metadata is None else dict(self._metadata)

    def get_tensor(self, name: str) -> torch.Tensor:
        e = self._entries[name]
        code, shape, (start, end) = e["dtype"], list(e["shape"]), e["data_offsets"]
        with open(self._path, "rb") as fh:
            fh.seek(self._data_start + start)
            raw = fh.read(end - start)
        if code in _ST_UNSIGNED:
            np_t, torch_t = _ST_UNSIGNED[code]
            arr = np.frombuffer(raw, dtype=np_t)
            if code == "U64" and arr.size and int(arr.max()) > _INT64_MAX:
                raise OverflowError(f"{self._path}: tensor {name!r} holds a U64 value above int64's range")
            t = torch.from_numpy(arr.astype(np.int64)).to(torch_t)
        elif code == "BF16":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.int16).copy()).view(torch.bfloat16)
        elif code == "C64":
            t = torch.view_as_complex(torch.from_numpy(np.frombuffer(raw, dtype=np.float32).copy()).reshape(-1, 2))
        elif code == "BOOL":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).copy()).to(torch.bool)
        else:
            np_t = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32,
                    "I16": np.int16, "I8": np.int8}[code]
            t = torch.from_numpy(np.frombuffer(raw, dtype=np_t).copy())
        t = t.reshape(shape)
        if name in self._scalars and shape == [1]:
            t = t.reshape(())
        return t.to(self._device) if self._device not in (None, "cpu") else t


def load_safetensors(path, device="cpu") -> dict[str, torch.Tensor]:
    """All tensors of a SafeTensors file, in file order."""
    with safe_open(path, device=device) as f:
        return {name: f.get_tensor(name) for name in f.keys()}


def save(obj, f, **kwargs) -> None:
    if isinstance(f, (str, os.PathLike)) and os.fspath(f).endswith(".safetensors"):
        return save_safetensors(obj, f)
    return torch.save(obj, f, **kwargs)


def load(f, map_location=None, *, weights_only: bool = True, **kwargs):
    if isinstance(f, (str, os.PathLike)) and os.fspath(f).endswith(".safetensors"):
        return load_safetensors(f, device=map_location or "cpu")
    return torch.load(f, map_location=map_location, weights_only=weights_only, **kwargs)


__all__ = ["save", "load", "save_safetensors", "load_safetensors", "safe_open", "SCALAR_KEYS_KEY"]
