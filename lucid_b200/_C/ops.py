"""torch-tensor front end of the C ABI: allocates outputs with torch, passes raw
device pointers and the current CUDA stream to liblucid_cuda.

PyTorch is used here for device memory and streams only; all arithmetic on the
quantized path happens in the library's kernels.  Every function requires CUDA
tensors and raises otherwise -- there is no CPU fallback.
"""
from __future__ import annotations

import math

import torch

from ._loader import (LC_BF16, LC_F16, LC_F32, LC_QLINEAR_MULTICAST_OUT, LC_QLINEAR_WAIT_TEST, LC_S8, LC_S16, LC_S32, LC_U8, LucidCudaError, check,
                      entry, lib)

_dynamic_linear_f32 = entry("dynamic_linear_f32")
_group_matmul_ex = entry("group_matmul_ex")
_wo_linear_s8_ex = entry("wo_linear_s8_ex")
_wo_swiglu_s8_ex = entry("wo_swiglu_s8_ex")

_DTYPE = {
    torch.float32: LC_F32,
    torch.bfloat16: LC_BF16,
    torch.float16: LC_F16,
    torch.int8: LC_S8,
    torch.uint8: LC_U8,
    torch.int16: LC_S16,
    torch.int32: LC_S32,
}


def _lc_dtype(dt: torch.dtype) -> int:
    try:
        return _DTYPE[dt]
    except KeyError:
        raise TypeError(f"dtype {dt} is not supported by liblucid_cuda") from None


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "liblucid_cuda kernels take CUDA tensors only (there is no CPU fallback); "
                f"got a tensor on {t.device}"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(dev: torch.device):
    """Context that makes ``dev`` current for the launch; free when it already is."""
    if dev.index is None or dev.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(dev)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(dev: torch.device) -> int:
    """The current stream of ``dev`` as a raw ``cudaStream_t`` value (the binding's direct query
    when it has one: building a ``torch.cuda.Stream`` object per launch costs several
    microseconds of host time)."""
    if _raw_stream is not None:
        return _raw_stream(dev.index if dev.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(dev).cuda_stream


def capture_id(dev: torch.device) -> int:
    """0 outside CUDA-graph capture, else the id of the capture the current stream records into."""
    import ctypes

    out = ctypes.c_uint64(0)
    with _on(dev):
        check(lib.lc_stream_capture_id(_stream(dev), ctypes.byref(out)))
    return int(out.value)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _f32c(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.float32:
        t = t.to(torch.float32)
    return t.contiguous()


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}


def observe_workspace(dev: torch.device) -> torch.Tensor:
    """Zero-filled scratch for the global-range kernels, one per (device, stream):
    calls on the same stream are ordered, so they can share it."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream(dev))
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(int(lib.lc_observe_tensor_workspace_bytes()), dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = ws
    return ws


_HIST_WORKSPACES: dict[tuple[int, int, int], torch.Tensor] = {}


def histc(x: torch.Tensor, bins: int, lo: float, hi: float, out: torch.Tensor | None = None,
          accumulate: bool = False) -> torch.Tensor:
    """fp32 counts of ``x`` in ``bins`` equal-width bins over the finite range ``lo < hi``
    (float64 bucketing, NaN and out-of-range values skipped); ``accumulate`` adds to ``out``."""
    dev = _need_cuda(x, out)
    x = _f32c(x)
    if out is None:
        out = torch.empty(bins, dtype=torch.float32, device=dev)
        accumulate = False
    if out.dtype != torch.float32 or out.numel() != bins or not out.is_contiguous():
        raise TypeError("histc: out must be a contiguous fp32 tensor of `bins` elements")
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream(dev), int(bins))
    ws = _HIST_WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(int(lib.lc_histc_workspace_bytes(int(bins))), dtype=torch.uint8, device=dev)
        _HIST_WORKSPACES[key] = ws
    with _on(dev):
        check(lib.lc_histc_f32(x.data_ptr(), x.numel(), int(bins), float(lo), float(hi), out.data_ptr(),
                               int(accumulate), ws.data_ptr(), ws.numel(), _stream(dev)))
    return out


def channel_layout(shape, ch_axis: int | None) -> tuple[int, int, int]:
    """(outer, channels, inner) of a contiguous tensor split at ``ch_axis``."""
    if ch_axis is None:
        return 1, 1, math.prod(shape)
    ax = ch_axis % len(shape)
    return math.prod(shape[:ax]), shape[ax], math.prod(shape[ax + 1:])


# ----------------------------------------------------------------------------
# observers / qparams
# ----------------------------------------------------------------------------
def observe_tensor(x, min_out, max_out, accumulate: bool, qspec=None):
    """Global running min/max of ``x`` into the 0-d buffers ``min_out``/``max_out``.

    ``qspec = (symmetric, qmin, qmax, signed, eps)`` additionally returns the
    ``(scale, zero_point)`` of the merged range, computed in the same launch.
    """
    dev = _need_cuda(x, min_out, max_out)
    x = _f32c(x)
    scale = zp = None
    sym, qmin, qmax, signed, eps = (0, 0, 255, 0, 1e-8)
    if qspec is not None:
        sym, qmin, qmax, signed, eps = qspec
        scale = torch.empty((), dtype=torch.float32, device=dev)
        zp = torch.empty((), dtype=torch.float32, device=dev)
    ws = observe_workspace(dev)
    with _on(dev):
        check(lib.lc_observe_tensor_f32(x.data_ptr(), x.numel(), min_out.data_ptr(), max_out.data_ptr(),
                                        int(accumulate), int(sym), int(qmin), int(qmax), int(signed),
                                        float(eps), _ptr(scale), _ptr(zp), ws.data_ptr(), ws.numel(),
                                        _stream(dev)))
    return (scale, zp) if qspec is not None else None


def observe_channel(x, ch_axis: int, min_out, max_out, accumulate: bool) -> None:
    dev = _need_cuda(x, min_out, max_out)
    x = _f32c(x)
    outer, ch, inner = channel_layout(x.shape, ch_axis)
    if min_out.numel() != ch or max_out.numel() != ch:
        raise ValueError(f"running buffers hold {min_out.numel()} channels, input has {ch}")
    with _on(dev):
        check(lib.lc_observe_channel_f32(x.data_ptr(), outer, ch, inner, min_out.data_ptr(),
                                         max_out.data_ptr(), int(accumulate), _stream(dev)))


def calculate_qparams(min_t, max_t, symmetric: bool, qmin: int, qmax: int, signed: bool, eps: float):
    dev = _need_cuda(min_t, max_t)
    mn, mx = _f32c(min_t), _f32c(max_t)
    if mn.shape != mx.shape:
        mn, mx = torch.broadcast_tensors(mn, mx)
        mn, mx = mn.contiguous(), mx.contiguous()
    scale, zp = torch.empty_like(mn), torch.empty_like(mn)
    with _on(dev):
        check(lib.lc_calculate_qparams_f32(mn.data_ptr(), mx.data_ptr(), mn.numel(), int(symmetric),
                                           int(qmin), int(qmax), int(signed), float(eps),
                                           scale.data_ptr(), zp.data_ptr(), _stream(dev)))
    return scale, zp


# ----------------------------------------------------------------------------
# quantize / dequantize / fake_quantize
# ----------------------------------------------------------------------------
def _params(scale, zero_point, dev, channels: int, per_channel: bool):
    """Split (scale, zero_point) into device tensors and host scalars.

    A tensor scale is inverted on the device (fp32 IEEE division); a Python
    number is inverted here in double precision and rounded once to fp32 when
    ctypes narrows it, exactly as the reference's dispatcher does with
    ``1.0 / s`` for a Python float (``lucid/_dispatch.py:154-170``).
    """
    s_t = z_t = None
    h_inv = h_s = h_z = 0.0
    if isinstance(scale, torch.Tensor):
        s_t = _f32c(scale.to(dev)).reshape(-1)
        if s_t.numel() != 1 and not (per_channel and s_t.numel() == channels):
            raise ValueError(f"scale has {s_t.numel()} entries; expected 1 or {channels} along ch_axis")
    else:
        h_s = float(scale)
        h_inv = 1.0 / h_s
    if isinstance(zero_point, torch.Tensor):
        z_t = _f32c(zero_point.to(dev)).reshape(-1)
        if z_t.numel() != 1 and not (per_channel and z_t.numel() == channels):
            raise ValueError(f"zero_point has {z_t.numel()} entries; expected 1 or {channels}")
    else:
        h_z = float(zero_point)
    return s_t, z_t, h_inv, h_s, h_z


def quantize(x, scale, zero_point, qmin: int, qmax: int, storage: torch.dtype, ch_axis=None):
    dev = _need_cuda(x)
    x = _f32c(x)
    per_channel = ch_axis is not None and isinstance(scale, torch.Tensor) and scale.numel() > 1
    outer, ch, inner = channel_layout(x.shape, ch_axis if per_channel else None)
    s_t, z_t, h_inv, _, h_z = _params(scale, zero_point, dev, ch, per_channel)
    out = torch.empty(x.shape, dtype=storage, device=dev)
    with _on(dev):
        check(lib.lc_quantize_f32(x.data_ptr(), outer, ch, inner, _ptr(s_t), 0 if s_t is None else s_t.numel(),
                                  _ptr(z_t), 0 if z_t is None else z_t.numel(), h_inv, h_z, int(qmin),
                                  int(qmax), out.data_ptr(), _lc_dtype(storage), _stream(dev)))
    return out


def dequantize(q, scale, zero_point, ch_axis=None, out_dtype: torch.dtype = torch.float32):
    dev = _need_cuda(q)
    q = q.contiguous()
    per_channel = ch_axis is not None and isinstance(scale, torch.Tensor) and scale.numel() > 1
    outer, ch, inner = channel_layout(q.shape, ch_axis if per_channel else None)
    s_t, z_t, _, h_s, h_z = _params(scale, zero_point, dev, ch, per_channel)
    out = torch.empty(q.shape, dtype=out_dtype, device=dev)
    with _on(dev):
        check(lib.lc_dequantize(q.data_ptr(), _lc_dtype(q.dtype), outer, ch, inner, _ptr(s_t),
                                0 if s_t is None else s_t.numel(), _ptr(z_t),
                                0 if z_t is None else z_t.numel(), h_s, h_z, out.data_ptr(),
                                _lc_dtype(out_dtype), _stream(dev)))
    return out


def fake_quantize(x, scale, zero_point, qmin: int, qmax: int, ch_axis=None, want_mask: bool = False):
    dev = _need_cuda(x)
    x = _f32c(x)
    per_channel = ch_axis is not None and isinstance(scale, torch.Tensor) and scale.numel() > 1
    outer, ch, inner = channel_layout(x.shape, ch_axis if per_channel else None)
    s_t, z_t, h_inv, h_s, h_z = _params(scale, zero_point, dev, ch, per_channel)
    out = torch.empty_like(x)
    mask = torch.empty_like(x) if want_mask else None
    with _on(dev):
        check(lib.lc_fake_quantize_f32(x.data_ptr(), outer, ch, inner, _ptr(s_t),
                                       0 if s_t is None else s_t.numel(), _ptr(z_t),
                                       0 if z_t is None else z_t.numel(), h_inv, h_s, h_z, int(qmin),
                                       int(qmax), out.data_ptr(), _ptr(mask), _stream(dev)))
    return out, mask


_MERGE_OPS = {"add": 0, "mul": 1, "add_relu": 2}


def fake_quantize_merge(a, b, op: str, scale, zero_point, qmin: int, qmax: int):
    """``fake_quantize(a + b)`` / ``(a * b)`` / ``relu(a + b)`` on a per-tensor grid in one pass;
    ``b`` is a same-shape tensor or a Python scalar."""
    dev = _need_cuda(a, b if isinstance(b, torch.Tensor) else None)
    a = _f32c(a)
    scalar = 0.0
    if isinstance(b, torch.Tensor):
        if b.shape != a.shape:
            raise ValueError(f"fake_quantize_merge: shapes differ, {tuple(a.shape)} vs {tuple(b.shape)}")
        b = _f32c(b)
    else:
        scalar, b = float(b), None
    s_t, z_t, h_inv, h_s, h_z = _params(scale, zero_point, dev, 1, False)
    out = torch.empty_like(a)
    with _on(dev):
        check(lib.lc_fake_quantize_merge_f32(a.data_ptr(), _ptr(b), scalar, _MERGE_OPS[op], a.numel(), _ptr(s_t),
                                             _ptr(z_t), h_inv, h_s, h_z, int(qmin), int(qmax), out.data_ptr(),
                                             _stream(dev)))
    return out


# ----------------------------------------------------------------------------
# fused dynamic activation quantization
# ----------------------------------------------------------------------------
def _pad16(k: int) -> int:
    return (k + 15) // 16 * 16


def dynamic_quantize_rows(x2d, symmetric: bool, qmin: int, qmax: int, signed: bool, eps: float = 1e-8,
                          out_dtype: torch.dtype = torch.int8, pad_rows_to_16: bool = False):
    """Per-row observer + qparams + quantize in one pass.  Returns ``(q, scale, zp)``;
    with ``pad_rows_to_16`` the code matrix is a view into storage whose row stride
    is a multiple of 16 bytes (what the TMA-fed GEMM needs)."""
    dev = _need_cuda(x2d)
    x2d = _f32c(x2d)
    rows, cols = x2d.shape
    ldq = _pad16(cols) if pad_rows_to_16 else cols
    store = torch.empty((rows, ldq), dtype=out_dtype, device=dev)
    scale = torch.empty(rows, dtype=torch.float32, device=dev)
    zp = torch.empty(rows, dtype=torch.float32, device=dev)
    with _on(dev):
        check(lib.lc_dynamic_quantize_rows_f32(x2d.data_ptr(), rows, cols, cols, int(symmetric), int(qmin),
                                               int(qmax), int(signed), float(eps), store.data_ptr(),
                                               _lc_dtype(out_dtype), ldq, scale.data_ptr(), zp.data_ptr(),
                                               _stream(dev)))
    return store[:, :cols], scale, zp


def dynamic_quantize_tensor(x2d, symmetric: bool, qmin: int, qmax: int, signed: bool, eps: float = 1e-8,
                            out_dtype: torch.dtype = torch.uint8, pad_rows_to_16: bool = False):
    """Global range -> qparams -> quantize, everything staying on the device.
    Returns ``(q, scale, zp, minmax)`` with 0-d ``scale``/``zp`` and ``minmax = [min, max]``."""
    dev = _need_cuda(x2d)
    x2d = _f32c(x2d)
    rows, cols = x2d.shape
    ldq = _pad16(cols) if pad_rows_to_16 else cols
    store = torch.empty((rows, ldq), dtype=out_dtype, device=dev)
    scale = torch.empty((), dtype=torch.float32, device=dev)
    zp = torch.empty((), dtype=torch.float32, device=dev)
    minmax = torch.empty(2, dtype=torch.float32, device=dev)
    ws = observe_workspace(dev)
    with _on(dev):
        check(lib.lc_dynamic_quantize_tensor_f32(x2d.data_ptr(), rows, cols, cols, int(symmetric), int(qmin),
                                                 int(qmax), int(signed), float(eps), store.data_ptr(),
                                                 _lc_dtype(out_dtype), ldq, scale.data_ptr(), zp.data_ptr(),
                                                 minmax.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)))
    return store[:, :cols], scale, zp, minmax


# ----------------------------------------------------------------------------
# int8 GEMM
# ----------------------------------------------------------------------------
def pad_rows_to_16(codes: torch.Tensor) -> torch.Tensor:
    """[R, K] int8/uint8 codes -> a view [R, K] into storage with a 16-byte row pitch."""
    r, k = codes.shape
    if codes.stride(1) == 1 and codes.stride(0) % 16 == 0 and codes.data_ptr() % 16 == 0:
        return codes
    store = torch.zeros((r, _pad16(k)), dtype=codes.dtype, device=codes.device)
    store[:, :k] = codes
    return store[:, :k]


def rowsum_s8(b: torch.Tensor) -> torch.Tensor:
    dev = _need_cuda(b)
    if b.dtype != torch.int8 or b.dim() != 2 or b.stride(1) != 1:
        raise TypeError("rowsum_s8 expects a 2-D int8 matrix with unit column stride")
    out = torch.empty(b.shape[0], dtype=torch.int32, device=dev)
    with _on(dev):
        check(lib.lc_rowsum_s8(b.data_ptr(), b.shape[0], b.shape[1], b.stride(0), out.data_ptr(), _stream(dev)))
    return out


def qlinear_i8(a, b, sx, sw, bias=None, zx=None, wsum=None, out_dtype: torch.dtype = torch.float32,
               status: torch.Tensor | None = None, variant: int = 0):
    """``out = f32(a @ b^T - zx*wsum) * sx * sw + bias`` on the tcgen05 int8 path.

    ``a``: [M,K] int8 or uint8 codes, ``b``: [N,K] int8 codes, both with unit
    column stride and a 16-byte row pitch (see :func:`pad_rows_to_16`).
    ``sx``: 0-d / 1-element (per tensor) or [M] (per row) fp32.  With
    ``out_dtype=torch.int32`` the raw (zero-point corrected) accumulator is returned.
    ``variant``: 0 automatic, 1 single-CTA tiles, 2 CTA-pair tiles (``cta_group::2``).
    """
    dev = _need_cuda(a, b, sx, sw, bias, zx, wsum, status)
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"qlinear_i8: shapes {tuple(a.shape)} x {tuple(b.shape)}^T do not contract")
    if a.dtype not in (torch.int8, torch.uint8) or b.dtype != torch.int8:
        raise TypeError("qlinear_i8: a must be int8/uint8 and b int8")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("qlinear_i8: operands need unit column stride")
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=dev)
    per_row = 0
    if sx is not None:
        sx = _f32c(sx).reshape(-1)
        if sx.numel() == M and M != 1:
            per_row = 1
        elif sx.numel() != 1:
            raise ValueError(f"qlinear_i8: sx has {sx.numel()} entries, expected 1 or {M}")
    for name, t in (("sw", sw), ("bias", bias), ("wsum", wsum)):
        if t is not None and t.numel() != N:
            raise ValueError(f"qlinear_i8: {name} has {t.numel()} entries, expected {N}")
    sw_c = None if sw is None else _f32c(sw)
    bias_c = None if bias is None else _f32c(bias)
    zx_c = None if zx is None else _f32c(zx).reshape(-1)
    wsum_c = None if wsum is None else wsum.to(torch.int32).contiguous()
    with _on(dev):
        check(lib.lc_qlinear_i8_ex(a.data_ptr(), int(a.dtype == torch.uint8), a.stride(0), b.data_ptr(),
                                   b.stride(0), M, N, K, _ptr(sx), per_row, _ptr(zx_c), _ptr(wsum_c),
                                   _ptr(sw_c), _ptr(bias_c), out.data_ptr(), _lc_dtype(out_dtype), N,
                                   _ptr(status), int(variant), _stream(dev)))
    return out


_ACT_SCHEME_ID = {"tensor_affine": 0, "tensor_symmetric": 1, "token_symmetric": 2}


def dynamic_linear_workspace(rows: int, cols: int, dev: torch.device) -> torch.Tensor:
    """Uninitialised scratch for :func:`dynamic_linear` (codes, scales, range scratch) for inputs of up
    to ``rows`` x ``cols``; pass ``fresh=True`` with it once."""
    return torch.empty(int(lib.lc_dynamic_linear_workspace_bytes(rows, cols)), dtype=torch.uint8, device=dev)


def raw_stream(dev: torch.device) -> int:
    """The current stream of ``dev`` as the integer value of its ``cudaStream_t``."""
    return _stream(dev)


def dynamic_linear(x2d: torch.Tensor, act_scheme: str, qmin: int, qmax: int, signed: bool, wq: torch.Tensor, sw, bias,
                   wsum, workspace: torch.Tensor, fresh: bool, out_dtype: torch.dtype = torch.float32,
                   eps: float = 1e-8, status=None, stream: int | None = None) -> torch.Tensor:
    """Forward of the dynamic Linear from one library call: quantize the fp32 ``x2d`` on the grid
    ``act_scheme`` and run the int8 GEMM against ``wq`` (16-byte row pitch), ``sw``, ``bias``.
    Arguments are taken as they are (contiguous fp32 tensors on one device); this is the
    low-overhead path of :class:`lucid_b200.nn.quantized.dynamic.Linear`."""
    dev = x2d.device
    m, k = x2d.shape
    n = wq.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    check(_dynamic_linear_f32(x2d.data_ptr(), x2d.stride(0), m, k, _ACT_SCHEME_ID[act_scheme], int(qmin), int(qmax),
                                    1 if signed else 0, float(eps), wq.data_ptr(), wq.stride(0), n, _ptr(sw), _ptr(bias),
                                    _ptr(wsum), out.data_ptr(), _lc_dtype(out_dtype), n, workspace.data_ptr(),
                                    workspace.numel(), 1 if fresh else 0, _ptr(status),
                                    _stream(dev) if stream is None else stream))
    return out


def qlinear_i8_into(a, b, sx, sw, out_ptrs, ldo: int, out_dtype: torch.dtype = torch.float32, bias=None, zx=None,
                    wsum=None, status: torch.Tensor | None = None, variant: int = 0, multicast: bool = False) -> None:
    """:func:`qlinear_i8` writing each output tile to every buffer in ``out_ptrs`` (1..8 raw
    device addresses, row pitch ``ldo`` elements): the caller's own buffer and, for a
    column-parallel Linear, the same column slice of every peer GPU's result buffer, so the
    all-gather of the shards happens inside the GEMM's epilogue.  With ``multicast`` the single
    entry of ``out_ptrs`` is a multicast address: each tile leaves the GPU once (``multimem.st``)
    and the NVSwitch writes it into every GPU's buffer."""
    import ctypes

    dev = _need_cuda(a, b, sx, sw, bias, zx, wsum, status)
    M, K = a.shape
    N = b.shape[0]
    per_row = 0
    if sx is not None:
        sx = _f32c(sx).reshape(-1)
        per_row = 1 if (sx.numel() == M and M != 1) else 0
    sw_c = None if sw is None else _f32c(sw)
    bias_c = None if bias is None else _f32c(bias)
    zx_c = None if zx is None else _f32c(zx).reshape(-1)
    wsum_c = None if wsum is None else wsum.to(torch.int32).contiguous()
    arr = (ctypes.c_void_p * len(out_ptrs))(*[int(p) for p in out_ptrs])
    with _on(dev):
        check(lib.lc_qlinear_i8_multi(a.data_ptr(), int(a.dtype == torch.uint8), a.stride(0), b.data_ptr(),
                                      b.stride(0), M, N, K, _ptr(sx), per_row, _ptr(zx_c), _ptr(wsum_c),
                                      _ptr(sw_c), _ptr(bias_c), arr, len(out_ptrs), _lc_dtype(out_dtype),
                                      int(ldo), _ptr(status), int(variant) | (LC_QLINEAR_MULTICAST_OUT if multicast else 0),
                                      _stream(dev)))


def peer_barrier(flag_ptrs, rank: int, epoch: int, status: torch.Tensor | None = None,
                 wait_cycles: int = 2_000_000_000, device: torch.device | None = None) -> None:
    """Barrier between the ranks of one node on the current stream of ``device``: ``flag_ptrs[r]`` is
    the address, in this process, of rank r's flag array (one uint32 per rank, zero-filled once).
    ``epoch`` must grow with every call.  The device-side wait gives up after ``wait_cycles`` SM
    cycles (about a second by default) and records code 4 in ``status``."""
    import ctypes

    dev = device if device is not None else (status.device if status is not None else torch.device(
        "cuda", torch.cuda.current_device()))
    arr = (ctypes.c_void_p * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
    with _on(dev):
        check(lib.lc_peer_barrier(arr, int(rank), len(flag_ptrs), int(epoch) & 0xFFFFFFFF, int(wait_cycles), _ptr(status),
                                  _stream(dev)))


def copy_2d(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width_bytes: int, rows: int,
            device: torch.device) -> None:
    """``rows`` x ``width_bytes`` between two device buffers (either may belong to a peer GPU) on the
    copy engines, on the current stream of ``device``."""
    with _on(device):
        check(lib.lc_copy_2d_async(int(dst_ptr), int(dst_pitch), int(src_ptr), int(src_pitch), int(width_bytes), int(rows),
                                   _stream(device)))


def qlinear_check_status(status: torch.Tensor, clear: bool = True) -> None:
    """Synchronise the current stream and raise :class:`LucidCudaError` (code ``LC_ERR_TIMEOUT``)
    if a bounded device-side wait of a GEMM launch that was given ``status`` ran out."""
    dev = _need_cuda(status)
    with _on(dev):
        check(lib.lc_qlinear_check_status(status.data_ptr(), 1 if clear else 0, _stream(dev)))


# ----------------------------------------------------------------------------
# weight-only Linear on the tensor cores
# ----------------------------------------------------------------------------
def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def widen_s8(codes: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """int8 codes ``[N, K]`` as the same integers in ``dtype`` (bf16 / f16, exact), ``[N, Kp]`` with
    ``Kp`` = K rounded up to 64 and the padding zero: the weight operand of :func:`wo_gemm_16`."""
    dev = _need_cuda(codes)
    if codes.dtype != torch.int8 or codes.dim() != 2 or codes.stride(1) != 1:
        raise TypeError("widen_s8: expected a 2-D int8 tensor with unit column stride")
    n, k = codes.shape
    out = torch.empty((n, _round_up(k, 64)), dtype=dtype, device=dev)
    with _on(dev):
        check(lib.lc_widen_s8(codes.data_ptr(), n, k, codes.stride(0), out.data_ptr(), _lc_dtype(dtype), out.stride(0),
                              _stream(dev)))
    return out


def split_f32_bf16x3(x2d: torch.Tensor, want_rowsum: bool = False):
    """fp32 ``[M, K]`` -> ``(terms [M, 3 * Kp] bf16, rowsum [M] or None)``; the three terms of a
    row add up to the fp32 values exactly.  ``Kp`` = K rounded up to 64, padding zero."""
    dev = _need_cuda(x2d)
    if x2d.dtype != torch.float32 or x2d.dim() != 2:
        raise TypeError("split_f32_bf16x3: expected a 2-D fp32 tensor")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    m, k = x2d.shape
    kp = _round_up(k, 64)
    terms = torch.empty((m, 3 * kp), dtype=torch.bfloat16, device=dev)
    rowsum = torch.empty((m,), dtype=torch.float32, device=dev) if want_rowsum else None
    with _on(dev):
        check(lib.lc_split_f32_bf16x3(x2d.data_ptr(), m, k, x2d.stride(0), terms.data_ptr(), kp, _ptr(rowsum),
                                      _stream(dev)))
    return terms, rowsum


def split_f32_digits(x2d: torch.Tensor, want_rowsum: bool = False):
    """fp32 ``[M, K]`` -> ``(digits, row_scale [M], rowsum [M] or None)``: each row scaled by a power
    of two (``1 / row_scale``) into the 31-bit integer range and cut into four signed base-256
    digit planes, ``digits`` being the int8 ``[128 * ceil(M / 32), pad16(K)]`` operand of
    :func:`wo_gemm_digits` (plane d of row 32 t + r in row 128 t + 32 d + r)."""
    dev = _need_cuda(x2d)
    if x2d.dtype != torch.float32 or x2d.dim() != 2:
        raise TypeError("split_f32_digits: expected a 2-D fp32 tensor")
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    m, k = x2d.shape
    digits = torch.empty((int(lib.lc_wo_digit_rows(m)), _pad16(k)), dtype=torch.int8, device=dev)
    row_scale = torch.empty((m,), dtype=torch.float32, device=dev)
    rowsum = torch.empty((m,), dtype=torch.float32, device=dev) if want_rowsum else None
    with _on(dev):
        check(lib.lc_split_f32_digits(x2d.data_ptr(), m, k, x2d.stride(0), digits.data_ptr(), digits.stride(0),
                                      row_scale.data_ptr(), _ptr(rowsum), _stream(dev)))
    return digits, row_scale, rowsum


def wo_gemm_digits(digits: torch.Tensor, row_scale: torch.Tensor, wq: torch.Tensor, sw=None, bias=None, rowsum=None,
                   colcorr=None, relu: bool = False, out_scale=None, out_zp=None, quant_min: int = 0,
                   quant_max: int = 255, status=None, variant: int = 0, wait_test: bool = False):
    """Exact weight-only Linear for fp32 activations: ``digits`` / ``row_scale`` from
    :func:`split_f32_digits`, ``wq`` int8 codes ``[N, K]`` with a 16-byte row pitch.  Returns fp32
    ``requant(relu(sum * row_scale * sw + rowsum x colcorr + bias))``, the dot product being exact."""
    dev = _need_cuda(digits, row_scale, wq, sw, bias, rowsum, colcorr, out_scale, out_zp, status)
    if digits.dtype != torch.int8 or wq.dtype != torch.int8 or digits.stride(1) != 1 or wq.stride(1) != 1:
        raise TypeError("wo_gemm_digits: digits and wq must be int8 with unit column stride")
    m = row_scale.numel()
    n, k = wq.shape
    if digits.shape[0] != int(lib.lc_wo_digit_rows(m)) or digits.shape[1] < k:
        raise ValueError("wo_gemm_digits: digits do not belong to these rows / this K")
    out = torch.empty((m, n), dtype=torch.float32, device=dev)
    sw_c = None if sw is None else _f32c(sw)
    bias_c = None if bias is None else _f32c(bias)
    rs_c = None if rowsum is None else _f32c(rowsum)
    cc_c = None if colcorr is None else _f32c(colcorr)
    os_c = None if out_scale is None else _f32c(out_scale)
    oz_c = None if out_zp is None else _f32c(out_zp)
    with _on(dev):
        check(lib.lc_wo_gemm_digits(digits.data_ptr(), digits.stride(0), _f32c(row_scale).data_ptr(), wq.data_ptr(),
                                    wq.stride(0), m, n, k, _ptr(sw_c), _ptr(bias_c), _ptr(rs_c), _ptr(cc_c),
                                    1 if relu else 0, _ptr(os_c), _ptr(oz_c), int(quant_min), int(quant_max),
                                    out.data_ptr(), n, _ptr(status),
                                    int(variant) | (LC_QLINEAR_WAIT_TEST if wait_test else 0), _stream(dev)))
    return out


def wo_gemm_16(a: torch.Tensor, n_terms: int, w16: torch.Tensor, sw=None, bias=None, rowsum=None, colcorr=None,
               relu: bool = False, out_scale=None, out_zp=None, quant_min: int = 0, quant_max: int = 255,
               out_dtype: torch.dtype = torch.float32, status=None, variant: int = 0, wait_test: bool = False):
    """Tensor-core weight-only Linear: ``a`` holds ``n_terms`` addends of the activations side by
    side (``[M, n_terms * K]``, bf16, or f16 with one term), ``w16`` the widened codes ``[N, K]``.
    Returns ``requant(relu(acc * sw + rowsum x colcorr + bias))`` as ``[M, N]`` of ``out_dtype``;
    ``out_scale`` / ``out_zp`` are device scalars of the output grid (both or neither)."""
    dev = _need_cuda(a, w16, sw, bias, rowsum, colcorr, out_scale, out_zp, status)
    if a.dtype not in (torch.bfloat16, torch.float16) or w16.dtype != a.dtype:
        raise TypeError("wo_gemm_16: a and w16 must both be bf16 or both f16")
    if a.stride(1) != 1 or w16.stride(1) != 1:
        raise ValueError("wo_gemm_16: operands need unit column stride")
    m, ka = a.shape
    n, k = w16.shape
    if ka != n_terms * k:
        raise ValueError(f"wo_gemm_16: a has {ka} columns, expected {n_terms} x {k}")
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    sw_c = None if sw is None else _f32c(sw)
    bias_c = None if bias is None else _f32c(bias)
    rs_c = None if rowsum is None else _f32c(rowsum)
    cc_c = None if colcorr is None else _f32c(colcorr)
    os_c = None if out_scale is None else _f32c(out_scale)
    oz_c = None if out_zp is None else _f32c(out_zp)
    with _on(dev):
        check(lib.lc_wo_gemm_16(a.data_ptr(), _lc_dtype(a.dtype), n_terms, a.stride(0), w16.data_ptr(), w16.stride(0),
                                m, n, k, _ptr(sw_c), _ptr(bias_c), _ptr(rs_c), _ptr(cc_c), 1 if relu else 0,
                                _ptr(os_c), _ptr(oz_c), int(quant_min), int(quant_max), out.data_ptr(),
                                _lc_dtype(out_dtype), n, _ptr(status), int(variant) | (LC_QLINEAR_WAIT_TEST if wait_test else 0),
                                _stream(dev)))
    return out


# ----------------------------------------------------------------------------
# weight-only paths
# ----------------------------------------------------------------------------
_WO_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_WO_WORKSPACE_ROWS = 1 << 20  # tickets for weights of up to this many rows; larger ones run without scratch


def wo_workspace(dev: torch.device, rows: int):
    """Zero-filled scratch of the weight-streaming kernels' balanced schedule, one per (device,
    stream): launches on one stream are ordered, so they can share it.  ``None`` for weights with
    more rows than the scratch has tickets for (the kernel then hands out whole boxes)."""
    if rows > _WO_WORKSPACE_ROWS:
        return None
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream(dev))
    ws = _WO_WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(int(lib.lc_wo_linear_workspace_bytes(_WO_WORKSPACE_ROWS)), dtype=torch.uint8, device=dev)
        _WO_WORKSPACES[key] = ws
    return ws


def wo_linear_s8(x2d, wq, sw, bias=None, overlap_previous: bool = False, relu: bool = False, out_scale=None,
                 out_zp=None, quant_min: int = 0, quant_max: int = 255, balanced: bool = False):
    """``y = (x @ wq^T) * sw + bias`` with float activations; ``y`` has ``x``'s dtype.  With
    ``relu`` / ``out_scale`` and ``out_zp`` (device scalars) the same kernel goes on to apply the
    ReLU and the fake-quantize onto the calibrated output grid of a static Linear.

    ``overlap_previous`` lets the kernel start (and prefetch weights) while the kernel before
    it on the stream drains; the caller asserts that ``wq``, ``sw`` and ``bias`` were complete
    before that kernel started.  ``balanced`` gives the weight-streaming kernel its scratch, so that every
    SM streams the same number of bytes (K is cut between CTAs); by default whole 32-row boxes are dealt
    out, which measures faster on B200 for the decode shapes (the ticketed finish of the shared boxes
    costs more than the idle SMs it removes: decode MLP 53 us against 41 us)."""
    dev = _need_cuda(x2d, wq, sw, bias, out_scale, out_zp)
    if x2d.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError(f"wo_linear_s8: activations must be fp32/bf16/fp16, got {x2d.dtype}")
    x2d = x2d.contiguous()
    if wq.dtype != torch.int8 or wq.stride(1) != 1:
        raise TypeError("wo_linear_s8: weights must be int8 with unit column stride")
    B, K = x2d.shape
    N = wq.shape[0]
    if wq.shape[1] != K:
        raise ValueError(f"wo_linear_s8: in_features mismatch {wq.shape[1]} vs {K}")
    if (out_scale is None) != (out_zp is None):
        raise ValueError("wo_linear_s8: out_scale and out_zp go together")
    y = torch.empty((B, N), dtype=x2d.dtype, device=dev)
    sw_c = None if sw is None else _f32c(sw)
    bias_c = None if bias is None else _f32c(bias)
    os_c = None if out_scale is None else _f32c(out_scale)
    oz_c = None if out_zp is None else _f32c(out_zp)
    with _on(dev):
        ws = wo_workspace(dev, N) if balanced else None
        check(_wo_linear_s8_ex(x2d.data_ptr(), _lc_dtype(x2d.dtype), B, K, x2d.stride(0), wq.data_ptr(),
                                     wq.stride(0), N, _ptr(sw_c), _ptr(bias_c), 1 if relu else 0, _ptr(os_c),
                                     _ptr(oz_c), int(quant_min), int(quant_max), y.data_ptr(), N,
                                     1 if overlap_previous else 0, _ptr(ws), 0 if ws is None else ws.numel(),
                                     _stream(dev)))
    return y


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack two [F, ...] tensors (weights, scales or biases of the gate and up projections)
    into the [2F, ...] layout of :func:`wo_swiglu_s8`: blocks of 8 gate rows followed by the
    matching 8 up rows."""
    if gate.shape != up.shape or gate.shape[0] % 8:
        raise ValueError("gate and up must have the same shape with a multiple of 8 rows")
    f = gate.shape[0]
    g = gate.reshape(f // 8, 8, *gate.shape[1:])
    u = up.reshape(f // 8, 8, *up.shape[1:])
    return torch.cat([g, u], dim=1).reshape(2 * f, *gate.shape[1:]).contiguous()


def wo_swiglu_s8(x2d, wq_gu, sw_gu, bias_gu=None, overlap_previous: bool = False, balanced: bool = False):
    """``silu(x @ Wg^T * sg) * (x @ Wu^T * su)`` with interleaved int8 gate/up weights
    (see :func:`interleave_gate_up`); bf16 / f16 activations, batch <= 32.
    ``overlap_previous`` as for :func:`wo_linear_s8`."""
    dev = _need_cuda(x2d, wq_gu, sw_gu, bias_gu)
    x2d = x2d.contiguous()
    B, K = x2d.shape
    N2 = wq_gu.shape[0]
    y = torch.empty((B, N2 // 2), dtype=x2d.dtype, device=dev)
    sw_c = None if sw_gu is None else _f32c(sw_gu)
    bias_c = None if bias_gu is None else _f32c(bias_gu)
    with _on(dev):
        ws = wo_workspace(dev, N2) if balanced else None
        check(_wo_swiglu_s8_ex(x2d.data_ptr(), _lc_dtype(x2d.dtype), B, K, x2d.stride(0), wq_gu.data_ptr(),
                                     wq_gu.stride(0), N2, _ptr(sw_c), _ptr(bias_c), y.data_ptr(), N2 // 2,
                                     1 if overlap_previous else 0, _ptr(ws), 0 if ws is None else ws.numel(),
                                     _stream(dev)))
    return y


def wo_linear_status(clear: bool = True) -> int:
    """Status word of the weight-only kernels on the current device (synchronises): 0, or the
    code of a bounded device-side wait that ran out."""
    import ctypes

    code = ctypes.c_int32(0)
    check(lib.lc_wo_linear_status(ctypes.byref(code), int(clear)))
    return int(code.value)


def group_quantize(w, group_size: int = 64, bits: int = 8):
    dev = _need_cuda(w)
    if w.dim() != 2:
        raise ValueError("group_quantize expects a 2-D weight")
    w = _f32c(w)
    N, K = w.shape
    if bits not in (4, 8) or K % group_size != 0:
        raise ValueError(f"group_quantize: bits={bits}, group_size={group_size}, K={K} not supported")
    packed = torch.empty((N, K * bits // 32), dtype=torch.int32, device=dev)
    scales = torch.empty((N, K // group_size), dtype=torch.float32, device=dev)
    biases = torch.empty((N, K // group_size), dtype=torch.float32, device=dev)
    with _on(dev):
        check(lib.lc_group_quantize_f32(w.data_ptr(), N, K, group_size, bits, packed.data_ptr(),
                                        scales.data_ptr(), biases.data_ptr(), _stream(dev)))
    return packed, scales, biases


def group_dequantize(packed, scales, biases, group_size: int = 64, bits: int = 8):
    dev = _need_cuda(packed, scales, biases)
    packed = packed.contiguous()
    N = packed.shape[0]
    K = packed.shape[1] * 32 // bits
    out = torch.empty((N, K), dtype=torch.float32, device=dev)
    with _on(dev):
        check(lib.lc_group_dequantize(packed.data_ptr(), _f32c(scales).data_ptr(), _f32c(biases).data_ptr(),
                                      N, K, group_size, bits, out.data_ptr(), _stream(dev)))
    return out


LC_GROUP_OUT_F32 = 2


def group_fp32_rows_stream(dtype, rows: int, n: int, k: int, group_size: int, bits: int) -> bool:
    """Whether fp32 activations go through the streaming kernel as bf16 addends: packed weights of 4 MB and more
    in a layout that kernel takes.  The direct kernel's FP32 multiply-adds need 46 / 101 / 240 / 489 us for
    1 / 4 / 16 / 32 rows against ``[14336, 4096]`` 8-bit codes; the three-addend form 23 / 29 / 72 / 135 us."""
    return (dtype is torch.float32 and 0 < rows <= 32 and n * k * bits >= (32 << 20) and group_size in (64, 128)
            and k % (4 * group_size) == 0 and k >= 1024)


def group_matmul(x2d, packed, scales, biases, group_size: int = 64, bits: int = 8, overlap_previous: bool = False):
    """``y[b, n] = sum_k x[b, k] * (code[n, k] * scale[n, g] + bias[n, g])`` for the packed group-wise
    format; ``y`` has ``x``'s dtype.  Packed weights of 4 MB and more (8-bit or 4-bit codes in groups of 64 / 128,
    bf16 / f16 activations) are streamed once through shared memory; ``overlap_previous`` as for
    :func:`wo_linear_s8`."""
    dev = _need_cuda(x2d, packed, scales, biases)
    x2d = x2d.contiguous()
    if x2d.data_ptr() % 16:  # a contiguous view that starts inside a larger storage: the kernels load 16 bytes at a time
        x2d = x2d.clone()
    packed = packed.contiguous()
    B, K = x2d.shape
    N = packed.shape[0]
    if packed.shape[1] * 32 // bits != K:
        raise ValueError("group_matmul: packed weight does not match x's inner dimension")
    sc, bi = _f32c(scales), _f32c(biases)
    if group_fp32_rows_stream(x2d.dtype, B, N, K, group_size, bits):
        # fp32 activations against a large packed weight: every row as three bf16 rows that add up to it exactly
        # (rows 3 b .. 3 b + 2 of the [3 B, K] view), one pass of the streaming kernel with fp32 results, and the
        # three results of a row added up
        terms, _ = split_f32_bf16x3(x2d)
        y3 = torch.empty((3 * B, N), dtype=torch.float32, device=dev)
        with _on(dev):
            check(_group_matmul_ex(terms.data_ptr(), LC_BF16, 3 * B, K, packed.data_ptr(), sc.data_ptr(), bi.data_ptr(), N,
                                   group_size, bits, y3.data_ptr(), LC_GROUP_OUT_F32 | (1 if overlap_previous else 0),
                                   None, 0, _stream(dev)))
        return y3.view(B, 3, N).sum(1)
    y = torch.empty((B, N), dtype=x2d.dtype, device=dev)
    with _on(dev):
        ws = None  # whole boxes per CTA: measured faster than the K-cutting schedule
        check(_group_matmul_ex(x2d.data_ptr(), _lc_dtype(x2d.dtype), B, K, packed.data_ptr(), sc.data_ptr(),
                                     bi.data_ptr(), N, group_size, bits, y.data_ptr(), 1 if overlap_previous else 0,
                                     _ptr(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return y


def group_matmul_lean(x2d, packed, scales, biases, group_size: int, bits: int):
    """:func:`group_matmul` for callers that have already established what it checks: all four
    tensors live on the current CUDA device, are contiguous, ``scales`` / ``biases`` are fp32 and the
    shapes agree.  One allocation, one stream query, one library call: the decode-time dispatch path."""
    B, K = x2d.shape
    N = packed.shape[0]
    if x2d.data_ptr() % 16:
        x2d = x2d.clone()
    y = torch.empty((B, N), dtype=x2d.dtype, device=x2d.device)
    check(_group_matmul_ex(x2d.data_ptr(), _DTYPE[x2d.dtype], B, K, packed.data_ptr(), scales.data_ptr(),
                                 biases.data_ptr(), N, group_size, bits, y.data_ptr(), 0, None, 0,
                                 _stream(x2d.device)))
    return y


# ----------------------------------------------------------------------------
# int8 embedding tables
# ----------------------------------------------------------------------------
BAG_MODES = {"sum": 0, "mean": 1, "max": 2}


def _table_args(table, scale, zero_point):
    if table.dtype != torch.int8 or table.dim() != 2:
        raise TypeError("embedding: the table must be a 2-D int8 tensor")
    table = table.contiguous()
    sc = _f32c(scale).reshape(-1)
    if sc.numel() != table.shape[0]:
        raise ValueError("embedding: one scale per table row is required")
    zp = None if zero_point is None else _f32c(zero_point).reshape(-1)
    if zp is not None and zp.numel() != table.shape[0]:
        raise ValueError("embedding: one zero-point per table row is required")
    return table, sc, zp


def embedding_s8(table, scale, zero_point, indices, status=None):
    """fp32 rows ``(f32(table[i]) - zero_point[i]) * scale[i]`` for every ``i`` in ``indices``
    (any shape, integer dtype); result ``indices.shape + (D,)``.  ``status``: optional int32
    device scalar set to 1 when an index lies outside the table (that row reads as zeros)."""
    dev = _need_cuda(table, scale, indices)
    table, sc, zp = _table_args(table, scale, zero_point)
    idx = indices.to(torch.int64).contiguous()
    V, D = table.shape
    out = torch.empty(tuple(idx.shape) + (D,), dtype=torch.float32, device=dev)
    with _on(dev):
        check(lib.lc_embedding_s8_f32(table.data_ptr(), sc.data_ptr(), zp.data_ptr() if zp is not None else None,
                                      idx.data_ptr(), idx.numel(), V, D, out.data_ptr(),
                                      status.data_ptr() if status is not None else None, _stream(dev)))
    return out


def embedding_bag_s8(table, scale, zero_point, indices, offsets, mode: str = "mean", padding_idx=None,
                     per_sample_weights=None, include_last_offset: bool = False, status=None):
    """Pooled lookups: bag ``b`` covers ``indices[offsets[b]:offsets[b+1]]`` (1-D indices), rows
    decoded like :func:`embedding_s8` and reduced in index order; result ``[bags, D]`` fp32."""
    dev = _need_cuda(table, scale, indices, offsets)
    if mode not in BAG_MODES:
        raise ValueError(f"embedding_bag: mode must be one of {sorted(BAG_MODES)}, got {mode!r}")
    table, sc, zp = _table_args(table, scale, zero_point)
    idx = indices.to(torch.int64).contiguous().reshape(-1)
    off = offsets.to(torch.int64).contiguous().reshape(-1)
    psw = None
    if per_sample_weights is not None:
        if mode != "sum":
            raise ValueError("embedding_bag: per_sample_weights is only supported with mode='sum'")
        psw = _f32c(per_sample_weights).reshape(-1)
        if psw.numel() != idx.numel():
            raise ValueError("embedding_bag: per_sample_weights must have one weight per index")
    V, D = table.shape
    bags = off.numel() - 1 if include_last_offset else off.numel()
    out = torch.empty((max(bags, 0), D), dtype=torch.float32, device=dev)
    with _on(dev):
        check(lib.lc_embedding_bag_s8_f32(table.data_ptr(), sc.data_ptr(), zp.data_ptr() if zp is not None else None,
                                          idx.data_ptr(), idx.numel(), off.data_ptr(), off.numel(),
                                          psw.data_ptr() if psw is not None else None, V, D, BAG_MODES[mode],
                                          -1 if padding_idx is None else int(padding_idx), int(include_last_offset),
                                          out.data_ptr(), status.data_ptr() if status is not None else None,
                                          _stream(dev)))
    return out


__all__ = [n for n in dir() if not n.startswith("_")] + ["LucidCudaError"]
