"""TEST INFRASTRUCTURE: an oracle-backed stand-in for ``lucid_b200._C.ops`` working on
CPU tensors, so that the host-side logic (module swapping, buffer handling, routing) can
be exercised without a GPU.  Installed only by tests through
``lucid_b200._backend._set_ops_for_testing``; the product never imports this file."""
import numpy as np
import torch

from oracle import oracle as O


def _np(t):
    return t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t


def _qd(qmin, qmax, storage="int8", signed=None):
    return O.QDtype("q", 8, qmin < 0 if signed is None else signed, qmin, qmax, storage)


_STORE = {torch.int8: "int8", torch.uint8: "uint8", torch.int16: "int16", torch.int32: "int32"}


def capture_id(dev):
    return 0


def fake_quantize_merge(a, b, op, scale, zero_point, qmin, qmax):
    an = _np(a.float())
    bn = _np(b.float()) if isinstance(b, torch.Tensor) else np.float32(b)
    t = (an * bn if op == "mul" else an + bn).astype(np.float32)
    if op == "add_relu":
        t = np.where(t < 0, np.float32(0), t)
    s = _np(scale) if isinstance(scale, torch.Tensor) else float(scale)
    z = _np(zero_point) if isinstance(zero_point, torch.Tensor) else float(zero_point)
    return torch.tensor(O.fake_quantize(t, s, z, qmin, qmax)[0])


def histc(x, bins, lo, hi, out=None, accumulate=False):
    h = torch.tensor(O.histc(_np(x.float()), bins, lo, hi))
    if out is None:
        return h
    out.copy_(out + h if accumulate else h)
    return out


def observe_tensor(x, min_out, max_out, accumulate, qspec=None):
    mn, mx = O.minmax_tensor(_np(x))
    if accumulate:
        mn, mx = min(mn, float(min_out)), max(mx, float(max_out))
    min_out.fill_(float(mn))
    max_out.fill_(float(mx))
    if qspec is not None:
        sym, qmin, qmax, signed, eps = qspec
        s, z = O.calculate_qparams(mn, mx, sym, _qd(qmin, qmax, signed=signed), eps)
        return torch.tensor(float(s)), torch.tensor(float(z))
    return None


def observe_channel(x, ch_axis, min_out, max_out, accumulate):
    mn, mx = O.minmax_channel(_np(x), ch_axis)
    if accumulate:
        mn, mx = np.minimum(mn, _np(min_out)), np.maximum(mx, _np(max_out))
    min_out.copy_(torch.tensor(mn))
    max_out.copy_(torch.tensor(mx))


def calculate_qparams(min_t, max_t, symmetric, qmin, qmax, signed, eps):
    s, z = O.calculate_qparams(_np(min_t), _np(max_t), symmetric, _qd(qmin, qmax, signed=signed), eps)
    return torch.tensor(s), torch.tensor(z)


def _p(v):
    return _np(v).reshape(-1) if isinstance(v, torch.Tensor) and v.numel() > 1 else (
        np.float32(_np(v)).reshape(()) if isinstance(v, torch.Tensor) else v)


def quantize(x, scale, zero_point, qmin, qmax, storage, ch_axis=None):
    q = O.quantize(_np(x), _p(scale), _p(zero_point), _qd(qmin, qmax, _STORE[storage]), ch_axis)
    return torch.tensor(q)


def dequantize(q, scale, zero_point, ch_axis=None, out_dtype=torch.float32):
    return torch.tensor(O.dequantize(_np(q), _p(scale), _p(zero_point), ch_axis)).to(out_dtype)


def fake_quantize(x, scale, zero_point, qmin, qmax, ch_axis=None, want_mask=False):
    dq, mask = O.fake_quantize(_np(x), _p(scale), _p(zero_point), qmin, qmax, ch_axis)
    return torch.tensor(dq), (torch.tensor(mask) if want_mask else None)


def dynamic_quantize_rows(x2d, symmetric, qmin, qmax, signed, eps=1e-8, out_dtype=torch.int8, pad_rows_to_16=False):
    x = _np(x2d)
    qd = _qd(qmin, qmax, _STORE[out_dtype], signed)
    s, z = O.calculate_qparams(*O.minmax_channel(x, 0), symmetric, qd, eps)
    return torch.tensor(O.quantize(x, s, z, qd, ch_axis=0)), torch.tensor(s), torch.tensor(z)


def dynamic_quantize_tensor(x2d, symmetric, qmin, qmax, signed, eps=1e-8, out_dtype=torch.uint8, pad_rows_to_16=False):
    x = _np(x2d)
    qd = _qd(qmin, qmax, _STORE[out_dtype], signed)
    mn, mx = O.minmax_tensor(x)
    s, z = O.calculate_qparams(mn, mx, symmetric, qd, eps)
    return (torch.tensor(O.quantize(x, s, z, qd)), torch.tensor(float(s)), torch.tensor(float(z)),
            torch.tensor([float(mn), float(mx)]))


def pad_rows_to_16(codes):
    return codes


def rowsum_s8(b):
    return b.to(torch.int32).sum(1, dtype=torch.int32)


def qlinear_i8(a, b, sx, sw, bias=None, zx=None, wsum=None, out_dtype=torch.float32, status=None):
    acc = O.int_gemm_exact(_np(a), _np(b)).astype(np.int64)
    if zx is not None:
        acc = acc - int(float(zx)) * _np(wsum).astype(np.int64)[None, :]
    if out_dtype == torch.int32:
        return torch.tensor(acc.astype(np.int32))
    sxv = _np(sx).astype(np.float64).reshape(-1)
    y = acc.astype(np.float64) * (sxv[:, None] if sxv.size > 1 else sxv[0])
    if sw is not None:
        y = y * _np(sw).astype(np.float64)[None, :]
    if bias is not None:
        y = y + _np(bias).astype(np.float64)[None, :]
    return torch.tensor(y.astype(np.float32)).to(out_dtype)


def _finish(y, relu, out_scale, out_zp, quant_min, quant_max):
    y = y.astype(np.float32)
    if relu:
        y = np.where(y < 0, np.float32(0), y)
    if out_scale is not None:
        y = O.fake_quantize(y, _p(out_scale), _p(out_zp), quant_min, quant_max)[0]
    return y


def wo_linear_s8(x2d, wq, sw, bias=None, overlap_previous=False, relu=False, out_scale=None, out_zp=None,
                 quant_min=0, quant_max=255, balanced=False):
    y = O.weight_only_linear_perchannel(_np(x2d.float()), _np(wq), _np(sw), None if bias is None else _np(bias))
    return torch.tensor(_finish(y, relu, out_scale, out_zp, quant_min, quant_max)).to(x2d.dtype)


def widen_s8(codes, dtype=torch.bfloat16):
    n, k = codes.shape
    out = torch.zeros((n, (k + 63) // 64 * 64), dtype=dtype)
    out[:, :k] = codes.to(dtype)
    return out


def split_f32_bf16x3(x2d, want_rowsum=False):
    m, k = x2d.shape
    kp = (k + 63) // 64 * 64
    terms = torch.zeros((m, 3 * kp), dtype=torch.bfloat16)
    rest = x2d.float()
    for t in range(3):
        part = rest.to(torch.bfloat16)
        terms[:, t * kp:t * kp + k] = part
        rest = rest - part.float()
    return terms, (x2d.float().sum(1) if want_rowsum else None)


def split_f32_digits(x2d, want_rowsum=False):
    """Stand-in: the 'digits' are the fp32 rows themselves (the host logic only passes them on)."""
    return x2d.float(), torch.ones(x2d.shape[0]), (x2d.float().sum(1) if want_rowsum else None)


def wo_gemm_digits(digits, row_scale, wq, sw=None, bias=None, rowsum=None, colcorr=None, relu=False, out_scale=None,
                   out_zp=None, quant_min=0, quant_max=255, status=None, variant=0, wait_test=False):
    y = _np(digits).astype(np.float64) @ _np(wq).astype(np.float64).T
    if sw is not None:
        y = y * _np(sw).astype(np.float64)[None, :]
    if rowsum is not None:
        y = y + _np(rowsum).astype(np.float64)[:, None] * _np(colcorr).astype(np.float64)[None, :]
    if bias is not None:
        y = y + _np(bias).astype(np.float64)[None, :]
    return torch.tensor(_finish(y, relu, out_scale, out_zp, quant_min, quant_max))


def wo_gemm_16(a, n_terms, w16, sw=None, bias=None, rowsum=None, colcorr=None, relu=False, out_scale=None,
               out_zp=None, quant_min=0, quant_max=255, out_dtype=torch.float32, status=None, variant=0,
               wait_test=False):
    k = w16.shape[1]
    x = sum(_np(a[:, t * k:(t + 1) * k].float()).astype(np.float64) for t in range(n_terms))
    y = x @ _np(w16.float()).astype(np.float64).T
    if sw is not None:
        y = y * _np(sw).astype(np.float64)[None, :]
    if rowsum is not None:
        y = y + _np(rowsum).astype(np.float64)[:, None] * _np(colcorr).astype(np.float64)[None, :]
    if bias is not None:
        y = y + _np(bias).astype(np.float64)[None, :]
    return torch.tensor(_finish(y, relu, out_scale, out_zp, quant_min, quant_max)).to(out_dtype)


def group_quantize(w, group_size=64, bits=8):
    p, s, b = O.group_quantize(_np(w), group_size, bits)
    return torch.tensor(p), torch.tensor(s), torch.tensor(b)


def group_dequantize(packed, scales, biases, group_size=64, bits=8):
    return torch.tensor(O.group_dequantize(_np(packed), _np(scales), _np(biases), group_size, bits))


def group_matmul(x2d, packed, scales, biases, group_size=64, bits=8, overlap_previous=False):
    y = O.group_matmul(_np(x2d.float()), _np(packed), _np(scales), _np(biases), group_size, bits)
    return torch.tensor(y).to(x2d.dtype)


def embedding_s8(table, scale, zero_point, indices, status=None):
    z = np.zeros(table.shape[0], np.float32) if zero_point is None else _np(zero_point)
    return torch.tensor(O.embedding_s8(_np(table), _np(scale), z, _np(indices)))


def embedding_bag_s8(table, scale, zero_point, indices, offsets, mode="mean", padding_idx=None,
                     per_sample_weights=None, include_last_offset=False, status=None):
    z = np.zeros(table.shape[0], np.float32) if zero_point is None else _np(zero_point)
    psw = None if per_sample_weights is None else _np(per_sample_weights)
    return torch.tensor(O.embedding_bag_s8(_np(table), _np(scale), z, _np(indices), _np(offsets), mode, padding_idx,
                                           psw, include_last_offset))
