"""GPU parity of the tcgen05 int8 Linear: int32 accumulator bit-exact against the
exact integer GEMM oracle, fp32 outputs within rtol 1e-5 of the float64 epilogue."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
RTOL, ATOL = 1e-5, 1e-6  # fp32 output tolerance stated for this path


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


def dev(a):
    return torch.tensor(np.ascontiguousarray(a), device="cuda")


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def status_word():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("M,N,K", [(1, 1, 16), (128, 256, 128), (128, 256, 512), (64, 4096, 1024), (7, 9, 48),
                                   (129, 257, 144), (300, 520, 1040), (256, 512, 8192), (1000, 130, 80), (5, 6, 24), (33, 40, 200)])
@pytest.mark.parametrize("a_unsigned", [False, True])
@pytest.mark.parametrize("variant", [1, 2])
def test_int32_accumulator_bit_exact(ops, M, N, K, a_unsigned, variant):
    r = np.random.default_rng(M * 7 + N * 3 + K)
    a = r.integers(0, 256, (M, K)).astype(np.uint8) if a_unsigned else r.integers(-128, 128, (M, K)).astype(np.int8)
    b = r.integers(-128, 128, (N, K)).astype(np.int8)
    st = status_word()
    acc = ops.qlinear_i8(ops.pad_rows_to_16(dev(a)), ops.pad_rows_to_16(dev(b)), None, None,
                         out_dtype=torch.int32, status=st, variant=variant)
    np.testing.assert_array_equal(host(acc), O.int_gemm_exact(a, b))
    assert int(host(st)[0]) == 0


def test_extreme_codes_do_not_overflow(ops):
    M, N, K = 128, 256, 8192
    a = np.full((M, K), 255, np.uint8)
    b = np.full((N, K), -128, np.int8)
    acc = ops.qlinear_i8(dev(a), dev(b), None, None, out_dtype=torch.int32)
    assert (host(acc) == 255 * -128 * K).all()


@pytest.mark.parametrize("mode,qd", [("tensor_affine", "quint8"), ("tensor_symmetric", "qint8"),
                                     ("token_symmetric", "qint8")])
def test_golden_dynamic_linear(ops, mode, qd):
    g = np.load(os.path.join(GOLDEN, "linear_golden.npz"))
    qdt = getattr(O, qd)
    x = dev(g["x"])
    wq = ops.pad_rows_to_16(dev(g["wq"]))
    if mode == "token_symmetric":
        xq, sx, zx = ops.dynamic_quantize_rows(x, True, qdt.quant_min, qdt.quant_max, True, 1e-8, torch.int8,
                                               pad_rows_to_16=True)
        zx_arg = wsum = None
    else:
        sym = mode == "tensor_symmetric"
        xq, sx, zx, _ = ops.dynamic_quantize_tensor(x, sym, qdt.quant_min, qdt.quant_max, qdt.signed, 1e-8,
                                                    torch.int8 if sym else torch.uint8, pad_rows_to_16=True)
        zx_arg = None if sym else zx
        wsum = None if sym else ops.rowsum_s8(wq)
    np.testing.assert_array_equal(host(xq).astype(np.int32), g[f"xq_{mode}"].astype(np.int32))
    np.testing.assert_array_equal(host(sx).reshape(-1), g[f"sx_{mode}"].reshape(-1))
    acc = ops.qlinear_i8(xq, wq, None, None, zx=zx_arg, wsum=wsum, out_dtype=torch.int32)
    np.testing.assert_array_equal(host(acc), g[f"acc_{mode}"])
    y = ops.qlinear_i8(xq, wq, sx, dev(g["sw"]), bias=dev(g["b"]), zx=zx_arg, wsum=wsum)
    np.testing.assert_allclose(host(y), g[f"y_{mode}"], rtol=RTOL, atol=ATOL)
    if mode == "tensor_affine":  # the reference's own float formulation, looser: fp32 summation order
        np.testing.assert_allclose(host(y), g["y_reference_float"], rtol=2e-4, atol=2e-5)
    yb = ops.qlinear_i8(xq, wq, sx, dev(g["sw"]), bias=dev(g["b"]), zx=zx_arg, wsum=wsum, out_dtype=torch.bfloat16)
    np.testing.assert_allclose(host(yb.float()), g[f"y_{mode}"], rtol=1e-2, atol=1e-3)


def test_config1_single_dynamic_linear(ops):
    """x [64,1024], W [4096,1024], per-tensor symmetric narrow-range int8 activations
    (scale = absmax/127, clamp [-127,127]), per-channel weights, fp32 bias."""
    x, w, b = O.synth_config1()
    qd = O.qint8_narrow
    mn, mx = O.minmax_channel(w, 0)
    sw, zw = O.calculate_qparams(mn, mx, True, qd)
    wq = O.quantize(w, sw, zw, qd, ch_axis=0)
    acc_o, y_o, xq_o, sx_o, _ = O.dynamic_linear_int(x, wq, sw, b, "tensor_symmetric", qd)
    xq, sx, zx, _ = ops.dynamic_quantize_tensor(dev(x), True, -127, 127, True, 1e-8, torch.int8)
    np.testing.assert_array_equal(host(xq), xq_o)
    assert float(host(sx)) == float(sx_o)
    wq_t = dev(wq)
    acc = ops.qlinear_i8(xq, wq_t, None, None, out_dtype=torch.int32)
    np.testing.assert_array_equal(host(acc), acc_o)
    y = ops.qlinear_i8(xq, wq_t, sx, dev(sw), bias=dev(b))
    np.testing.assert_allclose(host(y), y_o, rtol=RTOL, atol=ATOL)


def test_prefill_shape_properties(ops):
    """A slice of the prefill workload (K = 8192, per-token scales): bit-exact on a
    sample of rows/columns, linearity and column-shard independence on the whole."""
    M, N, K = 2048, 3584, 8192
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.02
    wq, sw, _ = ops.dynamic_quantize_rows(w, True, -128, 127, True)
    xq, sx, _ = ops.dynamic_quantize_rows(x, True, -128, 127, True)
    st = status_word()
    acc = ops.qlinear_i8(xq, wq, None, None, out_dtype=torch.int32, status=st)
    assert int(host(st)[0]) == 0
    rows = [0, 1, 127, 128, 1000, 2047]
    cols = [0, 255, 256, 1791, 1792, 3583]
    ref = O.int_gemm_exact(host(xq[rows]), host(wq[cols]))
    np.testing.assert_array_equal(host(acc[rows][:, cols]), ref)
    # checksum of checksums: sum_n acc[m,n] == xq[m,:] . sum_n wq[n,:]
    colsum = wq.to(torch.int64).sum(0)
    expect = (xq.to(torch.float64) @ colsum.to(torch.float64)).to(torch.int64)
    assert torch.equal(acc.to(torch.int64).sum(1), expect)
    # sharding over N (column-parallel) reproduces the same columns bit for bit
    shard = ops.qlinear_i8(xq, wq[1792:], None, None, out_dtype=torch.int32)
    assert torch.equal(shard, acc[:, 1792:])
    # single-CTA and CTA-pair tiles give the same accumulator
    for variant in (1, 2):
        assert torch.equal(ops.qlinear_i8(xq, wq, None, None, out_dtype=torch.int32, variant=variant), acc)
    y = ops.qlinear_i8(xq, wq, sx, sw)
    y64 = acc.to(torch.float64) * sx.to(torch.float64)[:, None] * sw.to(torch.float64)[None, :]
    assert torch.allclose(y.to(torch.float64), y64, rtol=RTOL, atol=ATOL)


def test_multi_destination_epilogue(ops):
    """The epilogue can write each tile to several buffers (the fused all-gather form): two
    column slices of two wider result buffers receive exactly the single-buffer result."""
    M, N, K = 300, 200, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-128, 128, (M, K), device="cuda", dtype=torch.int8, generator=g)
    b = torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
    sx = torch.rand(M, device="cuda", generator=g)
    sw = torch.rand(N, device="cuda", generator=g)
    ref = ops.qlinear_i8(a, b, sx, sw)
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        want = ops.qlinear_i8(a, b, sx, sw, out_dtype=dtype) if dtype != torch.int32 else ops.qlinear_i8(
            a, b, None, None, out_dtype=dtype)
        full0 = torch.zeros((M, 3 * N), dtype=dtype, device="cuda")
        full1 = torch.zeros((M, 3 * N), dtype=dtype, device="cuda")
        esz = full0.element_size()
        ptrs = [full0.data_ptr() + N * esz, full1.data_ptr() + 2 * N * esz]
        ops.qlinear_i8_into(a, b, sx if dtype != torch.int32 else None, sw if dtype != torch.int32 else None, ptrs,
                            3 * N, out_dtype=dtype, variant=2)
        assert torch.equal(full0[:, N:2 * N], want) and torch.equal(full1[:, 2 * N:], want)
        assert not full0[:, :N].any() and not full0[:, 2 * N:].any() and not full1[:, :2 * N].any()
    assert torch.equal(ref, ops.qlinear_i8(a, b, sx, sw, variant=1))


@pytest.mark.parametrize("scheme,qmin,qmax,signed", [("tensor_affine", 0, 255, False), ("tensor_symmetric", -128, 127, True),
                                                     ("token_symmetric", -128, 127, True)])
@pytest.mark.parametrize("M,N,K", [(1, 64, 16), (64, 4096, 1024), (300, 200, 328)])
def test_single_call_dynamic_linear_equals_the_separate_calls(scheme, qmin, qmax, signed, M, N, K):
    """lc_dynamic_linear_f32 (quantize + GEMM from one entry point, one workspace) gives the bits of
    the separate quantize and GEMM calls, call after call on a reused workspace."""
    from lucid_b200._C import ops

    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    wq = ops.pad_rows_to_16(torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g))
    sw = torch.rand(N, device="cuda", generator=g) * 0.01 + 1e-3
    bias = torch.randn(N, device="cuda", generator=g)
    wsum = ops.rowsum_s8(wq)
    ws = ops.dynamic_linear_workspace(M, K, torch.device("cuda", torch.cuda.current_device()))
    ws.fill_(0xFF)  # the entry point must not rely on what the buffer holds
    for i in range(3):
        x = torch.randn(M, K, device="cuda", generator=g) * (i + 1)
        y = ops.dynamic_linear(x, scheme, qmin, qmax, signed, wq, sw, bias, wsum, ws, fresh=(i == 0))
        code_dtype = torch.int8 if signed else torch.uint8
        if scheme == "token_symmetric":
            xq, sx, _ = ops.dynamic_quantize_rows(x, True, qmin, qmax, signed, 1e-8, code_dtype, pad_rows_to_16=True)
            want = ops.qlinear_i8(xq, wq, sx, sw, bias=bias)
        else:
            sym = scheme == "tensor_symmetric"
            xq, sx, zx, _ = ops.dynamic_quantize_tensor(x, sym, qmin, qmax, signed, 1e-8, code_dtype, pad_rows_to_16=True)
            needs_zp = not (sym and signed)
            want = ops.qlinear_i8(xq, wq, sx, sw, bias=bias, zx=zx if needs_zp else None, wsum=wsum if needs_zp else None)
        assert torch.equal(y, want)


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(4096, 1024), (2064, 2048), (1030, 4112), (4096, 14336)])
@pytest.mark.parametrize("a_unsigned", [False, True])
def test_decode_batches_take_the_streaming_kernel_with_identical_results(ops, M, N, K, a_unsigned):
    """Up to 32 rows against a weight of 4 MB and more: the GEMV-shaped `mma.sync` kernel.  Integer
    accumulation is exact, so the int32 accumulator equals the oracle's and the fp32 output equals, bit for bit,
    what the tensor-core GEMM (variant 1, which never takes this route) writes -- zero-point correction, per-row
    and per-tensor activation scales, bias; cold and warm launches agree."""
    r = np.random.default_rng(M * 7 + N * 3 + K + int(a_unsigned))
    a = r.integers(0, 256, (M, K)).astype(np.uint8) if a_unsigned else r.integers(-128, 128, (M, K)).astype(np.int8)
    b = r.integers(-128, 128, (N, K)).astype(np.int8)
    at, bt = dev(a), dev(b)
    st = status_word()
    acc = ops.qlinear_i8(at, bt, None, None, out_dtype=torch.int32, status=st)
    want = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.int64)  # exact: |sum| < 2^53
    np.testing.assert_array_equal(host(acc).astype(np.int64), want)
    sw = dev(r.random(N).astype(np.float32) * 0.01 + 1e-3)
    bias = dev(r.standard_normal(N).astype(np.float32))
    wsum = ops.rowsum_s8(bt)
    flush = torch.empty(300 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for per_row in (False, True):
        sx = dev(r.random(M if per_row else 1).astype(np.float32) * 0.05 + 1e-3)
        zx = dev(np.array([3.0 if a_unsigned else 0.0], np.float32))
        kw = dict(bias=bias, zx=zx if a_unsigned else None, wsum=wsum if a_unsigned else None, status=st)
        y = ops.qlinear_i8(at, bt, sx, sw, **kw)
        ref = ops.qlinear_i8(at, bt, sx, sw, variant=1, **kw)
        assert torch.equal(y, ref)
        flush.fill_(1)
        torch.cuda.synchronize()
        assert torch.equal(ops.qlinear_i8(at, bt, sx, sw, **kw), y)
    assert int(host(st)[0]) == 0
