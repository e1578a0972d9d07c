"""GPU parity: observers, calculate_qparams, quantize, dequantize, fake_quantize and
the fused dynamic quantizers, called through the C ABI, bit-compared with the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
STORAGE = {"int8": torch.int8, "int16": torch.int16, "int32": torch.int32}


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


def dev(a):
    return torch.tensor(np.ascontiguousarray(a), device="cuda")


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def rand(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


# ---------------------------------------------------------------------------
# golden fixtures
# ---------------------------------------------------------------------------
def test_golden_symmetric_extremum(ops):
    """The reference's bit-exact rounding case (test_functional.py:114-139)."""
    g = np.load(os.path.join(GOLDEN, "quant_golden.npz"))
    x = dev(g["x"])
    for axis, key in ((1, "ch1"), (0, "ch0")):
        C = x.shape[axis]
        mn = torch.empty(C, device="cuda")
        mx = torch.empty(C, device="cuda")
        ops.observe_channel(x, axis, mn, mx, accumulate=False)
        s, z = ops.calculate_qparams(mn, mx, True, -128, 127, True, 1e-8)
        np.testing.assert_array_equal(host(s), g[f"scale_{key}"])
        q = ops.quantize(x, s, z, -128, 127, torch.int8, ch_axis=axis)
        np.testing.assert_array_equal(host(q), g[f"q_{key}"])
    fq, mask = ops.fake_quantize(x, dev(g["scale_ch1"]), torch.zeros(256, device="cuda"), -128, 127,
                                 ch_axis=1, want_mask=True)
    np.testing.assert_array_equal(host(fq), g["fq_ch1"])
    np.testing.assert_array_equal(host(mask), g["mask_ch1"])
    assert (host(mask) == 0).any()
    dq = ops.dequantize(dev(g["q_ch0"]), dev(g["scale_ch0"]), torch.zeros(64, device="cuda"), ch_axis=0)
    np.testing.assert_array_equal(host(dq), g["dq_ch0"])
    # Python-float scale: reciprocal taken in double, rounded once
    np.testing.assert_array_equal(host(ops.quantize(x, 0.05, 0.0, -128, 127, torch.int8)), g["q_pyfloat"])


def test_golden_per_tensor(ops):
    g = np.load(os.path.join(GOLDEN, "quant_golden.npz"))
    x = dev(g["x"])
    mn = torch.empty((), device="cuda")
    mx = torch.empty((), device="cuda")
    s, z = ops.observe_tensor(x, mn, mx, accumulate=False, qspec=(False, 0, 255, False, 1e-8))
    np.testing.assert_array_equal(np.array([host(s), host(z)], np.float32), g["qparams_affine"])
    np.testing.assert_array_equal(host(ops.quantize(x, s, z, 0, 255, torch.int16)), g["q_affine"])
    s, z = ops.observe_tensor(x, mn, mx, accumulate=False, qspec=(True, -128, 127, True, 1e-8))
    np.testing.assert_array_equal(np.array([host(s), host(z)], np.float32), g["qparams_sym"])
    np.testing.assert_array_equal(host(ops.quantize(x, s, z, -128, 127, torch.int8)), g["q_sym"])


# ---------------------------------------------------------------------------
# reference unit-test assertions on the CUDA path
# ---------------------------------------------------------------------------
def test_reference_unit_cases(ops):
    x = dev(np.array([-1.0, -0.3, 0.0, 0.7, 2.0], np.float32))
    q = ops.quantize(x, 0.05, 0.0, -128, 127, torch.int8)
    assert np.allclose(host(ops.dequantize(q, 0.05, 0.0)), host(x), atol=1e-6)
    q = ops.quantize(dev(np.array([-1000.0, 1000.0], np.float32)), 0.1, 0.0, -128, 127, torch.int8)
    assert host(q).tolist() == [-128, 127]
    q = ops.quantize(dev(np.array([0.0], np.float32)), 0.02, 128.0, 0, 255, torch.int16)
    assert int(host(q)[0]) == 128
    _, m = ops.fake_quantize(dev(np.array([-100.0, 0.2, 0.5, 100.0], np.float32)), 0.05, 0.0, -128, 127,
                             want_mask=True)
    assert host(m).tolist() == [0.0, 1.0, 1.0, 0.0]
    nan = ops.quantize(dev(np.array([np.nan, 1.0], np.float32)), 0.5, 0.0, -128, 127, torch.int8)
    assert host(nan).tolist() == [0, 2]


def test_running_observers(ops):
    a, b = rand((33, 77), 1), rand((5, 77), 2) * 3
    mn = torch.full((), float("inf"), device="cuda")
    mx = torch.full((), float("-inf"), device="cuda")
    ops.observe_tensor(dev(a), mn, mx, accumulate=True)
    ops.observe_tensor(dev(b), mn, mx, accumulate=True)
    assert float(host(mn)) == min(a.min(), b.min()) and float(host(mx)) == max(a.max(), b.max())
    for axis in (0, 1):
        c = a.shape[axis]
        mn = torch.full((c,), float("inf"), device="cuda")
        mx = torch.full((c,), float("-inf"), device="cuda")
        ops.observe_channel(dev(a), axis, mn, mx, accumulate=True)
        omn, omx = O.minmax_channel(a, axis)
        np.testing.assert_array_equal(host(mn), omn)
        np.testing.assert_array_equal(host(mx), omx)


@pytest.mark.parametrize("shape,axis", [((9, 5, 1024), 1), ((8, 3, 128), 1), ((20, 6, 384), 1), ((7, 5, 1024), 1), ((16, 2, 1920), 1),
                                        ((64, 4, 256), 1), ((3, 8, 64, 2), 1)])
def test_channel_observer_layouts(ops, shape, axis):
    """Per-channel running ranges for 128..2047 elements per channel (the column-walk kernel from 8 outer rows
    on) and the neighbouring layouts, accumulated over two batches; equal to the oracle's."""
    a, b = rand(shape, sum(shape)), rand(shape, sum(shape) + 1) * 2.0
    c = shape[axis]
    mn = torch.full((c,), float("inf"), device="cuda")
    mx = torch.full((c,), float("-inf"), device="cuda")
    ops.observe_channel(dev(a), axis, mn, mx, accumulate=False)
    ops.observe_channel(dev(b), axis, mn, mx, accumulate=True)
    amn, amx = O.minmax_channel(a, axis)
    bmn, bmx = O.minmax_channel(b, axis)
    np.testing.assert_array_equal(host(mn), np.minimum(amn, bmn))
    np.testing.assert_array_equal(host(mx), np.maximum(amx, bmx))


@pytest.mark.parametrize("shape,axis", [((7,), None), ((1, 1), None), ((129, 513), None), ((4096, 1024), 0),
                                        ((3, 5, 7), 1), ((2, 300, 130), 1), ((64, 4100), 0), ((70, 9), 1),
                                        ((1000, 1003), 0), ((16, 8192), 0), ((5, 16388), 0),
                                        # channel axis last / short inner extents: the column kernels (rows of
                                        # channels * inner elements, a multiple of 4, at least 4 of them)
                                        ((70, 12), 1), ((37, 1024), 1), ((5, 7, 9, 64), 3), ((6, 20, 6), 1),
                                        ((33, 8, 2), 1), ((3, 16), 1), ((2000, 260), 1), ((4, 2052), 1),
                                        ((16, 6, 256), 1), ((9, 5, 1024), 1), ((7, 5, 1024), 1), ((8, 3, 2048), 1)])
@pytest.mark.parametrize("qd", ["qint8", "quint8", "qint4", "qint8_narrow"])
def test_quantize_dequantize_matches_oracle(ops, shape, axis, qd):
    qdt = getattr(O, qd)
    x = rand(shape, sum(shape) * 7 + (axis or 0)) * 2.5
    xt = dev(x)
    if axis is None:
        mn, mx = O.minmax_tensor(x)
    else:
        mn, mx = O.minmax_channel(x, axis)
    symmetric = qdt.signed
    s, z = O.calculate_qparams(mn, mx, symmetric, qdt)
    gs, gz = ops.calculate_qparams(dev(np.atleast_1d(mn)), dev(np.atleast_1d(mx)), symmetric, qdt.quant_min,
                                   qdt.quant_max, qdt.signed, 1e-8)
    np.testing.assert_array_equal(host(gs), np.atleast_1d(s))
    np.testing.assert_array_equal(host(gz), np.atleast_1d(z))
    q = ops.quantize(xt, gs, gz, qdt.quant_min, qdt.quant_max, STORAGE[qdt.storage], ch_axis=axis)
    qo = O.quantize(x, s, z, qdt, ch_axis=axis)
    np.testing.assert_array_equal(host(q), qo)
    np.testing.assert_array_equal(host(ops.dequantize(q, gs, gz, ch_axis=axis)), O.dequantize(qo, s, z, ch_axis=axis))
    fq, mask = ops.fake_quantize(xt, gs, gz, qdt.quant_min, qdt.quant_max, ch_axis=axis, want_mask=True)
    ofq, omask = O.fake_quantize(x, s, z, qdt.quant_min, qdt.quant_max, ch_axis=axis)
    np.testing.assert_array_equal(host(fq), ofq)
    np.testing.assert_array_equal(host(mask), omask)


def test_qint32_and_unaligned_views(ops):
    x = rand((37, 41), 3) * 1e4
    q = ops.quantize(dev(x), 1e-6, 0.0, -2**31, 2**31 - 1, torch.int32)
    np.testing.assert_array_equal(host(q), O.quantize(x, 1e-6, 0.0, O.qint32))
    # a tensor whose storage does not start on a 16-byte boundary
    base = dev(rand((4100,), 4))
    xv = base[1:].view(1, 4099)
    assert xv.is_contiguous() and xv.data_ptr() % 16 != 0
    np.testing.assert_array_equal(host(ops.quantize(xv, 0.03, 1.0, -128, 127, torch.int8)),
                                  O.quantize(host(xv), 0.03, 1.0, O.qint8))


def test_empty_inputs(ops):
    e = torch.empty((0, 8), device="cuda")
    assert ops.quantize(e, 0.1, 0.0, -128, 127, torch.int8).shape == (0, 8)
    assert ops.dequantize(e.to(torch.int8), 0.1, 0.0).shape == (0, 8)


@pytest.mark.parametrize("rows,cols", [(1, 4), (64, 1024), (33, 512), (17, 200), (9, 4100), (5, 8192),
                                       (3, 16384), (2, 20000), (7, 1023),
                                       # rows of up to 2048 elements: a warp per row, eight rows per CTA
                                       (1000, 64), (9, 128), (37, 132), (15, 256), (21, 1028), (11, 2048), (10, 2052)])
@pytest.mark.parametrize("mode", ["sym_s8", "sym_narrow", "affine_u8"])
def test_dynamic_quantize_rows(ops, rows, cols, mode):
    x = rand((rows, cols), rows * 31 + cols)
    x[0, 0] = 7.5
    qdt = {"sym_s8": O.qint8, "sym_narrow": O.qint8_narrow, "affine_u8": O.quint8}[mode]
    sym = mode != "affine_u8"
    out_dtype = torch.int8 if sym else torch.uint8
    for pad in (False, True):
        q, s, z = ops.dynamic_quantize_rows(dev(x), sym, qdt.quant_min, qdt.quant_max, qdt.signed, 1e-8,
                                            out_dtype, pad_rows_to_16=pad)
        mn, mx = O.minmax_channel(x, 0)
        os_, oz = O.calculate_qparams(mn, mx, sym, qdt)
        np.testing.assert_array_equal(host(s), os_)
        np.testing.assert_array_equal(host(z), oz)
        np.testing.assert_array_equal(host(q).astype(np.int32), O.quantize(x, os_, oz, qdt, ch_axis=0).astype(np.int32))


@pytest.mark.parametrize("rows,cols", [(1, 1), (2, 4), (33, 64), (64, 1024), (128, 1024), (129, 1024), (257, 300), (100, 4099)])
@pytest.mark.parametrize("mode", ["sym_s8", "affine_u8"])
def test_dynamic_quantize_tensor(ops, rows, cols, mode):
    x = rand((rows, cols), rows + cols) * 1.7
    qdt = O.qint8 if mode == "sym_s8" else O.quint8
    sym = mode == "sym_s8"
    for pad in (False, True):
        q, s, z, mm = ops.dynamic_quantize_tensor(dev(x), sym, qdt.quant_min, qdt.quant_max, qdt.signed, 1e-8,
                                                  torch.int8 if sym else torch.uint8, pad_rows_to_16=pad)
        mn, mx = O.minmax_tensor(x)
        os_, oz = O.calculate_qparams(mn, mx, sym, qdt)
        assert host(mm).tolist() == [float(mn), float(mx)]
        assert float(host(s)) == float(os_) and float(host(z)) == float(oz)
        np.testing.assert_array_equal(host(q).astype(np.int32), O.quantize(x, os_, oz, qdt).astype(np.int32))


def test_full_size_roundtrip_properties(ops):
    """[8192, 8192] with 0.1 % outliers x50 (the standalone roundtrip workload):
    oracle comparison on a row sample, size-independent properties on the rest."""
    torch.manual_seed(0)
    x = torch.randn(8192, 8192, device="cuda")
    idx = torch.randint(0, x.numel(), (x.numel() // 1000,), device="cuda")
    x.view(-1)[idx] *= 50.0
    q, s, z = ops.dynamic_quantize_rows(x, True, -128, 127, True)
    mn = torch.empty(8192, device="cuda")
    mx = torch.empty(8192, device="cuda")
    ops.observe_channel(x, 0, mn, mx, accumulate=False)
    s2, z2 = ops.calculate_qparams(mn, mx, True, -128, 127, True, 1e-8)
    q2 = ops.quantize(x, s2, z2, -128, 127, torch.int8, ch_axis=0)
    assert torch.equal(s, s2) and torch.equal(q, q2)           # fused == observer + quantize
    dq = ops.dequantize(q, s, z, ch_axis=0)
    assert torch.equal(ops.quantize(dq, s, z, -128, 127, torch.int8, ch_axis=0), q)  # idempotent on the grid
    err = (dq - x).abs()
    assert bool((err <= s[:, None] * 0.5 * 1.0001 + 1e-7).all())  # half a step, nothing saturates (symmetric)
    assert int(q.abs().max()) <= 128
    rows = [0, 1, 4095, 8191]
    xs = host(x[rows])
    smn, smx = O.minmax_channel(xs, 0)
    so, zo = O.calculate_qparams(smn, smx, True, O.qint8)
    np.testing.assert_array_equal(host(s[rows]), so)
    np.testing.assert_array_equal(host(q[rows]), O.quantize(xs, so, zo, O.qint8, ch_axis=0))
    # per-tensor path on the same tensor
    qt, st, zt, mm = ops.dynamic_quantize_tensor(x, True, -128, 127, True, 1e-8, torch.int8)
    assert float(mm[0]) == float(x.min()) and float(mm[1]) == float(x.max())
    np.testing.assert_array_equal(host(qt[rows]), O.quantize(xs, host(st), 0.0 + host(zt), O.qint8))


@pytest.mark.parametrize("n", [1, 5, 4096, 4099, 1 << 20])
@pytest.mark.parametrize("op", ["add", "mul", "add_relu"])
def test_fake_quantize_merge_matches_oracle(n, op):
    """One-pass merge + fake-quantize against the oracle's composition of the eager ops
    (bit-exact: both round the merge once in fp32), tensor and scalar operands, device and
    host qparams, NaN passing through the ReLU."""
    from lucid_b200._C import ops

    r = np.random.default_rng(n)
    a = (r.standard_normal(n) * 3).astype(np.float32)
    b = (r.standard_normal(n) * 3).astype(np.float32)
    if n > 4:
        a[2], b[3] = np.nan, np.inf
    s, z = np.float32(0.043), np.float32(101.0)

    def want(bb):
        t = (a * bb if op == "mul" else a + bb).astype(np.float32)
        if op == "add_relu":
            t = np.where(t < 0, np.float32(0), t)
        return O.fake_quantize(t, s, z, 0, 255)[0]

    at, bt = torch.tensor(a, device="cuda"), torch.tensor(b, device="cuda")
    got = ops.fake_quantize_merge(at, bt, op, torch.tensor(s, device="cuda"), torch.tensor(z, device="cuda"), 0, 255)
    np.testing.assert_array_equal(got.cpu().numpy(), want(b))
    got = ops.fake_quantize_merge(at, 0.75, op, float(s), float(z), 0, 255)
    np.testing.assert_array_equal(got.cpu().numpy(), O.fake_quantize(
        (lambda t: np.where(t < 0, np.float32(0), t) if op == "add_relu" else t)(
            (a * np.float32(0.75) if op == "mul" else a + np.float32(0.75)).astype(np.float32)), float(s), float(z), 0, 255)[0])
    got = ops.fake_quantize_merge(at[1:], bt[1:], op, float(s), float(z), 0, 255)  # unaligned views
    np.testing.assert_array_equal(got.cpu().numpy(), want(b)[1:])
