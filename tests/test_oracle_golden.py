"""Pins the NumPy oracle against the reference's own known-answer tests.

Each case restates an assertion of the reference test-suite (file:line in the
docstring) or cross-checks against ``torch.quantize_per_tensor``, which the
reference's parity tier declares array-equal to its ``quantize``.
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_qdtype_ranges():
    """lucid/test/unit/quantization/test_functional.py:11-15."""
    assert (O.qint8.quant_min, O.qint8.quant_max) == (-128, 127)
    assert (O.quint8.quant_min, O.quint8.quant_max) == (0, 255)
    assert (O.qint4.quant_min, O.qint4.quant_max) == (-8, 7)
    assert O.qint8.signed and not O.quint8.signed


def test_round_trip_on_grid():
    """test_functional.py:35-42."""
    x = np.array([-1.0, -0.3, 0.0, 0.7, 2.0], dtype=np.float32)
    q = O.quantize(x, 0.05, 0.0, O.qint8)
    assert q.dtype == np.int8
    assert np.allclose(O.dequantize(q, 0.05, 0.0), x, atol=1e-6)


def test_saturation():
    """test_functional.py:44-48."""
    q = O.quantize(np.array([-1000.0, 1000.0], dtype=np.float32), 0.1, 0.0, O.qint8)
    assert q.tolist() == [-128, 127]


def test_affine_zero_point():
    """test_functional.py:50-54."""
    q = O.quantize(np.array([0.0], dtype=np.float32), 0.02, 128.0, O.quint8)
    assert q.dtype == np.int16 and int(q[0]) == 128


def test_fake_equals_dequant_of_quant():
    """test_functional.py:58-63."""
    x = np.array([-1.0, -0.31, 0.0, 0.72, 2.0], dtype=np.float32)
    fq, _ = O.fake_quantize(x, 0.05, 0.0, -128, 127)
    dq = O.dequantize(O.quantize(x, 0.05, 0.0, O.qint8), 0.05, 0.0)
    assert np.allclose(fq, dq, atol=1e-6)


def test_ste_masks():
    """test_functional.py:65-79."""
    _, m = O.fake_quantize(np.array([-100.0, 0.2, 0.5, 100.0], np.float32), 0.05, 0.0, -128, 127)
    assert m.tolist() == [0.0, 1.0, 1.0, 0.0]
    w = np.array([[1.0, 2.0, 300.0], [-400.0, 0.5, 0.1]], np.float32)
    _, m = O.fake_quantize(w, np.array([0.02, 0.03], np.float32), np.zeros(2, np.float32), -128, 127, ch_axis=0)
    assert m.tolist() == [[1.0, 1.0, 0.0], [0.0, 1.0, 1.0]]


def test_per_channel_error_bound():
    """test_functional.py:83-93."""
    w = np.array([[1.0, 2.0, 3.0], [-4.0, 0.5, 0.1]], np.float32)
    s = np.array([0.03, 0.05], np.float32)
    z = np.zeros(2, np.float32)
    dq = O.dequantize(O.quantize(w, s, z, O.qint8, ch_axis=0), s, z, ch_axis=0)
    assert (np.abs(dq - w) <= np.array([[0.015], [0.025]]) + 1e-6).all()


def test_calculate_qparams():
    """test_functional.py:97-111 and test_observer.py:25-30."""
    s, z = O.calculate_qparams(-1.0, 3.0, False, O.quint8)
    assert float(s) == pytest.approx(4.0 / 255.0, rel=1e-5) and 0.0 <= float(z) <= 255.0
    s, z = O.calculate_qparams(-2.5, 2.0, True, O.qint8)
    assert float(z) == 0.0 and float(s) > 0.0
    s, _ = O.calculate_qparams(0.0, 0.0, False, O.qint8)
    assert float(s) > 0.0
    # symmetric scale is amax / 127.5 (test_functional.py:114-139 docstring)
    s, _ = O.calculate_qparams(-2.5, 2.0, True, O.qint8)
    assert s == np.float32(2.5) / np.float32(127.5)


def test_symmetric_extremum_reciprocal_rounding():
    """test_functional.py:114-139: codes follow round(x * (f32(1)/scale)),
    and at least one extremum lands off the grid."""
    data = np.random.default_rng(0).standard_normal((64, 256)).astype(np.float32)
    obs = O.MinMaxObserver(symmetric=True, qdtype=O.qint8, ch_axis=1)
    obs(data)
    scale, zp = obs.calculate_qparams()
    inv = np.float32(1.0) / scale
    codes = np.round(data * inv)
    expected_mask = ((codes >= -128) & (codes <= 127)).astype(np.float32)
    assert (expected_mask == 0.0).any()
    _, mask = O.fake_quantize(data, scale, zp, -128, 127, ch_axis=1)
    np.testing.assert_array_equal(mask, expected_mask)
    q = O.quantize(data, scale, zp, O.qint8, ch_axis=1)
    np.testing.assert_array_equal(q, np.clip(codes, -128, 127))
    # dividing instead of multiplying by the reciprocal gives other codes
    assert (np.clip(np.round(data / scale), -128, 127) != q).any()


def test_observers():
    """test_observer.py:12-17, 43-50."""
    o = O.MinMaxObserver()
    o(np.array([[-1.0, 2.0], [0.5, 3.0]], np.float32))
    o(np.array([[-2.0, 1.0]], np.float32))
    assert float(o.min_val) == -2.0 and float(o.max_val) == 3.0
    o = O.MinMaxObserver(symmetric=True, qdtype=O.qint8, ch_axis=0)
    o(np.array([[1.0, 2.0, 3.0], [-4.0, 0.5, 0.1]], np.float32))
    assert o.min_val.tolist() == [1.0, -4.0] and o.max_val.tolist() == [3.0, 0.5]
    s, z = o.calculate_qparams()
    assert s.shape == (2,) and z.tolist() == [0.0, 0.0]


def test_torch_quantize_per_tensor_cross_check():
    """lucid/test/parity/quantization/test_functional_parity.py:20-39: int
    codes array-equal to torch.quantize_per_tensor(...).int_repr()."""
    torch = pytest.importorskip("torch")
    for seed, shape in ((0, (3, 16)), (1, (4, 8)), (7, (257, 129))):
        data = np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
        q = O.quantize(data, 0.05, 0.0, O.qint8)
        r = torch.quantize_per_tensor(torch.tensor(data), 0.05, 0, torch.qint8)
        assert np.array_equal(q.astype(np.int64), r.int_repr().numpy().astype(np.int64))
        assert np.allclose(O.dequantize(q, 0.05, 0.0), r.dequantize().numpy(), atol=1e-4)
    data = np.random.default_rng(3).standard_normal((5, 7)).astype(np.float32)
    fq, _ = O.fake_quantize(data, 0.02, 128.0, 0, 255)
    r = torch.fake_quantize_per_tensor_affine(torch.tensor(data), 0.02, 128, 0, 255)
    assert np.allclose(fq, r.numpy(), atol=1e-4)


def test_torch_observer_cross_check():
    """lucid/test/parity/quantization/test_observer_parity.py:24-72: scales
    within 1e-6, zero-points within 1 of torch.ao observers."""
    torch = pytest.importorskip("torch")
    from torch.ao.quantization.observer import MinMaxObserver as TM

    data = np.random.default_rng(0).standard_normal((8, 32)).astype(np.float32)
    t = TM(dtype=torch.quint8, qscheme=torch.per_tensor_affine)
    t(torch.tensor(data))
    ts, tz = t.calculate_qparams()
    s, z = O.calculate_qparams(*O.minmax_tensor(data), False, O.quint8)
    assert float(s) == pytest.approx(float(ts), abs=1e-6) and abs(float(z) - float(tz)) <= 1


def test_dynamic_linear_quality_and_forms_agree():
    """lucid/test/unit/quantization/test_dynamic_ptq.py:40-46: mean relative
    error of the dynamic Linear below 5 %; and the integer formulation agrees
    with the reference's float formulation up to fp32 summation order."""
    r = np.random.default_rng(0)
    x = r.standard_normal((16, 64)).astype(np.float32)
    w = (r.standard_normal((32, 64)) * 0.1).astype(np.float32)
    b = (r.standard_normal(32) * 0.01).astype(np.float32)
    wq, sw, zw = O.quantize_weight_per_channel(w)
    y_ref = O.dynamic_linear_reference(x, wq, sw, zw, b)
    y_fp = O.linear_f32(x, w, b)
    assert np.abs(y_ref - y_fp).mean() / np.abs(y_fp).mean() < 0.05
    _, y_int, _, _, _ = O.dynamic_linear_int(x, wq, sw, b, "tensor_affine", O.quint8)
    np.testing.assert_allclose(y_int, y_ref, rtol=2e-4, atol=2e-5)


def test_group_format_round_trip():
    """_qgemm.py:164-165: |dequantize(quantize(w)) - w| <= s_g / 2."""
    w = np.random.default_rng(5).standard_normal((64, 128)).astype(np.float32)
    for bits in (8, 4):
        p, s, b = O.group_quantize(w, 64, bits)
        assert p.dtype == np.int32 and p.shape == (64, 128 * bits // 32)
        wh = O.group_dequantize(p, s, b, 64, bits)
        bound = np.repeat(s, 64, axis=1) / 2 + 1e-5
        assert (np.abs(wh - w) <= bound).all()


def test_committed_golden_vectors_match_oracle():
    """The committed fixtures are what the oracle produces today."""
    path = os.path.join(GOLDEN, "quant_golden.npz")
    g = np.load(path)
    meta = json.loads(str(g["meta"]))
    x = g["x"]
    s, z = O.calculate_qparams(*O.minmax_channel(x, 1), True, O.qint8)
    np.testing.assert_array_equal(s, g["scale_ch1"])
    np.testing.assert_array_equal(O.quantize(x, s, z, O.qint8, ch_axis=1), g["q_ch1"])
    st, zt = O.calculate_qparams(*O.minmax_tensor(x), False, O.quint8)
    np.testing.assert_array_equal(np.array([st, zt], np.float32), g["qparams_affine"])
    np.testing.assert_array_equal(O.quantize(x, st, zt, O.quint8), g["q_affine"])
    assert meta["seed"] == 0


# ---- histc: the reference pins lucid.histc to torch.histc on these cases
# (lucid/test/unit/ops/test_adapter_index_stats.py:107-127, refusals :130-144)
_NAN, _INFTY = float("nan"), float("inf")
_HISTC_CASES = [
    ([_NAN, 1.0, 2.0], 2, 0.0, 2.0),
    ([3.0, 3.0], 4, 0.0, 0.0),
    ([3.0], 3, 5.0, 5.0),
    ([1.0, 3.0], 4, 2.0, 2.0),
    ([_INFTY, 1.0, 2.0], 2, 0.0, 2.0),
    ([-_INFTY, _NAN, 0.5], 2, 0.0, 1.0),
    ([5.0, -1.0, 1.0], 2, 0.0, 2.0),
    ([], 3, 0.0, 0.0),
    ([0.25, 0.5, 0.75, 1.0], 4, 0.0, 0.0),
]


@pytest.mark.parametrize("data,bins,lo,hi", _HISTC_CASES, ids=str)
def test_histc_matches_the_references_pin(data, bins, lo, hi):
    torch = pytest.importorskip("torch")
    got = O.histc(np.array(data, dtype=np.float32), bins, lo, hi)
    want = torch.histc(torch.tensor(data, dtype=torch.float32), bins, lo, hi).numpy()
    assert got.dtype == np.float32 and np.array_equal(got, want)


def test_histc_refusals_and_bulk():
    torch = pytest.importorskip("torch")
    with pytest.raises(ValueError, match="not finite"):
        O.histc(np.array([_NAN, 1.0], dtype=np.float32), 2, 0.0, 0.0)
    with pytest.raises(ValueError, match="not finite"):
        O.histc(np.array([1.0], dtype=np.float32), 2, 0.0, _INFTY)
    with pytest.raises(ValueError, match="at least min"):
        O.histc(np.array([1.0], dtype=np.float32), 2, 3.0, 1.0)
    x = np.random.default_rng(5).standard_normal(200_000).astype(np.float32)
    x[::1000] *= 50.0
    for bins in (7, 256, 2048):
        lo, hi = float(x.min()), float(x.max())
        got = O.histc(x, bins, lo, hi)
        assert got.sum() == x.size  # both edges are inside
        # torch buckets in float32; away from bin edges the two agree, and the totals always do
        want = torch.histc(torch.tensor(x), bins, lo, hi).numpy()
        assert np.abs(got - want).sum() <= 4


@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
def test_embedding_oracle_against_torch(mode):
    """The quantized table forwards are 'dequantize the table, then the float lookup'; torch
    implements the float lookups with the semantics the reference mirrors (padding entries
    skipped, mean over the entries kept, empty bags zero), on the index pattern of the
    reference's own case (lucid/test/unit/quantization/test_module_breadth.py:96-108)."""
    import torch

    r = np.random.default_rng(0)
    q = r.integers(-128, 128, size=(50, 16), dtype=np.int8)
    s = (r.random(50).astype(np.float32) + 0.01) * np.float32(0.02)
    z = r.integers(-5, 5, size=50).astype(np.float32)
    w = torch.tensor(O.dequantize(q, s, z, ch_axis=0))
    idx = np.array([1, 5, 9, 3, 7, 2, 8, 9, 9])
    off = np.array([0, 3, 5, 5, 7])
    assert np.array_equal(O.embedding_s8(q, s, z, idx.reshape(3, 3)),
                          torch.nn.functional.embedding(torch.tensor(idx.reshape(3, 3)), w).numpy())
    for pad in (None, 9):
        want = torch.nn.functional.embedding_bag(torch.tensor(idx), w, torch.tensor(off), mode=mode, padding_idx=pad)
        got = O.embedding_bag_s8(q, s, z, idx, off, mode, pad)
        assert np.allclose(got, want.numpy(), rtol=1e-6, atol=1e-7)
    want = torch.nn.functional.embedding_bag(torch.tensor(idx), w, torch.tensor(np.append(off, 9)), mode=mode,
                                             include_last_offset=True)
    assert np.allclose(O.embedding_bag_s8(q, s, z, idx, np.append(off, 9), mode, None, None, True), want.numpy(),
                       rtol=1e-6, atol=1e-7)
    if mode == "sum":
        psw = r.standard_normal(9).astype(np.float32)
        want = torch.nn.functional.embedding_bag(torch.tensor(idx), w, torch.tensor(off), mode="sum",
                                                 per_sample_weights=torch.tensor(psw))
        assert np.allclose(O.embedding_bag_s8(q, s, z, idx, off, "sum", None, psw), want.numpy(), rtol=1e-5, atol=1e-6)
    with pytest.raises(IndexError):
        O.embedding_s8(q, s, z, np.array([50]))
