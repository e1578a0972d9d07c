"""GPU parity of the int8 embedding lookups: decoded rows and max / sum / mean pools are
compared bit for bit with the oracle (same fp32 operations in the same order); pools with
per-sample weights within rtol 1e-6."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


def _table(r, V, D, affine=False):
    q = r.integers(-128, 128, size=(V, D), dtype=np.int8)
    s = (r.random(V).astype(np.float32) + 0.01) * np.float32(0.05)
    z = r.integers(-20, 20, size=V).astype(np.float32) if affine else np.zeros(V, np.float32)
    return q, s, z


def _dev(*arrays):
    return [torch.tensor(a, device="cuda") for a in arrays]


@pytest.mark.parametrize("V,D", [(7, 1), (50, 16), (33, 130), (100, 1024), (64, 4096), (19, 1027), (40, 2052)])
@pytest.mark.parametrize("affine", [False, True])
def test_embedding_matches_oracle(ops, V, D, affine):
    r = np.random.default_rng(V * 131 + D)
    q, s, z = _table(r, V, D, affine)
    for shape in [(1,), (5,), (3, 4), (257,)]:
        idx = r.integers(0, V, size=shape)
        tq, ts, tz, ti = _dev(q, s, z, idx)
        got = ops.embedding_s8(tq, ts, tz if affine else None, ti)
        want = O.embedding_s8(q, s, z, idx)
        assert got.shape == idx.shape + (D,) and got.dtype == torch.float32
        assert np.array_equal(got.cpu().numpy(), want)
    empty = ops.embedding_s8(tq, ts, None, torch.zeros(0, dtype=torch.int64, device="cuda"))
    assert empty.shape == (0, D)


def test_embedding_index_dtypes_views_and_bad_indices(ops):
    r = np.random.default_rng(5)
    q, s, z = _table(r, 30, 64)
    tq, ts = _dev(q, s)
    idx = r.integers(0, 30, size=12)
    want = O.embedding_s8(q, s, z, idx)
    for dt in (torch.int32, torch.int64, torch.int16):
        assert np.array_equal(ops.embedding_s8(tq, ts, None, torch.tensor(idx, device="cuda").to(dt)).cpu().numpy(), want)
    # an unaligned table view takes the scalar path and gives the same rows
    flat = torch.zeros(30 * 64 + 1, dtype=torch.int8, device="cuda")
    flat[1:] = tq.reshape(-1)
    view = flat[1:].reshape(30, 64)
    assert np.array_equal(ops.embedding_s8(view, ts, None, torch.tensor(idx, device="cuda")).cpu().numpy(), want)
    # out-of-range indices: a row of zeros and the status flag, no fault
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad = torch.tensor([3, 30, -1, 4], device="cuda")
    got = ops.embedding_s8(tq, ts, None, bad, status=status).cpu().numpy()
    assert int(status.item()) == 1
    assert np.array_equal(got[[0, 3]], O.embedding_s8(q, s, z, np.array([3, 4])))
    assert not got[[1, 2]].any()
    status.zero_()
    ops.embedding_s8(tq, ts, None, torch.tensor(idx, device="cuda"), status=status)
    assert int(status.item()) == 0


@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
@pytest.mark.parametrize("V,D", [(50, 16), (33, 130), (64, 512), (21, 7)])
def test_embedding_bag_matches_oracle(ops, mode, V, D):
    r = np.random.default_rng(V + D + len(mode))
    q, s, z = _table(r, V, D, affine=True)
    tq, ts, tz = _dev(q, s, z)
    n = 97
    idx = r.integers(0, V, size=n)
    cuts = np.sort(r.choice(np.arange(1, n), size=11, replace=False))
    off = np.concatenate([[0], cuts, [cuts[-1]], [cuts[-1]]])  # the last two bags: one empty, one to the end
    pad = int(idx[5])
    for padding_idx in (None, pad):
        for include_last in (False, True):
            o = np.concatenate([off, [n]]) if include_last else off
            got = ops.embedding_bag_s8(tq, ts, tz, torch.tensor(idx, device="cuda"), torch.tensor(o, device="cuda"),
                                       mode, padding_idx, None, include_last)
            want = O.embedding_bag_s8(q, s, z, idx, o, mode, padding_idx, None, include_last)
            assert got.shape == want.shape
            assert np.array_equal(got.cpu().numpy(), want), (mode, padding_idx, include_last)
    # a bag made only of padding entries is an empty bag
    only_pad = np.full(4, pad)
    got = ops.embedding_bag_s8(tq, ts, tz, torch.tensor(only_pad, device="cuda"), torch.tensor([0, 2], device="cuda"),
                               mode, pad)
    assert not got.cpu().numpy().any()


@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
def test_embedding_bag_many_bags_wide_pieces(ops, mode):
    """Enough (bag, column piece) items that the kernel takes its 16-byte-per-thread form."""
    r = np.random.default_rng(77)
    V, D, bags = 300, 256, 6000
    q, s, z = _table(r, V, D, affine=True)
    lengths = r.integers(0, 9, size=bags)
    off = np.concatenate([[0], np.cumsum(lengths)[:-1]])
    n = int(lengths.sum())
    idx = r.integers(0, V, size=n)
    w = r.standard_normal(n).astype(np.float32) if mode == "sum" else None
    tq, ts, tz = _dev(q, s, z)
    got = ops.embedding_bag_s8(tq, ts, tz, torch.tensor(idx, device="cuda"), torch.tensor(off, device="cuda"), mode, 7)
    assert np.array_equal(got.cpu().numpy(), O.embedding_bag_s8(q, s, z, idx, off, mode, 7))
    if w is not None:
        got = ops.embedding_bag_s8(tq, ts, tz, torch.tensor(idx, device="cuda"), torch.tensor(off, device="cuda"), mode,
                                   None, torch.tensor(w, device="cuda"))
        assert np.allclose(got.cpu().numpy(), O.embedding_bag_s8(q, s, z, idx, off, mode, None, w), rtol=1e-6, atol=1e-7)


def test_embedding_bag_per_sample_weights_and_refusals(ops):
    r = np.random.default_rng(9)
    q, s, z = _table(r, 40, 96)
    tq, ts = _dev(q, s)
    idx = r.integers(0, 40, size=33)
    off = np.array([0, 4, 4, 20])
    w = r.standard_normal(33).astype(np.float32)
    got = ops.embedding_bag_s8(tq, ts, None, torch.tensor(idx, device="cuda"), torch.tensor(off, device="cuda"), "sum",
                               None, torch.tensor(w, device="cuda"))
    want = O.embedding_bag_s8(q, s, z, idx, off, "sum", None, w)
    assert np.allclose(got.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    with pytest.raises(ValueError):
        ops.embedding_bag_s8(tq, ts, None, torch.tensor(idx, device="cuda"), torch.tensor(off, device="cuda"), "mean",
                             None, torch.tensor(w, device="cuda"))
    with pytest.raises(ValueError):
        ops.embedding_bag_s8(tq, ts, None, torch.tensor(idx, device="cuda"), torch.tensor(off, device="cuda"), "median")
    with pytest.raises(TypeError):
        ops.embedding_s8(tq.float(), ts, None, torch.tensor(idx, device="cuda"))


def test_embedding_full_size_properties(ops):
    """A 128k x 4096 table and 16384 looked-up tokens: the kernel equals the reference's
    formulation (decode, then gather) evaluated with torch ops on the rows it touches, and a
    sum bag over single-entry bags equals the plain lookup."""
    g = torch.Generator(device="cuda").manual_seed(11)
    V, D, n = 128 * 1024, 4096, 16384
    tq = torch.randint(-128, 128, (V, D), dtype=torch.int8, device="cuda", generator=g)
    ts = torch.rand(V, device="cuda", generator=g) * 0.05 + 1e-3
    tz = torch.randint(-8, 8, (V,), device="cuda", generator=g).float()
    idx = torch.randint(0, V, (n,), device="cuda", generator=g)
    got = ops.embedding_s8(tq, ts, tz, idx)
    want = (tq[idx].float() - tz[idx, None]) * ts[idx, None]
    assert torch.equal(got, want)
    del want
    bags = ops.embedding_bag_s8(tq, ts, tz, idx, torch.arange(n, device="cuda"), "sum")
    assert torch.equal(bags, got + 0.0)
