"""GPU parity of the histogram kernel behind lucid.histc and the histogram observer: counts
are integers, so the comparison with the oracle is exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


@pytest.mark.parametrize("n", [0, 1, 5, 1023, 4096 + 3, 1 << 20])
@pytest.mark.parametrize("bins", [1, 7, 256, 2048, 16384])
def test_histc_matches_oracle(ops, n, bins):
    r = np.random.default_rng(n + bins)
    x = r.standard_normal(n).astype(np.float32)
    if n > 8:
        x[::7] *= 30.0
        x[3], x[4], x[5] = np.nan, np.inf, -np.inf
    lo, hi = (-3.5, 11.25) if n else (0.0, 1.0)
    got = ops.histc(torch.tensor(x, device="cuda"), bins, lo, hi)
    want = O.histc(x, bins, lo, hi) if n else np.zeros(bins, np.float32)
    assert got.dtype == torch.float32
    assert np.array_equal(got.cpu().numpy(), want)


def test_histc_edges_and_accumulate(ops):
    # values exactly on bin edges, on the range ends, and just outside
    bins, lo, hi = 8, -1.0, 1.0
    edges = np.linspace(lo, hi, bins + 1)
    x = np.concatenate([edges, np.nextafter(edges, np.inf), np.nextafter(edges, -np.inf)]).astype(np.float32)
    xt = torch.tensor(x, device="cuda")
    out = ops.histc(xt, bins, lo, hi)
    want = O.histc(x, bins, lo, hi)
    assert np.array_equal(out.cpu().numpy(), want)
    for _ in range(3):  # the workspace is left clean: repeated calls accumulate exactly
        ops.histc(xt, bins, lo, hi, out=out, accumulate=True)
    assert np.array_equal(out.cpu().numpy(), 4 * want)
    # unaligned view (no 16-byte loads) gives the same counts as its copy
    y = torch.randn(10_001, device="cuda")[1:]
    assert torch.equal(ops.histc(y, 64, -4.0, 4.0), ops.histc(y.clone(), 64, -4.0, 4.0))


def test_histc_full_size_conservation(ops):
    """[8192, 8192] standard normal with outliers: every finite value inside the data range is
    counted exactly once, and the counts of two halves add up to the counts of the whole."""
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(8192, 8192, device="cuda", generator=g)
    x.view(-1)[::1000] *= 50.0
    lo, hi = float(x.min()), float(x.max())
    whole = ops.histc(x, 2048, lo, hi)
    assert float(whole.double().sum()) == x.numel()
    halves = ops.histc(x[:4096], 2048, lo, hi)
    ops.histc(x[4096:], 2048, lo, hi, out=halves, accumulate=True)
    assert torch.equal(halves, whole)


def test_lucid_histc_front_end():
    import lucid_b200 as lucid

    x = torch.tensor([0.25, 0.5, 0.75, 1.0, float("nan")], device="cuda")
    with pytest.raises(ValueError, match="not finite"):
        lucid.histc(x, 4)
    x = x[:4]
    assert lucid.histc(x, 4).tolist() == [1.0, 1.0, 1.0, 1.0]
    assert lucid.histc(torch.tensor([3.0, 3.0], device="cuda"), 4).tolist() == [0.0, 0.0, 2.0, 0.0]
    with pytest.raises(ValueError, match="at least min"):
        lucid.histc(x, 2, 3.0, 1.0)
    assert lucid.histc(x.cpu(), 4).tolist() == [1.0, 1.0, 1.0, 1.0]


def test_histogram_observer_matches_oracle_counts():
    import lucid_b200.quantization as Q

    r = np.random.default_rng(3)
    a = r.standard_normal((64, 1024)).astype(np.float32)
    b = (r.standard_normal((64, 1024)) * 3.0).astype(np.float32)  # widens the range: rebinning
    obs = Q.HistogramObserver(bins=512)
    obs(torch.tensor(a, device="cuda"))
    lo, hi = float(a.min()), float(a.max())
    assert np.array_equal(obs.histogram.cpu().numpy(), O.histc(a, 512, lo, hi))
    obs(torch.tensor(b, device="cuda"))
    assert float(obs.histogram.sum()) == a.size + b.size
    assert float(obs.min_val) == min(lo, float(b.min())) and float(obs.max_val) == max(hi, float(b.max()))
    scale, zp = obs.calculate_qparams()
    assert float(scale) > 0 and 0 <= float(zp) <= 255


@pytest.mark.parametrize("lo,hi", [(1000.0, 1001.0), (-1e-3, 2e-3), (-3.0, 3.0), (0.1, 0.7), (-1e30, 1e30)])
def test_histc_fp32_placement_is_exact(ops, lo, hi):
    """Values are placed in fp32 where that provably gives the float64 bin and in float64
    elsewhere: ranges far from zero, tiny and huge ranges, and values piled up on bin edges
    (multiples of the float64 step, and their fp32 neighbours) all match the oracle."""
    bins = 2048
    r = np.random.default_rng(int(abs(lo) * 7) % 1000)
    x = (lo + (hi - lo) * r.random(300_000)).astype(np.float32)
    step = (hi - lo) / bins
    edges = (lo + step * r.integers(0, bins + 1, 50_000)).astype(np.float32)
    x = np.concatenate([x, edges, np.nextafter(edges, np.float32(np.inf)), np.nextafter(edges, np.float32(-np.inf))])
    got = ops.histc(torch.tensor(x, device="cuda"), bins, lo, hi).cpu().numpy()
    assert np.array_equal(got, O.histc(x, bins, lo, hi))
