"""GPU parity of the weight-only paths: per-channel int8 GEMV-shaped Linear and the
group-wise affine format (tolerance parity: float activations, fp32 accumulation)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tolerances import abs_terms, assert_rounded_product

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


def dev(a, dtype=None):
    t = torch.tensor(np.ascontiguousarray(a), device="cuda")
    return t if dtype is None else t.to(dtype)


def host(t):
    torch.cuda.synchronize()
    return t.float().cpu().numpy()


@pytest.mark.parametrize("B", [1, 2, 4, 8, 16, 17, 32, 40])
@pytest.mark.parametrize("N,K", [(64, 64), (100, 144), (4096, 1024), (1000, 4096), (300, 200)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_wo_linear_per_channel(ops, B, N, K, dtype):
    r = np.random.default_rng(B * 1000 + N + K)
    w = (r.standard_normal((N, K)) * 0.02).astype(np.float32)
    wq, sw, _ = O.quantize_weight_per_channel(w)
    bias = (r.standard_normal(N) * 0.01).astype(np.float32)
    x = dev(r.standard_normal((B, K)).astype(np.float32), dtype)
    wq_t = ops.pad_rows_to_16(dev(wq))
    y = ops.wo_linear_s8(x, wq_t, dev(sw), dev(bias))
    assert y.dtype == dtype and y.shape == (B, N)
    ref = O.weight_only_linear_perchannel(host(x), wq, sw, bias)
    assert_rounded_product(y, ref, abs_terms(x.cpu(), wq, sw), K, dtype)


def test_decode_mlp_shapes(ops):
    """hidden 4096 <-> FFN 14336 at batch 1/4/16 with bf16 activations."""
    torch.manual_seed(0)
    for N, K in ((14336, 4096), (4096, 14336)):
        w = torch.randn(N, K, device="cuda") * 0.02
        wq, sw, _ = ops.dynamic_quantize_rows(w, True, -128, 127, True)
        for B in (1, 4, 16):
            x = torch.randn(B, K, device="cuda").to(torch.bfloat16)
            y = ops.wo_linear_s8(x, wq, sw)
            ref = (x.double() @ wq.double().T) * sw.double()[None, :]
            assert_rounded_product(y, ref.cpu().numpy(), abs_terms(x, wq, sw), K, torch.bfloat16)
    assert ops.wo_linear_status() == 0, "a bounded device-side wait ran out"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,N,K", [(1, 2048, 2048), (3, 2050, 2064), (8, 4097, 1040), (9, 2400, 3072), (16, 5000, 1024),
                                   (17, 2048, 2048), (32, 2048, 4096), (5, 16, 262144), (2, 37000, 128)])
def test_wo_linear_ring_kernel_shapes(ops, dtype, B, N, K):
    """Weights of 4 MB and more go through the shared-memory ring kernel: ragged N (partial row
    tile), K not a multiple of the 1024-byte chunk, every batch-tile width, very long and very
    short rows."""
    g = torch.Generator(device="cuda").manual_seed(B * 7 + N + K)
    wq = torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
    sw = torch.rand(N, device="cuda", generator=g) * 0.01 + 0.001
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    x = torch.randn(B, K, device="cuda", generator=g).to(dtype)
    y = ops.wo_linear_s8(x, wq, sw, bias)
    ref = (x.double() @ wq.double().T) * sw.double()[None, :] + bias.double()[None, :]
    assert_rounded_product(y, ref.cpu().numpy(), abs_terms(x, wq, sw), K, dtype)
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_group_format_matches_oracle(ops, bits, gs):
    w = np.random.default_rng(bits + gs).standard_normal((64, 256)).astype(np.float32)
    w[3, :gs] = 0.25  # a constant group
    p, s, b = ops.group_quantize(dev(w), gs, bits)
    po, so, bo = O.group_quantize(w, gs, bits)
    assert p.dtype == torch.int32 and tuple(p.shape) == (64, 256 * bits // 32)
    np.testing.assert_array_equal(p.cpu().numpy(), po)
    np.testing.assert_array_equal(host(s), so)
    np.testing.assert_array_equal(host(b), bo)
    wh = ops.group_dequantize(p, s, b, gs, bits)
    np.testing.assert_array_equal(host(wh), O.group_dequantize(po, so, bo, gs, bits))
    assert (np.abs(host(wh) - w) <= np.repeat(so, gs, axis=1) / 2 + 1e-5).all()


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("rows", [1, 2, 8, 32])
def test_group_matmul_reference_cases(ops, bits, rows):
    """lucid/test/unit/quantization/test_real_gemm.py:92-107: kernel vs own dequant
    path, atol 1e-3, W [64,128], group 64; and the bench's 1e-4 relative gate."""
    r = np.random.default_rng(rows)
    w = r.standard_normal((64, 128)).astype(np.float32)
    x = r.standard_normal((rows, 128)).astype(np.float32)
    p, s, b = ops.group_quantize(dev(w), 64, bits)
    y = ops.group_matmul(dev(x), p, s, b, 64, bits)
    dense = ops.group_dequantize(p, s, b, 64, bits)
    expected = host(dev(x) @ dense.T)
    np.testing.assert_allclose(host(y), expected, atol=1e-3)
    assert np.abs(host(y) - expected).max() / max(np.abs(expected).max(), 1e-12) <= 1e-4
    ref = O.group_matmul(x, p.cpu().numpy(), host(s), host(b), 64, bits)
    np.testing.assert_allclose(host(y), ref, rtol=1e-4, atol=1e-4)


def test_group_matmul_bench_width(ops):
    """tools/bench_quantized_dispatch.py:29-54: N = K = 1024, M in {1,2,8,32}, gs 64."""
    torch.manual_seed(20260920)
    for bits in (4, 8):
        w = torch.randn(1024, 1024, device="cuda")
        p, s, b = ops.group_quantize(w, 64, bits)
        dense = ops.group_dequantize(p, s, b, 64, bits)
        for m in (1, 2, 8, 32):
            x = torch.randn(m, 1024, device="cuda")
            expected = x.double() @ dense.double().T
            actual = ops.group_matmul(x, p, s, b, 64, bits).double()
            assert float((expected - actual).abs().max()) / max(float(expected.abs().max()), 1e-12) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,K", [(256, 256), (4096, 1024)])
def test_int8_widening_is_exact_for_every_code(ops, dtype, N, K):
    """One-hot activations pick single weights: with unit scales the output must be the int8
    code itself, exactly, for all 256 codes (both kernels: direct-load and ring)."""
    n = torch.arange(N, device="cuda").view(-1, 1)
    k = torch.arange(K, device="cuda").view(1, -1)
    wq = (((n * 7 + k * 3) % 256) - 128).to(torch.int8)
    assert wq.unique().numel() == 256
    cols = [0, 1, 63, 64, 255, K - 1, K // 2, 17]
    x = torch.zeros(len(cols), K, device="cuda", dtype=dtype)
    for i, c in enumerate(cols):
        x[i, c] = 1.0
    y = ops.wo_linear_s8(x, wq, torch.ones(N, device="cuda"))
    assert torch.equal(y.float(), wq[:, cols].T.float())
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,F,K", [(1, 2048, 1024), (4, 14336, 4096), (16, 1000 * 8, 512), (9, 4096, 2064)])
def test_wo_swiglu_fused(ops, dtype, B, F, K):
    """Fused gate/up + SwiGLU against the float64 composition of the unfused definition."""
    g = torch.Generator(device="cuda").manual_seed(F + K + B)
    wg = torch.randint(-128, 128, (F, K), device="cuda", dtype=torch.int8, generator=g)
    wu = torch.randint(-128, 128, (F, K), device="cuda", dtype=torch.int8, generator=g)
    sg = torch.rand(F, device="cuda", generator=g) * 2e-3
    su = torch.rand(F, device="cuda", generator=g) * 2e-3
    x = torch.randn(B, K, device="cuda", generator=g).to(dtype)
    y = ops.wo_swiglu_s8(x, ops.interleave_gate_up(wg, wu), ops.interleave_gate_up(sg, su))
    gate = (x.double() @ wg.double().T) * sg.double()
    up = (x.double() @ wu.double().T) * su.double()
    ref = torch.nn.functional.silu(gate) * up
    assert y.shape == (B, F) and y.dtype == dtype
    # error of silu(g) * u from the accumulation errors eg, eu of the two projections
    # (|silu'| <= 1.1, |silu(g)| <= |g|), plus the kernel's fast exponential (2 ulp of fp32 on silu)
    eg, eu = abs_terms(x, wg, sg), abs_terms(x, wu, su)
    depth = (K / 32.0 + 32.0) * 2.0 ** -24
    extra = depth * (1.1 * eg * up.abs().cpu().numpy() + gate.abs().cpu().numpy() * eu) + 4 * 2.0 ** -24 * ref.abs().cpu().numpy()
    assert_rounded_product(y, ref.cpu().numpy(), np.zeros_like(eg), K, dtype, extra=extra)
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("B", [1, 16])
def test_launch_overlap_is_bit_identical(ops, B):
    """A chain of MLPs in which every kernel may start while its predecessor drains
    (weights prefetched early, activations read only after the predecessor is complete)
    gives the same bits as the fully serialised chain, eagerly and as a replayed graph."""
    H, F = 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(7 + B)
    wgu = torch.randint(-128, 128, (2 * F, H), device="cuda", dtype=torch.int8, generator=g)
    sgu = torch.rand(2 * F, device="cuda", generator=g) * 4e-4
    wd = torch.randint(-128, 128, (H, F), device="cuda", dtype=torch.int8, generator=g)
    sd = torch.rand(H, device="cuda", generator=g) * 4e-4
    x0 = torch.randn(B, H, device="cuda", generator=g).to(torch.bfloat16)
    torch.cuda.synchronize()

    def chain(overlap, depth=3):
        x = x0 * 1.0  # an ordinary kernel writes the first input right before the chain
        outs = []
        for _ in range(depth):
            h = ops.wo_swiglu_s8(x, wgu, sgu, overlap_previous=overlap)
            x = ops.wo_linear_s8(h, wd, sd, overlap_previous=overlap)
            outs.append(x)
        return torch.stack(outs)

    want = chain(False)
    got = chain(True)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert float(want[0].float().abs().max()) > 0.0
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain(True)  # warm-up outside capture
        with torch.cuda.graph(graph, stream=side):
            captured = chain(True)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured.view(torch.int16), want.view(torch.int16))
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("B", [1, 8, 9, 16, 32])
@pytest.mark.parametrize("N,K", [(4096, 14336), (28672, 4096)])
def test_streaming_kernel_cold_and_warm_launches_agree(ops, B, N, K):
    """A launch that finds nothing in L2 (weights, activations and scales all come from DRAM, boxes land slowly and
    the warps of a CTA drift apart) gives the bits of a launch that finds everything cached: a ring slot read
    before its copy has landed, or reused before every warp has left it, shows up here and not in back-to-back
    launches.  Covers one and several row tiles per CTA, one and two CTAs per SM, passes with an odd last tile."""
    g = torch.Generator(device="cuda").manual_seed(B + N + K)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    wq, sw, _ = ops.dynamic_quantize_rows(w, True, -128, 127, True)
    del w
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    flush = torch.empty(384 * 1024 * 1024, dtype=torch.uint8, device="cuda")  # three times the L2
    warm = ops.wo_linear_s8(x, wq, sw)
    warm = ops.wo_linear_s8(x, wq, sw)
    ref = (x.double() @ wq.double().T) * sw.double()[None, :]
    assert_rounded_product(warm, ref.cpu().numpy(), abs_terms(x, wq, sw), K, torch.bfloat16)
    for i in range(4):
        flush.fill_(i)
        torch.cuda.synchronize()
        cold = ops.wo_linear_s8(x, wq, sw)
        assert torch.equal(cold.view(torch.int16), warm.view(torch.int16)), f"cold launch {i} differs from the warm one"
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("B", [17, 24, 32])
def test_rows_17_to_32_equal_two_passes_of_16(ops, B):
    """17..32 rows run as two passes over the weights of at most 16 rows each: the result is, bit for bit, what
    the two row blocks give when the caller passes them separately, for the plain and the fused SwiGLU form."""
    g = torch.Generator(device="cuda").manual_seed(B)
    N, K = 8192, 4096
    wq = torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
    sw = torch.rand(N, device="cuda", generator=g) * 0.01 + 0.001
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    for call in (lambda v: ops.wo_linear_s8(v, wq, sw, bias), lambda v: ops.wo_swiglu_s8(v, wq, sw)):
        whole = call(x)
        parts = torch.cat([call(x[:16].contiguous()), call(x[16:].contiguous())])
        assert torch.equal(whole.view(torch.int16), parts.view(torch.int16))
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("B", [1, 16])
def test_fused_and_group_streaming_cold_and_warm_launches_agree(ops, B):
    """The same for the fused gate / up / SwiGLU epilogue and for the group-wise 8-bit format."""
    g = torch.Generator(device="cuda").manual_seed(B)
    F, K = 14336, 4096
    wg = torch.randint(-128, 128, (F, K), device="cuda", dtype=torch.int8, generator=g)
    wu = torch.randint(-128, 128, (F, K), device="cuda", dtype=torch.int8, generator=g)
    wgu = ops.interleave_gate_up(wg, wu)
    sgu = torch.rand(2 * F, device="cuda", generator=g) * 1e-3 + 1e-4
    packed, scales, biases = ops.group_quantize(torch.randn(F, K, device="cuda", generator=g) * 0.02, 64, 8)
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    flush = torch.empty(384 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    calls = (lambda: ops.wo_swiglu_s8(x, wgu, sgu), lambda: ops.group_matmul(x, packed, scales, biases, 64, 8))
    for call in calls:
        call()
        warm = call()
        for i in range(3):
            flush.fill_(i)
            torch.cuda.synchronize()
            assert torch.equal(call().view(torch.int16), warm.view(torch.int16)), f"cold launch {i} differs from the warm one"
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("B,N,K", [(1, 4096, 14336), (4, 14336, 4096), (16, 512, 65536), (32, 6000, 3000 * 16 // 16 * 16)])
def test_streaming_kernel_is_deterministic(ops, B, N, K):
    """The split-K sums of the streaming kernel are added in a fixed order: 25 back-to-back
    launches, alternately serialised and overlapping their predecessor, give identical bits."""
    g = torch.Generator(device="cuda").manual_seed(B + N + K)
    wq = torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
    sw = torch.rand(N, device="cuda", generator=g) * 0.01 + 0.001
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    first = ops.wo_linear_s8(x, wq, sw)
    ref = (x.double() @ wq.double().T) * sw.double()[None, :]
    assert_rounded_product(first, ref.cpu().numpy(), abs_terms(x, wq, sw), K, torch.bfloat16)
    for i in range(24):
        again = ops.wo_linear_s8(x, wq, sw, overlap_previous=bool(i & 1))
        assert torch.equal(again.view(torch.int16), first.view(torch.int16)), f"launch {i + 2} differs"
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("transpose", [True, False])
@pytest.mark.parametrize("bits", [8, 4])
def test_quantized_matmul_backward(transpose, bits):
    """d/dx of quantized_matmul is grad @ dequant(w) (or its transpose): checked against
    autograd through the dense reconstruction."""
    import lucid_b200.quantization._qgemm as G

    torch.manual_seed(bits)
    w = torch.randn(96, 128, device="cuda")
    wq, sc, bi = G.quantize(w, 64, bits)
    dense = G.dequantize(wq, sc, bi, 64, bits)
    for rows in (3, 40):  # GEMV-shaped kernel and dense route
        x = torch.randn(rows, 128 if transpose else 96, device="cuda", requires_grad=True)
        y = G.quantized_matmul(x, wq, sc, bi, transpose=transpose, group_size=64, bits=bits)
        g = torch.randn_like(y)
        (gx,) = torch.autograd.grad(y, x, g)
        x2 = x.detach().clone().requires_grad_(True)
        y2 = x2 @ (dense.T if transpose else dense)
        (gx2,) = torch.autograd.grad(y2, x2, g)
        assert torch.allclose(y, y2, rtol=1e-4, atol=1e-4 * float(y2.abs().max()))
        assert torch.allclose(gx, gx2, rtol=1e-4, atol=1e-4 * float(gx2.abs().max()))
    with torch.no_grad():
        assert not G.quantized_matmul(torch.randn(2, 128, device="cuda"), wq, sc, bi, group_size=64, bits=bits).requires_grad


@pytest.mark.parametrize("B,N,K", [(1, 4096, 14336), (4, 28672, 4096), (16, 4096, 14336), (8, 2048, 2048), (3, 2050, 2064),
                                   (5, 16, 262144), (2, 37000, 128), (32, 6000, 3008)])
def test_balanced_schedule_agrees_with_whole_boxes(ops, B, N, K):
    """The schedule that cuts K between CTAs (equal bytes per SM) against the one that deals out whole
    boxes: both within the rounding bound of the float64 product, equal to each other up to the last
    bits (sums over a split K range are added in another order), bit-identical from launch to launch,
    and the scratch (tickets) back at zero after every launch."""
    g = torch.Generator(device="cuda").manual_seed(B + N + K)
    wq = torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
    sw = torch.rand(N, device="cuda", generator=g) * 0.01 + 0.001
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    ref = ((x.double() @ wq.double().T) * sw.double()[None, :]).cpu().numpy()
    whole = ops.wo_linear_s8(x, wq, sw, balanced=False)
    split = ops.wo_linear_s8(x, wq, sw, balanced=True)
    for y in (whole, split):
        assert_rounded_product(y, ref, abs_terms(x, wq, sw), K, torch.bfloat16)
    assert (whole.float() - split.float()).abs().max() <= 2.0 ** -7 * whole.float().abs().max()
    for i in range(10):
        again = ops.wo_linear_s8(x, wq, sw, balanced=True, overlap_previous=bool(i & 1))
        assert torch.equal(again.view(torch.int16), split.view(torch.int16))
    torch.cuda.synchronize()
    ws = ops.wo_workspace(x.device, N)
    tickets = ws[-(ops._WO_WORKSPACE_ROWS // 16) * 4:]  # the tail of the scratch holds the tickets
    assert not bool(tickets.any())
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("B,F,K", [(1, 14336, 4096), (16, 14336, 4096), (9, 4096, 2064)])
def test_balanced_swiglu_agrees_with_whole_boxes(ops, B, F, K):
    g = torch.Generator(device="cuda").manual_seed(F + K + B)
    wgu = torch.randint(-128, 128, (2 * F, K), device="cuda", dtype=torch.int8, generator=g)
    sgu = torch.rand(2 * F, device="cuda", generator=g) * 2e-3
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    whole = ops.wo_swiglu_s8(x, wgu, sgu, balanced=False)
    split = ops.wo_swiglu_s8(x, wgu, sgu, balanced=True)
    assert torch.allclose(whole.float(), split.float(), rtol=2.0 ** -6, atol=2.0 ** -7 * float(whole.float().abs().max()))
    for i in range(6):
        assert torch.equal(ops.wo_swiglu_s8(x, wgu, sgu, balanced=True, overlap_previous=bool(i & 1)).view(torch.int16),
                           split.view(torch.int16))
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("gs", [64, 128])
@pytest.mark.parametrize("B,N,K", [(1, 14336, 4096), (4, 4096, 14336), (16, 4096, 4096), (32, 2064, 2048), (3, 2050, 2176)])
def test_group_matmul_streaming_kernel(ops, dtype, gs, B, N, K):
    """8-bit group-wise weights of 4 MB and more go through the streaming kernel: against the oracle's
    float64 product of the SAME packed codes, scales and biases, within the rounding bound of an
    fp32-accumulated result in the activation type (the bound counts |x| * (255 s + |b|) per term)."""
    g = torch.Generator(device="cuda").manual_seed(B + N + K + gs)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    p, s, b = ops.group_quantize(w, gs, 8)
    x = torch.randn(B, K, device="cuda", generator=g).to(dtype)
    y = ops.group_matmul(x, p, s, b, gs, 8)
    assert y.dtype == dtype and y.shape == (B, N)
    ref = O.group_matmul(x.double().cpu().numpy(), p.cpu().numpy(), host(s), host(b), gs, 8)
    mag = (x.double().abs() @ (255.0 * s.double().repeat_interleave(gs, 1) + b.double().abs().repeat_interleave(gs, 1)).T)
    assert_rounded_product(y, ref, mag.cpu().numpy(), K, dtype)
    again = ops.group_matmul(x, p, s, b, gs, 8, overlap_previous=True)
    assert torch.equal(again.view(torch.int16), y.view(torch.int16))
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("gs", [64, 128])
@pytest.mark.parametrize("B,N,K", [(1, 14336, 4096), (4, 4096, 14336), (8, 2064, 4160), (9, 4096, 4096), (16, 14336, 4096),
                                   (32, 2064, 4096), (3, 4100, 2176)])
def test_group_matmul_streaming_kernel_4bit(ops, dtype, gs, B, N, K):
    """4-bit codes in groups of 64 or 128, 4 MB of packed words and more: the streaming kernel, against the oracle's
    float64 product of the same packed words, scales and biases within the rounding bound of an
    fp32-accumulated result (|x| * (15 s + |b|) per term), and against the direct kernel, which serves the
    same words below that size; cold and warm launches agree bit for bit."""
    if K % gs:
        pytest.skip("K is not a whole number of groups")
    g = torch.Generator(device="cuda").manual_seed(B + N + K + gs)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    p, s, b = ops.group_quantize(w, gs, 4)
    assert p.shape == (N, K // 8) and N * K // 2 >= 4 << 20
    x = torch.randn(B, K, device="cuda", generator=g).to(dtype)
    y = ops.group_matmul(x, p, s, b, gs, 4)
    assert y.dtype == dtype and y.shape == (B, N)
    ref = O.group_matmul(x.double().cpu().numpy(), p.cpu().numpy(), host(s), host(b), gs, 4)
    mag = (x.double().abs() @ (15.0 * s.double().repeat_interleave(gs, 1) + b.double().abs().repeat_interleave(gs, 1)).T)
    assert_rounded_product(y, ref, mag.cpu().numpy(), K, dtype)
    rows = min(N, 64)  # a slice this small goes to the direct kernel
    small = ops.group_matmul(x, p[:rows].contiguous(), s[:rows].contiguous(), b[:rows].contiguous(), gs, 4)
    assert_rounded_product(small, ref[:, :rows], mag[:, :rows].cpu().numpy(), K, dtype)
    again = ops.group_matmul(x, p, s, b, gs, 4, overlap_previous=True)
    assert torch.equal(again.view(torch.int16), y.view(torch.int16))
    flush = torch.empty(384 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for i in range(2):
        flush.fill_(i)
        torch.cuda.synchronize()
        assert torch.equal(ops.group_matmul(x, p, s, b, gs, 4).view(torch.int16), y.view(torch.int16))
    assert ops.wo_linear_status() == 0


def test_group_matmul_4bit_streaming_places_every_nibble(ops):
    """One-hot activations against unit scales and zero biases return the codes themselves: every nibble of
    every word position of a K chunk lands in its own column."""
    N, K = 4096, 2048
    k = torch.arange(K, device="cuda").view(1, -1)
    n = torch.arange(N, device="cuda").view(-1, 1)
    codes = ((n * 5 + k * 3 + (k // 8)) % 16).to(torch.int64)
    words = (codes.view(N, K // 8, 8) << (4 * torch.arange(8, device="cuda"))).sum(-1)
    packed = words.to(torch.int32) if int(words.max()) < 2 ** 31 else (words - (words >= 2 ** 31) * 2 ** 32).to(torch.int32)
    s = torch.ones(N, K // 64, device="cuda")
    b = torch.zeros(N, K // 64, device="cuda")
    assert torch.equal(ops.group_dequantize(packed, s, b, 64, 4), codes.float())
    for start in range(0, K, 8):
        x = torch.zeros(8, K, device="cuda", dtype=torch.bfloat16)
        x[torch.arange(8), start + torch.arange(8)] = 1.0
        y = ops.group_matmul(x, packed, s, b, 64, 4)
        assert torch.equal(y.float(), codes[:, start:start + 8].T.float()), start
    assert ops.wo_linear_status() == 0


def test_group_matmul_accepts_a_view_that_starts_off_a_16_byte_boundary(ops):
    """A contiguous activation view into a larger storage (here: starting one element in) is copied to an
    aligned buffer by the front end instead of reaching the kernels' 16-byte loads."""
    g = torch.Generator(device="cuda").manual_seed(3)
    w = torch.randn(64, 128, device="cuda", generator=g)
    p, s, b = ops.group_quantize(w, 64, 8)
    store = torch.randn(2 * 128 + 8, device="cuda", generator=g).to(torch.bfloat16)
    x = store[1:1 + 2 * 128].view(2, 128)
    assert x.data_ptr() % 16 != 0 and x.is_contiguous()
    y = ops.group_matmul(x, p, s, b, 64, 8)
    assert torch.equal(y, ops.group_matmul(x.clone(), p, s, b, 64, 8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("bits,gs", [(8, 64), (4, 32)])
@pytest.mark.parametrize("M,N,K", [(33, 256, 512), (200, 1000, 1024)])
def test_group_wide_product_matches_the_decoded_weight(ops, dtype, bits, gs, M, N, K):
    """More than 32 rows: ``x @ decode(W)^T`` with the weight decoded to the activation type; 16-bit
    activations run on the library's tensor-core kernel (fp32 accumulation, one rounding of the result),
    so the output is the fp64 product of the same operands within that rounding; the module adds bias
    and ReLU in the same kernel and decodes once."""
    from lucid_b200.nn.quantized.mlx_linear import QuantizedLinearMLX
    from lucid_b200.quantization import _qgemm

    g = torch.Generator(device="cuda").manual_seed(M * 7 + bits)
    w = torch.randn(N, K, device="cuda", generator=g)
    p, s, b = ops.group_quantize(w, gs, bits)
    dense = ops.group_dequantize(p, s, b, gs, bits).to(dtype)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    ref = x.double() @ dense.double().T
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -24}[dtype]
    # fp32 accumulation of K terms plus one rounding to the output type
    bound = (x.double().abs() @ dense.double().abs().T) * (K * 2.0 ** -24) + ref.abs() * eps + 1e-30
    y = _qgemm.quantized_matmul(x, p, s, b, transpose=True, group_size=gs, bits=bits)
    assert y.dtype == dtype and y.shape == (M, N)
    assert bool(((y.double() - ref).abs() <= bound).all())

    lin = torch.nn.Linear(K, N).cuda()
    with torch.no_grad():
        lin.weight.copy_(w)
    m = QuantizedLinearMLX.from_float(lin, bits=bits, group_size=gs, relu=True)
    refm = torch.relu(ref + lin.bias.double())
    boundm = bound + refm.abs() * eps + lin.bias.double().abs() * 2.0 ** -23
    y1 = m(x)
    assert bool(((y1.double() - refm).abs() <= boundm).all())
    held = m._wide_cache["w"]
    assert torch.equal(m(x), y1) and m._wide_cache["w"] is held  # second forward: no second decode
    m.scales.mul_(2.0)  # an in-place change of a buffer invalidates the decoded copy
    y2 = m(x)
    assert m._wide_cache["w"] is not held
    ref2 = torch.relu(x.double() @ ops.group_dequantize(p, m.scales, b, gs, bits).to(dtype).double().T + lin.bias.double())
    assert float((y2.double() - ref2).abs().max()) <= float(ref2.abs().max()) * 4 * eps + 1e-3


@pytest.mark.parametrize("bits", [8, 4])
def test_group_linear_modules_chain_with_launch_overlap(ops, bits):
    """Two group-wise Linear modules back to back at a decode batch: from the second forward on the modules let
    each kernel fetch its weights while its predecessor drains; eager and CUDA-graph results stay those of the
    first forward."""
    from lucid_b200.nn.quantized.mlx_linear import QuantizedLinearMLX

    torch.manual_seed(bits)
    up = QuantizedLinearMLX.from_float(torch.nn.Linear(4096, 8192).cuda(), bits=bits, group_size=64, relu=True)
    down = QuantizedLinearMLX.from_float(torch.nn.Linear(8192, 4096).cuda(), bits=bits, group_size=64)
    x = (torch.randn(4, 4096, device="cuda") * 0.5).to(torch.bfloat16)
    first = down(up(x))
    dense = down(up(x.float())).to(torch.bfloat16)  # fp32 activations: the direct kernel
    assert float((first.float() - dense.float()).abs().max()) <= 0.02 * float(dense.float().abs().max()) + 1e-3
    for _ in range(3):
        assert torch.equal(down(up(x)).view(torch.int16), first.view(torch.int16))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = down(up(x))
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), first.view(torch.int16))
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("gs", [64, 128])
@pytest.mark.parametrize("B,N,K", [(5, 1024, 1024), (8, 1040, 2048), (16, 1024, 1024), (32, 2048, 1024), (4, 1024, 1024)])
def test_group_matmul_small_matrices_from_five_rows_on(ops, bits, gs, B, N, K):
    """Packed weights below 4 MB go to the streaming kernel from five rows on (four rows: the direct kernel);
    either way the result is the oracle's product of the same packed words within the rounding bound."""
    g = torch.Generator(device="cuda").manual_seed(B + N + K + gs + bits)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    p, s, b = ops.group_quantize(w, gs, bits)
    x = torch.randn(B, K, device="cuda", generator=g).to(torch.bfloat16)
    y = ops.group_matmul(x, p, s, b, gs, bits)
    ref = O.group_matmul(x.double().cpu().numpy(), p.cpu().numpy(), host(s), host(b), gs, bits)
    top = float(2 ** bits - 1)
    mag = (x.double().abs() @ (top * s.double().repeat_interleave(gs, 1) + b.double().abs().repeat_interleave(gs, 1)).T)
    assert_rounded_product(y, ref, mag.cpu().numpy(), K, torch.bfloat16)
    assert torch.equal(ops.group_matmul(x, p, s, b, gs, bits, overlap_previous=True).view(torch.int16), y.view(torch.int16))
    assert ops.wo_linear_status() == 0


@pytest.mark.parametrize("rows", [1, 4, 5, 17, 32])
@pytest.mark.parametrize("N,K", [(300, 328), (4096, 1024)])
def test_weight_only_linear_fp32_activations_route(ops, rows, N, K):
    """fp32 activations: up to four rows on the FP32 multiply-add kernel, five and more on the exact digit-plane
    product; both are the float64 product of the same codes within fp32 rounding of the result and of the
    accumulation."""
    from lucid_b200.nn.quantized.weight_only import WeightOnlyLinear, fp32_rows_take_the_gemv

    assert fp32_rows_take_the_gemv(4, N * K) and not fp32_rows_take_the_gemv(5, N * K)
    assert not fp32_rows_take_the_gemv(1, 14336 * 4096)
    torch.manual_seed(rows + N)
    m = WeightOnlyLinear.from_float(torch.nn.Linear(K, N).cuda())
    x = torch.randn(rows, K, device="cuda")
    y = m(x)
    assert y.dtype == torch.float32 and y.shape == (rows, N)
    w = m.weight_int8.double() * m.weight_scale.double()[:, None]
    ref = x.double() @ w.T + m.bias.double()
    bound = (x.double().abs() @ w.abs().T) * (K * 2.0 ** -24) + ref.abs() * 2.0 ** -23 + 1e-30
    assert bool(((y.double() - ref).abs() <= bound).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 9, 32])
@pytest.mark.parametrize("N,K", [(520, 1000), (300, 1001)])
def test_weight_only_linear_rows_of_odd_length(ops, dtype, rows, N, K):
    """K that is not a multiple of 16 keeps 16-bit activations off the tensor-core GEMV kernels too: few rows on
    the multiply-add kernel, more on the wide products; the result is the float64 product within the rounding of
    the activation type."""
    from lucid_b200.nn.quantized.weight_only import WeightOnlyLinear

    torch.manual_seed(rows + K)
    m = WeightOnlyLinear.from_float(torch.nn.Linear(K, N).cuda())
    x = torch.randn(rows, K, device="cuda").to(dtype)
    y = m(x)
    assert y.dtype == dtype and y.shape == (rows, N)
    w = m.weight_int8.double() * m.weight_scale.double()[:, None]
    ref = x.double() @ w.T + m.bias.double()
    eps = 2.0 ** -8 if dtype is torch.bfloat16 else 2.0 ** -23
    bound = (x.double().abs() @ w.abs().T) * (K * 2.0 ** -24) + ref.abs() * eps + 1e-6
    assert bool(((y.double() - ref).abs() <= bound).all())


@pytest.mark.parametrize("bits,gs", [(8, 64), (4, 64), (8, 128), (4, 128)])
@pytest.mark.parametrize("B,N,K", [(1, 14336, 4096), (4, 4096, 14336), (11, 8200, 4096), (32, 4096, 8192)])
def test_group_matmul_fp32_rows_on_the_streaming_kernel(ops, bits, gs, B, N, K):
    """fp32 activations against a packed weight of 4 MB and more: three bf16 addends per row through the streaming
    kernel with fp32 results.  The addends are exact, so the result is the oracle's float64 product within fp32
    accumulation error -- tighter than what a single 16-bit rounding of the activations would allow -- and the
    module and the functional entry point take the same route."""
    from lucid_b200._C.ops import group_fp32_rows_stream
    from lucid_b200.quantization import _qgemm

    assert group_fp32_rows_stream(torch.float32, B, N, K, gs, bits)
    assert not group_fp32_rows_stream(torch.float32, B, 1024, 1024, gs, bits)
    g = torch.Generator(device="cuda").manual_seed(B + N + K + gs + bits)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    p, s, b = ops.group_quantize(w, gs, bits)
    x = torch.randn(B, K, device="cuda", generator=g)
    y = ops.group_matmul(x, p, s, b, gs, bits)
    assert y.dtype == torch.float32 and y.shape == (B, N)
    ref = O.group_matmul(x.double().cpu().numpy(), p.cpu().numpy(), host(s), host(b), gs, bits)
    top = float(2 ** bits - 1)
    mag = (x.double().abs() @ (top * s.double().repeat_interleave(gs, 1) + b.double().abs().repeat_interleave(gs, 1)).T)
    err = np.abs(host(y).astype(np.float64) - ref)
    assert (err <= mag.cpu().numpy() * (K * 2.0 ** -24) + np.abs(ref) * 2.0 ** -22).all()
    assert float(err.max()) <= 2e-6 * float(mag.max())  # far inside a 16-bit rounding of x (2^-9)
    assert torch.equal(_qgemm.quantized_matmul(x, p, s, b, transpose=True, group_size=gs, bits=bits), y)
    assert torch.equal(ops.group_matmul(x, p, s, b, gs, bits, overlap_previous=True), y)
    assert ops.wo_linear_status() == 0
