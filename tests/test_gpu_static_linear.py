"""GPU parity of the statically quantized Linear (nnq.Linear / LinearReLU) and of the tensor-core
weight-only kernel under it, against the oracle's restatement of the reference's forward
(dequantize W -> fp32 linear -> (ReLU) -> fake-quantize, lucid/nn/quantized/linear.py:206-214)."""
import numpy as np
import pytest
import torch
from torch import nn

import lucid_b200.quantization as Q
from lucid_b200.nn import quantized as nnq
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


def accumulation_bound(x, wq, sw, K):
    """A-priori bound of an fp32-accumulated dot product against its exact value, per output:
    (number of accumulation steps) * 2^-23 * sum_k |x_k| |w_k| * s.  Steps: 3 K / 16 tensor-core
    instructions of the three-term bf16 kernel, K / 8 for a blocked host sgemm (what the oracle
    runs), a few for the epilogue."""
    terms = (np.abs(x).astype(np.float64) @ np.abs(wq).astype(np.float64).T) * np.asarray(sw, np.float64)[None, :]
    return (3 * K / 16 + K / 8 + 16) * 2.0 ** -23 * terms


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_widen_is_exact_and_padded(ops, dtype):
    q = torch.arange(-128, 128, device="cuda", dtype=torch.int16).to(torch.int8).repeat(5, 1)[:, :200].contiguous()
    w = ops.widen_s8(q, dtype)
    assert tuple(w.shape) == (5, 256) and w.dtype == dtype
    assert torch.equal(w[:, :200].float(), q.float()) and not bool(w[:, 200:].any())


@pytest.mark.parametrize("M,K", [(1, 64), (7, 100), (300, 512), (64, 4100)])
def test_split_terms_add_up_exactly(ops, M, K):
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = torch.randn(M, K, device="cuda", generator=g) * torch.logspace(-6, 6, K, device="cuda")
    x[0, 0] = 0.0
    terms, rs = ops.split_f32_bf16x3(x, want_rowsum=True)
    kp = (K + 63) // 64 * 64
    assert tuple(terms.shape) == (M, 3 * kp)
    t = terms.double().reshape(M, 3, kp)
    assert torch.equal(t.sum(1)[:, :K], x.double()), "x1 + x2 + x3 must be x, bit for bit"
    assert not bool(t[:, :, K:].any())
    assert torch.allclose(rs.double(), x.double().sum(1), rtol=1e-5, atol=1e-5 * float(x.abs().sum(1).max()))


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (33, 200, 320), (128, 256, 512), (129, 300, 1000), (600, 1000, 256),
                                   (2048, 512, 2048)])
def test_wo_gemm_three_term_product(ops, M, N, K, variant):
    """fp32 activations x int8 codes: the tensor-core result against the exact float64 product,
    elementwise within the accumulation bound and on average at fp32-GEMM level (the three bf16
    terms carry every bit of x, so nothing but the accumulation rounds)."""
    r = np.random.default_rng(M + N + K)
    x = (r.standard_normal((M, K)) * np.exp(r.standard_normal((M, K)))).astype(np.float32)
    wq = r.integers(-128, 128, (N, K)).astype(np.int8)
    sw = (r.random(N) * 0.01 + 1e-3).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    xt, wt = torch.tensor(x, device="cuda"), torch.tensor(wq, device="cuda")
    terms, _ = ops.split_f32_bf16x3(xt)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = ops.wo_gemm_16(terms, 3, ops.widen_s8(wt), sw=torch.tensor(sw, device="cuda"),
                       bias=torch.tensor(bias, device="cuda"), status=status, variant=variant)
    ops.qlinear_check_status(status)
    ref = (x.astype(np.float64) @ wq.astype(np.float64).T) * sw.astype(np.float64)[None, :] + bias[None, :]
    err = np.abs(y.double().cpu().numpy() - ref)
    bound = accumulation_bound(x, wq, sw, K) + 2.0 ** -22 * np.abs(ref)
    assert (err <= bound).all(), f"worst {float((err / bound).max()):.2f} x bound"
    # the tensor cores truncate when they add into the fp32 accumulator, so the error grows with the number of
    # accumulation steps instead of with its square root: 2.4e-6 of the output RMS at K = 512 (an IEEE fp32 GEMM: ~3e-7)
    assert np.sqrt((err ** 2).mean()) <= 5e-6 * max(1.0, K / 512) * np.sqrt((ref ** 2).mean()), "not at fp32-GEMM accuracy"
    # and against the fp32 host product the oracle uses
    w = O.dequantize(wq, sw, np.zeros(N, np.float32), ch_axis=0)
    err_o = np.abs(y.cpu().numpy().astype(np.float64) - O.linear_f32(x, w, bias))
    assert (err_o <= 2 * bound).all()


@pytest.mark.parametrize("M,K", [(1, 16), (33, 100), (300, 512), (64, 4100)])
def test_digit_planes_reassemble_the_rows(ops, M, K):
    """sum_d digit_d * 256^d * row_scale gives back every entry within 2^-6 of its row's maximum
    exactly, and every other entry to 2^-30 of that maximum; digits of the padding are zero."""
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = torch.randn(M, K, device="cuda", generator=g) * torch.logspace(-6, 2, K, device="cuda")
    x[0] = 0.0
    digits, scale, rs = ops.split_f32_digits(x, want_rowsum=True)
    kp = (K + 15) // 16 * 16
    assert tuple(digits.shape) == ((M + 31) // 32 * 128, kp) and digits.dtype == torch.int8
    d = digits.cpu().numpy().astype(np.int64).reshape(-1, 4, 32, kp)          # [tile, digit, row, k]
    X = sum(d[:, i] * 256 ** i for i in range(4)).reshape(-1, kp)[:M]
    assert not X[:, K:].any()
    s = scale.double().cpu().numpy()[:, None]
    assert np.all(np.log2(s[1:]) == np.round(np.log2(s[1:]))), "row scales are powers of two"
    back = X[:, :K] * s
    xh = x.double().cpu().numpy()
    rowmax = np.abs(xh).max(1, keepdims=True)
    big = np.abs(xh) >= rowmax * 2.0 ** -6
    assert np.array_equal(back[big], xh[big])
    assert (np.abs(back - xh) <= rowmax * 2.0 ** -30).all()
    assert (np.abs(X).max(1)[1:] >= 2 ** 29).all() and (np.abs(X) < 2 ** 30).all()
    assert torch.allclose(rs.double(), x.double().sum(1), rtol=1e-5, atol=1e-5 * float(x.abs().sum(1).max()))


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (33, 200, 320), (128, 256, 512), (129, 300, 1000), (600, 1000, 256),
                                   (2048, 512, 2048), (100, 260, 8192)])
def test_wo_gemm_digits_is_exact(ops, M, N, K, variant):
    """fp32 activations x int8 codes through the digit planes: the result equals the float64 value
    of sum_k X[m,k] * w[n,k] (X the integer image of the row), rounded once -- checked as
    |y - exact| <= 1.5 ulp of the three epilogue roundings -- and sits far inside fp32-GEMM error."""
    r = np.random.default_rng(M + N + K)
    x = (r.standard_normal((M, K)) * np.exp(r.standard_normal((M, K)))).astype(np.float32)
    wq = r.integers(-128, 128, (N, K)).astype(np.int8)
    sw = (r.random(N) * 0.01 + 1e-3).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    xt, wt = torch.tensor(x, device="cuda"), ops.pad_rows_to_16(torch.tensor(wq, device="cuda"))
    digits, scale, _ = ops.split_f32_digits(xt)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = ops.wo_gemm_digits(digits, scale, wt, sw=torch.tensor(sw, device="cuda"), bias=torch.tensor(bias, device="cuda"),
                           status=status, variant=variant)
    ops.qlinear_check_status(status)
    s = scale.double().cpu().numpy()[:, None]
    X = np.rint(x.astype(np.float64) / s)                       # the integers the kernel multiplies
    acc = X @ wq.astype(np.float64).T                            # exact: |acc| < 2^53
    prod = acc * s * sw.astype(np.float64)[None, :]
    ref = prod + bias[None, :]
    got = y.double().cpu().numpy()
    ulp = lambda v: 2.0 ** (np.floor(np.log2(np.maximum(np.abs(v), 1e-300))) - 23)
    assert (np.abs(got - ref) <= 1.5 * ulp(prod) + 0.5 * ulp(ref)).all()
    exact = (x.astype(np.float64) @ wq.astype(np.float64).T) * sw.astype(np.float64)[None, :] + bias[None, :]
    err = np.abs(got - exact)
    assert np.sqrt((err ** 2).mean()) <= 2e-7 * np.sqrt((exact ** 2).mean())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(40, 300, 328), (256, 512, 1024), (1000, 130, 72)])
def test_wo_gemm_single_term_16bit_activations(ops, dtype, M, N, K):
    from tolerances import abs_terms, assert_rounded_product

    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    wq = torch.randint(-128, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
    sw = torch.rand(N, device="cuda", generator=g) * 0.01 + 1e-3
    y = ops.wo_gemm_16(x, 1, ops.widen_s8(wq, dtype)[:, :K], sw=sw, out_dtype=dtype)
    ref = (x.double() @ wq.double().T) * sw.double()[None, :]
    assert_rounded_product(y, ref.cpu().numpy(), abs_terms(x, wq, sw, offset=0.0), K, dtype)


def calibrated(relu: bool, rows: int, affine_weights: bool = False, ch_axis: int = 0):
    torch.manual_seed(11 + rows + int(relu))
    K, N = 320, 200
    lin = nn.Linear(K, N)
    with torch.no_grad():
        lin.weight.normal_(0.0, 0.05)
        lin.weight[:, 7] += 0.2  # a lopsided column so that affine weight grids get non-zero zero-points
        lin.bias.normal_(0.0, 0.1)
    model = nn.Sequential(lin, nn.ReLU()) if relu else nn.Sequential(lin)
    if relu:
        model = Q.fuse_modules(model.eval(), [["0", "1"]])
    weight_obs = Q.get_default_qconfig().weight
    if affine_weights:
        from lucid_b200.quantization._qscheme import per_channel_affine, qint8

        weight_obs = Q.PerChannelMinMaxObserver.with_args(ch_axis=ch_axis, qscheme=per_channel_affine, qdtype=qint8)
    elif ch_axis != 0:
        from lucid_b200.quantization._qscheme import per_channel_symmetric, qint8

        weight_obs = Q.PerChannelMinMaxObserver.with_args(ch_axis=ch_axis, qscheme=per_channel_symmetric, qdtype=qint8)
    qcfg = Q.QConfig(activation=Q.MinMaxObserver.with_args(), weight=weight_obs)
    prepared = Q.prepare(model, qcfg).cuda()
    x = torch.randn(rows, K, device="cuda")
    prepared(x)
    return Q.convert(prepared), x


def check_against_oracle(qlin, x, relu):
    wq = qlin.weight_int8.cpu().numpy()
    sw = qlin.weight_scale.cpu().numpy()
    zw = qlin.weight_zero_point.cpu().numpy()
    b = qlin.bias.cpu().numpy()
    S, Z = float(qlin.scale), float(qlin.zero_point)
    xh = x.cpu().numpy()
    want = O.static_linear_reference(xh, wq, sw, zw, b, np.float32(S), np.float32(Z), O.quint8, relu=relu,
                                     ch_axis=qlin.weight_ch_axis)
    with torch.no_grad():
        got = qlin(x).cpu().numpy()
    assert got.dtype == np.float32 and got.shape == want.shape
    # exact pre-requant value and how far either fp32 evaluation may sit from it
    w64 = O.dequantize(wq, sw, zw, ch_axis=qlin.weight_ch_axis if np.size(sw) > 1 else None).astype(np.float64)
    y64 = xh.astype(np.float64) @ w64.T + b
    if relu:
        y64 = np.maximum(y64, 0.0)
    K = xh.shape[1]
    tol = (3 * K / 16 + K / 8 + 16) * 2.0 ** -23 * (np.abs(xh).astype(np.float64) @ np.abs(w64).T) + 2.0 ** -22 * np.abs(y64)
    code = y64 / S
    near_edge = np.abs(code - np.floor(code) - 0.5) <= 2 * tol / S
    assert near_edge.mean() < 0.1, "the (worst-case) tolerance band around grid edges should stay narrow"
    assert np.array_equal(got[~near_edge], want[~near_edge]), "requantized output differs away from a grid edge"
    assert (np.abs(got[near_edge] - want[near_edge]) <= S * 1.0001).all(), "more than one grid step at an edge"
    assert (got != want).mean() < 0.005, "far more outputs flipped a grid step than fp32 rounding explains"
    return int(near_edge.sum()), int((got != want).sum())


@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("rows", [1, 4, 5, 32, 256])
def test_static_linear_matches_oracle(relu, rows):
    """Both routes (GEMV kernel for up to 4 rows, tensor-core kernel from 5 on) of Linear and LinearReLU:
    equal to the oracle everywhere except within the fp32 accumulation tolerance of a grid edge,
    where one grid step is allowed."""
    qm, x = calibrated(relu, rows)
    qlin = qm[0]
    assert type(qlin) is (nnq.LinearReLU if relu else nnq.Linear)
    edge, differ = check_against_oracle(qlin, x, relu)
    assert differ <= edge


@pytest.mark.parametrize("rows", [4, 7, 256])
@pytest.mark.parametrize("ch_axis", [0, 1])
def test_static_linear_affine_weights(rows, ch_axis):
    """Weight grids with a zero-point (affine weight observer) and scales along the input axis go
    through the tensor-core kernel's rowsum x colcorr term."""
    qm, x = calibrated(False, rows, affine_weights=True, ch_axis=ch_axis)
    qlin = qm[0]
    assert bool((qlin.weight_zero_point != 0).any())
    edge, differ = check_against_oracle(qlin, x, False)
    assert differ <= edge


def test_static_linear_large_shape_route():
    """An FFN-sized layer (8192 x 2048 x 512) through the module: pair kernel, several waves."""
    torch.manual_seed(5)
    lin = nn.Linear(512, 2048).cuda()
    prepared = Q.prepare(nn.Sequential(lin), Q.QConfig(activation=Q.MinMaxObserver.with_args(),
                                                     weight=Q.get_default_qconfig().weight))
    x = torch.randn(8192, 512, device="cuda")
    prepared(x)
    qlin = Q.convert(prepared)[0]
    rows = np.r_[0:130, 4000:4100, 8000:8192]
    with torch.no_grad():
        got = qlin(x)[rows].cpu().numpy()
    want = O.static_linear_reference(x[rows].cpu().numpy(), qlin.weight_int8.cpu().numpy(), qlin.weight_scale.cpu().numpy(),
                                     qlin.weight_zero_point.cpu().numpy(), qlin.bias.cpu().numpy(),
                                     np.float32(float(qlin.scale)), np.float32(float(qlin.zero_point)), O.quint8)
    S = float(qlin.scale)
    assert (np.abs(got - want) <= S * 1.0001).all()
    assert (got != want).mean() < 0.01


def test_bounded_waits_run_out_and_report(ops):
    """Wait test of the GEMM kernels: the producer issues nothing, every wait gives up after a few
    thousand cycles, the kernel returns, the status word maps to LC_ERR_TIMEOUT, and the next
    ordinary launch is correct."""
    from lucid_b200._C import LC_ERR_TIMEOUT, LucidCudaError

    g = torch.Generator(device="cuda").manual_seed(0)
    for M in (64, 512):  # single-CTA kernel and CTA-pair kernel
        a = torch.randint(-128, 128, (M, 256), device="cuda", dtype=torch.int8, generator=g)
        b = torch.randint(-128, 128, (512, 256), device="cuda", dtype=torch.int8, generator=g)
        sx, sw = torch.rand(M, device="cuda"), torch.rand(512, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.qlinear_i8(a, b, sx, sw, status=status, variant=256)
        with pytest.raises(LucidCudaError) as info:
            ops.qlinear_check_status(status)
        assert info.value.code == LC_ERR_TIMEOUT and "ran out" in str(info.value)
        assert int(status.item()) == 0  # cleared
        acc = ops.qlinear_i8(a, b, None, None, out_dtype=torch.int32, status=status)
        ops.qlinear_check_status(status)
        assert torch.equal(acc.cpu(), (a.cpu().int() @ b.cpu().int().T))
        x = torch.randn(M, 256, device="cuda", generator=g).to(torch.bfloat16)
        ops.wo_gemm_16(x, 1, ops.widen_s8(b), status=status, wait_test=True)
        with pytest.raises(LucidCudaError) as info:
            ops.qlinear_check_status(status)
        assert info.value.code == LC_ERR_TIMEOUT
        y = ops.wo_gemm_16(x, 1, ops.widen_s8(b), status=status)
        ops.qlinear_check_status(status)
        assert torch.allclose(y.double(), x.double() @ b.double().T, rtol=1e-5, atol=1e-3)
        digits, scale, _ = ops.split_f32_digits(x.float())
        ops.wo_gemm_digits(digits, scale, b, status=status, wait_test=True)
        with pytest.raises(LucidCudaError) as info:
            ops.qlinear_check_status(status)
        assert info.value.code == LC_ERR_TIMEOUT
        y = ops.wo_gemm_digits(digits, scale, b, status=status)
        ops.qlinear_check_status(status)
        assert torch.allclose(y.double(), x.double() @ b.double().T, rtol=1e-6, atol=1e-4)
