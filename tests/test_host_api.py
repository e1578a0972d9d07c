"""Host-side mirror of the reference API: same names, arguments, buffers, warnings and
error types.  Every case runs twice: on the CPU with an oracle-backed stand-in for the
kernel front end (checks the Python logic only), and on a GPU with the real kernels."""
import copy
import warnings

import numpy as np
import pytest
import torch
from torch import nn

import lucid_b200 as lucid
import lucid_b200.quantization as Q
from lucid_b200 import _backend
from lucid_b200.nn import quantized as nnq
from lucid_b200.nn.quantized import dynamic as nnqd


@pytest.fixture(params=["cpu-standin", pytest.param("cuda", marks=pytest.mark.gpu)])
def device(request, monkeypatch):
    if request.param == "cpu-standin":
        from tests import fake_ops

        cpu = torch.device("cpu")
        monkeypatch.setattr(_backend, "ops", lambda: fake_ops)
        monkeypatch.setattr(_backend, "on_cuda", lambda t: t.to(cpu))
        monkeypatch.setattr(_backend, "cuda_device", lambda index=None: cpu)
        return "cpu"
    return "cuda"


def T(a, device, **kw):
    return torch.tensor(a, device=device, dtype=torch.float32, **kw)


# ---- primitives (lucid/test/unit/quantization/test_functional.py) -------------------
def test_public_names():
    for name in ("QScheme", "QDtype", "qint8", "quint8", "qint32", "qint4", "QParams", "calculate_qparams",
                 "quantize", "dequantize", "fake_quantize", "MinMaxObserver", "PerChannelMinMaxObserver",
                 "HistogramObserver", "PlaceholderObserver", "FakeQuantize", "QConfig", "QConfigMapping",
                 "prepare", "convert", "quantize_dynamic", "get_default_qconfig"):
        assert name in Q.__all__ and hasattr(Q, name)
    assert (Q.qint8.quant_min, Q.qint8.quant_max) == (-128, 127)
    assert (Q.quint8.quant_min, Q.quint8.quant_max, Q.quint8.storage) == (0, 255, "int16")
    assert repr(Q.qint8) == "lucid.quantization.qint8"
    assert Q.per_channel_symmetric.is_per_channel and Q.per_tensor_symmetric.is_symmetric
    assert not Q.per_tensor_affine.is_per_channel and not Q.per_channel_affine.is_symmetric
    for qd in (Q.qint8, Q.quint8, Q.qint32, Q.qint4):
        assert isinstance(getattr(lucid, qd.storage), lucid.dtype)


def test_quantize_dequantize(device):
    x = T([-1.0, -0.3, 0.0, 0.7, 2.0], device)
    q = Q.quantize(x, 0.05, 0.0, Q.qint8)
    assert q.dtype is torch.int8
    assert np.allclose(Q.dequantize(q, 0.05, 0.0).cpu().numpy(), x.cpu().numpy(), atol=1e-6)
    assert Q.quantize(T([-1000.0, 1000.0], device), 0.1, 0.0, Q.qint8).tolist() == [-128, 127]
    assert Q.quantize(T([0.0], device), 0.02, 128.0, Q.quint8).item() == 128


def test_fake_quantize_and_ste(device):
    x = T([-1.0, -0.31, 0.0, 0.72, 2.0], device)
    fq = Q.fake_quantize(x, 0.05, 0.0, -128, 127)
    dq = Q.dequantize(Q.quantize(x, 0.05, 0.0, Q.qint8), 0.05, 0.0)
    assert np.allclose(fq.cpu().numpy(), dq.cpu().numpy(), atol=1e-6)
    xg = T([-100.0, 0.2, 0.5, 100.0], device, requires_grad=True)
    Q.fake_quantize(xg, 0.05, 0.0, -128, 127).sum().backward()
    assert xg.grad.tolist() == [0.0, 1.0, 1.0, 0.0]
    w = T([[1.0, 2.0, 300.0], [-400.0, 0.5, 0.1]], device, requires_grad=True)
    Q.fake_quantize(w, T([0.02, 0.03], device), T([0.0, 0.0], device), -128, 127, ch_axis=0).sum().backward()
    assert w.grad.tolist() == [[1.0, 1.0, 0.0], [0.0, 1.0, 1.0]]


def test_calculate_qparams(device):
    s, z = Q.calculate_qparams(-1.0, 3.0, Q.per_tensor_affine, Q.quint8)
    assert s.item() == pytest.approx(4.0 / 255.0, rel=1e-5) and 0.0 <= z.item() <= 255.0
    s, z = Q.calculate_qparams(-2.5, 2.0, Q.per_tensor_symmetric, Q.qint8)
    assert z.item() == 0.0 and s.item() == float(np.float32(2.5) / np.float32(127.5))
    s, _ = Q.calculate_qparams(0.0, 0.0, Q.per_tensor_affine, Q.qint8)
    assert s.item() > 0.0


def test_symmetric_extremum(device):
    """test_functional.py:114-139."""
    data = np.random.default_rng(0).standard_normal((64, 256)).astype(np.float32)
    obs = Q.PerChannelMinMaxObserver(ch_axis=1)
    obs(T(data, device))
    scale, zp = obs.calculate_qparams()
    x = T(data, device, requires_grad=True)
    Q.fake_quantize(x, scale, zp, -128, 127, ch_axis=1).sum().backward()
    codes = np.round(data * (np.float32(1.0) / scale.cpu().numpy()))
    expected = ((codes >= -128) & (codes <= 127)).astype(np.float32)
    assert (expected == 0.0).any()
    np.testing.assert_array_equal(x.grad.cpu().numpy(), expected)
    q = Q.quantize(x.detach(), scale, zp, Q.qint8, ch_axis=1)
    np.testing.assert_array_equal(q.cpu().numpy(), np.clip(codes, -128, 127))


# ---- observers (lucid/test/unit/quantization/test_observer.py) ------------------------
def test_observers(device):
    obs = Q.MinMaxObserver()
    x = T([[-1.0, 2.0], [0.5, 3.0]], device)
    assert obs(x) is x
    obs(T([[-2.0, 1.0]], device))
    assert obs.min_val.item() == -2.0 and obs.max_val.item() == 3.0
    obs = Q.MinMaxObserver(qscheme=Q.per_tensor_affine, qdtype=Q.quint8)
    obs(T([-1.0, 3.0], device))
    s, z = obs.calculate_qparams()
    assert s.item() == pytest.approx(4.0 / 255.0, rel=1e-5) and 0.0 <= z.item() <= 255.0
    ema = Q.MovingAverageMinMaxObserver(averaging_constant=0.5)
    ema(T([-2.0, 2.0], device))
    ema(T([-4.0, 4.0], device))
    assert ema.min_val.item() == pytest.approx(-3.0) and ema.max_val.item() == pytest.approx(3.0)
    pc = Q.PerChannelMinMaxObserver(ch_axis=0)
    pc(T([[1.0, 2.0, 3.0], [-4.0, 0.5, 0.1]], device))
    assert pc.min_val.tolist() == [1.0, -4.0] and pc.max_val.tolist() == [3.0, 0.5]
    s, z = pc.calculate_qparams()
    assert s.shape == (2,) and z.tolist() == [0.0, 0.0]
    with pytest.raises(RuntimeError, match="collects no statistics"):
        Q.PlaceholderObserver().calculate_qparams()
    fx = Q.FixedQParamsObserver(1.0 / 256, 0)
    assert fx.calculate_qparams()[0].item() == 1.0 / 256


def test_histogram_observer(device):
    g = torch.Generator().manual_seed(0)
    data = torch.randn(2000, generator=g)
    obs = Q.HistogramObserver(bins=256)
    obs(data.to(device))
    assert obs.histogram.sum().item() == pytest.approx(2000, abs=2)
    assert obs.calculate_qparams()[0].item() > 0.0
    tail = torch.cat([torch.randn(3000, generator=g), torch.rand(150, generator=g) * 7 + 5])
    h, m = Q.HistogramObserver(bins=512), Q.MinMaxObserver()
    h(tail.to(device))
    m(tail.to(device))
    assert h.calculate_qparams()[0].item() <= m.calculate_qparams()[0].item()


def test_observer_state_dict_round_trip(device):
    obs = Q.MinMaxObserver()
    obs(T([-2.0, 5.0], device))
    sd = obs.state_dict()
    assert set(sd) == {"min_val", "max_val"}
    fresh = Q.MinMaxObserver()
    fresh.load_state_dict(sd)
    assert fresh.min_val.item() == -2.0 and fresh.max_val.item() == 5.0
    pc = Q.PerChannelMinMaxObserver(ch_axis=0)
    pc(T([[1.0, 2.0], [-4.0, 0.5], [0.0, 9.0]], device))
    fresh = Q.PerChannelMinMaxObserver(ch_axis=0)
    fresh.load_state_dict(pc.state_dict())
    assert fresh.max_val.tolist() == [2.0, 0.5, 9.0]


def test_fake_quantize_module(device):
    fq = Q.FakeQuantize(observer=Q.MinMaxObserver)
    fq(T([-1.0, 0.0, 2.0], device))
    frozen = fq.scale.item()
    assert frozen > 0.0
    fq.disable_observer()
    fq(T([-100.0, 100.0], device))
    assert fq.scale.item() == frozen
    ident = Q.FakeQuantize(observer=Q.MinMaxObserver).disable_fake_quant()
    x = T([0.123, -4.5, 7.8], device)
    assert torch.equal(ident(x), x)


def test_qconfig_mapping():
    qc, qat = Q.get_default_qconfig(), Q.get_default_qat_qconfig()
    assert isinstance(qc.weight(), Q.PerChannelMinMaxObserver) and isinstance(qc.activation(), Q.HistogramObserver)
    assert isinstance(qat.weight(), Q.FakeQuantize)
    m = Q.QConfigMapping().set_global(qc).set_object_type(nn.Linear, qat).set_module_name("head", None)
    assert m.get_qconfig(nn.Conv2d, "backbone") is qc
    assert m.get_qconfig(nn.Linear, "fc") is qat
    assert m.get_qconfig(nn.Linear, "head") is None


def test_backend_selector():
    be = lucid.backends.quantized
    assert be.engine == "auto" and not be.use_mlx()
    with pytest.raises(ValueError, match="quantized.engine must be"):
        be.engine = "tensorrt"
    for value in ("reference", "mlx_group", "cuda_int8", "auto"):
        be.engine = value
        assert be.use_mlx() == (value == "mlx_group")
    with pytest.raises(ValueError, match="Apple-only"):
        lucid.device("metal")
    assert lucid.device("cuda:0").type == "cuda"


# ---- dynamic PTQ (test_dynamic_ptq.py, test_qconfig_propagation.py:236-382) ---------------
def mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16))


def test_quantize_dynamic_swaps_and_is_accurate(device):
    model = mlp()
    qm = Q.quantize_dynamic(model)
    assert isinstance(qm[0], nnqd.Linear) and isinstance(qm[2], nnqd.Linear) and isinstance(qm[1], nn.ReLU)
    assert isinstance(model[0], nn.Linear), "the input model must not be modified"
    assert not any(hasattr(m, "qconfig") for m in qm.modules())
    assert set(qm[0].state_dict()) == {"weight_int8", "weight_scale", "weight_zero_point", "bias"}
    assert qm[0].weight_int8.dtype is torch.int8 and tuple(qm[0].weight_int8.shape) == (64, 32)
    x = torch.randn(8, 32)
    ref = model(x)
    out = qm(x.to(device)).cpu()
    assert out.shape == ref.shape
    assert (out - ref).abs().mean() / ref.abs().mean() < 0.05
    # three activation grids, leading dims are flattened like F.linear does
    for scheme in ("tensor_affine", "tensor_symmetric", "token_symmetric"):
        qm[0].set_activation_scheme(scheme)
        y = qm[0](x.to(device).reshape(2, 4, 32))
        assert tuple(y.shape) == (2, 4, 64)
        assert (y.reshape(8, 64).cpu() - model[0](x)).abs().mean() / model[0](x).abs().mean() < 0.05


def test_quantize_dynamic_spec_forms(device):
    assert isinstance(Q.quantize_dynamic(mlp(), {nn.Linear})[0], nnqd.Linear)
    assert isinstance(Q.quantize_dynamic(mlp(), {nn.Linear: Q.qint8})[2], nnqd.Linear)
    by_name = Q.quantize_dynamic(mlp(), {"0"})
    assert isinstance(by_name[0], nnqd.Linear) and isinstance(by_name[2], nn.Linear)
    skip = Q.quantize_dynamic(mlp(), {nn.Linear: Q.qint8, "2": None})
    assert isinstance(skip[0], nnqd.Linear) and isinstance(skip[2], nn.Linear)
    bare = Q.quantize_dynamic(nn.Linear(8, 4))
    assert isinstance(bare, nnqd.Linear)
    model = mlp()
    model[2].qconfig = None  # a module attribute beats a mapping rule
    assert isinstance(Q.quantize_dynamic(model)[2], nn.Linear)
    with pytest.warns(UserWarning, match="no module of a targeted type"):
        Q.quantize_dynamic(nn.Sequential(nn.ReLU()), {"missing"})
    with pytest.warns(UserWarning, match="no dynamically quantized form"):
        Q.quantize_dynamic(nn.Sequential(nn.ReLU()), {nn.ReLU})
    with pytest.raises(TypeError, match="qconfig_spec must be"):
        Q.quantize_dynamic(mlp(), 3)
    with pytest.raises(TypeError, match="keys must be"):
        Q.quantize_dynamic(mlp(), {3: Q.qint8})
    with pytest.raises(TypeError, match="must be a QConfig, a QDtype or None"):
        Q.quantize_dynamic(mlp(), {nn.Linear: "int8"})


def test_dynamic_linear_state_dict_round_trip(device):
    qm = Q.quantize_dynamic(mlp())
    x = torch.randn(4, 32).to(device)
    y = qm(x)
    fresh = Q.quantize_dynamic(nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16)))
    fresh.load_state_dict(qm.state_dict(), strict=True)
    assert torch.equal(fresh(x), y)
    clone = copy.deepcopy(qm)
    assert torch.equal(clone(x), y)


# ---- static PTQ and the group-wise engine -----------------------------------------------
def test_prepare_convert_static(device):
    model = mlp()
    prepared = Q.prepare(model)
    assert hasattr(prepared[0], "activation_post_process") and isinstance(prepared[0].qconfig, Q.QConfig)
    x = torch.randn(64, 32)
    prepared = prepared.to(device)
    for _ in range(2):
        prepared(x.to(device))
    qm = Q.convert(prepared)
    assert isinstance(qm[0], nnq.Linear) and isinstance(qm[2], nnq.Linear)
    assert not any(hasattr(m, "qconfig") for m in qm.modules())
    assert {"weight_int8", "weight_scale", "weight_zero_point", "bias", "scale", "zero_point"} == set(
        qm[0].state_dict())
    ref = model(x)
    for rows in (x[:4], x):  # GEMV-shaped and dense routes
        out = qm(rows.to(device)).cpu()
        assert (out - ref[: rows.shape[0]]).abs().mean() / ref.abs().mean() < 0.08
    with pytest.warns(UserWarning, match="matched no quantizable modules"):
        Q.prepare(nn.Sequential(nn.ReLU()))
    with pytest.warns(UserWarning, match="never saw data"):
        Q.convert(Q.prepare(mlp(), Q.QConfig(activation=Q.MinMaxObserver.with_args(),
                                              weight=Q.get_default_qconfig().weight)))


def test_group_engine_routing(device):
    be = lucid.backends.quantized
    be.engine = "mlx_group"
    try:
        qm = Q.quantize_dynamic(nn.Sequential(nn.Linear(128, 64), nn.ReLU(), nn.Linear(64, 20)))
        assert isinstance(qm[0], nnq.QuantizedLinearMLX) and qm[0].group_size == 64 and qm[0].bits == 8
        assert qm[0].packed_weight.dtype is torch.int32 and tuple(qm[0].packed_weight.shape) == (64, 32)
        assert tuple(qm[0].scales.shape) == (64, 2)
        odd = Q.quantize_dynamic(nn.Linear(20, 8))  # no group size divides 20 -> per-channel module
        assert isinstance(odd, nnqd.Linear)
    finally:
        be.engine = "auto"
    torch.manual_seed(1)
    lin = nn.Linear(128, 64)
    m = nnq.QuantizedLinearMLX.from_float(lin, bits=8, group_size=64)
    x = torch.randn(2, 128)
    out = m(x.to(device)).cpu()
    assert (out - lin(x)).abs().max() / lin(x).abs().max() < 0.02   # test_real_gemm.py:44-63
    m4 = nnq.QuantizedLinearMLX.from_float(lin, bits=4, group_size=64)
    assert (m4(x.to(device)).cpu() - lin(x)).abs().max() / lin(x).abs().max() < 0.15
    assert m.packed_weight.numel() * 4 < lin.weight.numel() * 4 / 2   # packed bytes < half
    fresh = nnq.QuantizedLinearMLX(128, 64, bits=8, group_size=64)
    fresh.load_state_dict(m.state_dict(), strict=True)                # test_real_gemm.py:75-90
    assert torch.allclose(fresh(x.to(device)).cpu(), out, atol=1e-4)


def test_group_linear_above_32_rows_decodes_once(device):
    """More than 32 rows: the module hands the decoded weight, its bias and ReLU to the tensor-core product and
    keeps the decoded copy until a buffer changes in place; the rows agree with the 32-row path."""
    torch.manual_seed(5)
    lin = nn.Linear(128, 48)
    m = nnq.QuantizedLinearMLX.from_float(lin, bits=8, group_size=64, relu=True)
    x = torch.randn(3, 20, 128).to(torch.bfloat16).to(device)
    wide = m(x)
    assert wide.shape == (3, 20, 48) and wide.dtype is torch.bfloat16
    held = m._wide_cache["w"]
    assert held.dtype is torch.bfloat16 and tuple(held.shape) == (48, 128)
    m(x)
    assert m._wide_cache["w"] is held
    narrow = torch.cat([m(x[i]) for i in range(3)]).reshape(3, 20, 48)
    assert (wide.float() - narrow.float()).abs().max() <= 0.02 * narrow.float().abs().max()
    m.biases.add_(0.01)
    m(x)
    assert m._wide_cache["w"] is not held


@pytest.mark.gpu
def test_forward_from_host_matches_whole_batch():
    from lucid_b200.nn.quantized.streaming import forward_from_host

    torch.manual_seed(3)
    lin = nn.Linear(96, 80)
    q = Q.quantize_dynamic(lin).set_activation_scheme("token_symmetric")
    x = torch.randn(1000, 96).pin_memory()
    out = torch.empty(1000, 80).pin_memory()
    forward_from_host(q, x, out, chunk_rows=192)
    torch.cuda.synchronize()
    assert torch.equal(out, q(x.cuda()).cpu())
    q.set_activation_scheme("tensor_affine")
    with pytest.raises(ValueError, match="per-row"):
        forward_from_host(q, x, out)


@pytest.mark.gpu
def test_weight_only_modules():
    torch.manual_seed(5)
    H, F = 256, 512
    gate, up, down = nn.Linear(H, F, bias=False), nn.Linear(H, F, bias=False), nn.Linear(F, H, bias=False)
    mlp = nnq.WeightOnlySwiGLU.from_float(gate, up, down)
    assert set(mlp.state_dict()) == {"gate_up_int8", "gate_up_scale", "down.weight_int8", "down.weight_scale"}
    ref = lambda x: down(torch.nn.functional.silu(gate(x)) * up(x))
    for rows, dtype in ((4, torch.bfloat16), (4, torch.float32), (100, torch.bfloat16)):
        x = torch.randn(rows, H)
        y = mlp(x.cuda().to(dtype)).float().cpu()
        assert (y - ref(x)).abs().mean() / ref(x).abs().mean() < 0.05
    lin = nn.Linear(H, F)
    wo = nnq.WeightOnlyLinear.from_float(lin)
    x = torch.randn(3, 7, H)
    assert tuple(wo(x.cuda().bfloat16()).shape) == (3, 7, F)
    assert (wo(x.cuda()).cpu() - lin(x)).abs().mean() / lin(x).abs().mean() < 0.02


# ---- stubs, functional merges, differentiable quantized_matmul ---------------------------
class _ResidualBlock(nn.Module):
    """quant -> fc1 -> relu -> fc2 -> (+ skip, relu) -> dequant, the shape of the reference's
    FloatFunctional example (lucid/nn/quantized/functional_module.py)."""

    def __init__(self) -> None:
        super().__init__()
        self.quant, self.dequant = nnq.QuantStub(), nnq.DeQuantStub()
        self.fc1, self.act, self.fc2 = nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 32)
        self.skip = nnq.FloatFunctional()

    def forward(self, x):
        x = self.quant(x)
        return self.dequant(self.skip.add_relu(self.fc2(self.act(self.fc1(x))), x))


def test_static_workflow_with_stubs_and_functional(device):
    torch.manual_seed(0)
    model = _ResidualBlock()
    ff = nnq.FloatFunctional()
    a, b = torch.randn(4), torch.randn(4)
    assert torch.equal(ff.add(a, b), a + b) and torch.equal(ff.mul_scalar(a, 2.0), a * 2.0)  # passthrough
    x = torch.randn(48, 32)
    ref = model(x)
    prepared = Q.prepare(model).to(device)
    assert all(hasattr(m, "activation_post_process") for m in (prepared.quant, prepared.skip, prepared.fc1))
    assert not hasattr(prepared.dequant, "activation_post_process")
    for _ in range(2):
        prepared(x.to(device))
    qm = Q.convert(prepared)
    assert isinstance(qm.quant, nnq.Quantize) and isinstance(qm.dequant, nnq.DeQuantize)
    assert isinstance(qm.skip, nnq.QFunctional) and isinstance(qm.fc1, nnq.Linear)
    assert set(qm.skip.state_dict()) == {"scale", "zero_point"} == set(qm.quant.state_dict())
    out = qm(x.to(device)).cpu()
    assert (out - ref).abs().mean() / ref.abs().mean() < 0.1
    # every output of the merge lies on its calibrated grid
    s, z = float(qm.skip.scale), float(qm.skip.zero_point)
    codes = out / s + z
    assert float((codes - codes.round()).abs().max()) < 1e-3 and float(out.min()) >= 0.0
    # integer inputs pass the Quantize marker untouched
    idx = torch.arange(6)
    assert torch.equal(qm.quant(idx), idx)
    wrapped = nnq.QuantWrapper(nn.Linear(4, 4))
    assert isinstance(wrapped.quant, nnq.QuantStub) and isinstance(wrapped.dequant, nnq.DeQuantStub)


def test_qfunctional_merges_match_unfused_definition(device):
    torch.manual_seed(3)
    qf = nnq.QFunctional(torch.tensor(0.05), torch.tensor(12.0)).to(device)
    a, b = torch.randn(7, 33).to(device), torch.randn(7, 33).to(device)
    fq = lambda t: Q.fake_quantize(t, qf.scale, qf.zero_point, 0, 255)  # noqa: E731
    assert torch.equal(qf.add(a, b), fq(a + b))
    assert torch.equal(qf.mul(a, b), fq(a * b))
    assert torch.equal(qf.add_relu(a, b), fq(torch.relu(a + b)))
    assert torch.equal(qf.add_scalar(a, 0.3), fq(a + 0.3))
    assert torch.equal(qf.mul_scalar(a, -1.7), fq(a * -1.7))
    assert torch.equal(qf.cat([a, b], dim=1), fq(torch.cat([a, b], dim=1)))
    row = torch.randn(33).to(device)  # broadcasting merge
    assert torch.equal(qf.add(a, row), fq(a + row))


@pytest.mark.parametrize("kind", ["LSTM", "GRU", "LSTMCell", "GRUCell", "RNNCell"])
def test_dynamic_recurrent(device, kind):
    """int8 weight buffers under the float module's flat names, float biases, the float shell
    outside state_dict; output within weight-quantization error of the float module."""
    torch.manual_seed(2)
    cell = kind.endswith("Cell")
    fl = getattr(nn, kind)(16, 24) if cell else getattr(nn, kind)(16, 24, num_layers=2, batch_first=True)
    q = getattr(nnqd, kind).from_float(fl)
    keys = set(q.state_dict())
    names = [n for n, _ in fl.named_parameters()]
    want = {n + "_int8" for n in names if n.startswith("weight")} | {n + "_scale" for n in names if n.startswith("weight")} \
        | {n for n in names if n.startswith("bias")}
    assert keys == want
    assert all(q.state_dict()[k].dtype is torch.int8 for k in keys if k.endswith("_int8"))
    x = torch.randn(5, 16) if cell else torch.randn(3, 7, 16)
    ref = fl(x)
    out = q(x.to(device))
    ref0, out0 = (ref[0], out[0]) if isinstance(ref, tuple) else (ref, out)
    assert out0.shape == ref0.shape
    assert (out0.cpu() - ref0).abs().max() < 0.05
    with pytest.raises(TypeError, match="expects an nn."):
        getattr(nnqd, kind).from_float(nn.Linear(2, 2))
    swapped = Q.quantize_dynamic(nn.Sequential(fl) if cell else nn.ModuleDict({"rnn": fl}))
    assert isinstance(next(swapped.children()), getattr(nnqd, kind))


def test_reference_module_paths_resolve_to_the_same_modules():
    """Code written against the reference imports ``lucid...``; each such path must be the
    package's own module object (a second copy would break isinstance checks in convert)."""
    import importlib

    import lucid as alias

    assert alias is lucid
    for path in ("quantization", "quantization._qgemm", "quantization.observer", "quantization.fuse_modules",
                 "nn.quantized", "nn.quantized.dynamic", "nn.quantized.sparse", "nn.qat", "nn.intrinsic",
                 "backends", "serialization"):
        assert importlib.import_module(f"lucid.{path}") is importlib.import_module(f"lucid_b200.{path}"), path
    from lucid.nn.qat import Linear as AliasQatLinear
    from lucid_b200.nn.qat import Linear as QatLinear

    assert AliasQatLinear is QatLinear
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("lucid.no_such_module")


def test_dynamic_linear_refuses_affine_weights(device):
    """The integer GEMM form equals the reference's (q - z_w) * s_w dequantization only for z_w = 0;
    a state dict carrying a non-zero weight zero-point must not be computed silently wrong."""
    q = Q.quantize_dynamic(nn.Linear(32, 8))
    x = torch.randn(4, 32).to(device)
    q(x)
    q.weight_zero_point[3] = 2.0
    with pytest.raises(NotImplementedError, match="weight_zero_point"):
        q(x)


def test_prepare_fx_convert_fx(device):
    """Graph-mode names (lucid/quantization/_quantize_fx.py:30,112): boundaries are added for the
    caller, then the eager flow runs underneath."""
    model = mlp()
    prepared = Q.prepare_fx(model, example_inputs=torch.randn(2, 32))
    assert isinstance(prepared, nnq.QuantWrapper) and hasattr(prepared.module[0], "activation_post_process")
    assert not hasattr(model[0], "activation_post_process")  # the caller's model is untouched
    prepared = prepared.to(device)
    x = torch.randn(16, 32)
    prepared(x.to(device))
    qm = Q.convert_fx(prepared)
    assert isinstance(qm.module[0], nnq.Linear) and isinstance(qm.quant, nnq.Quantize)
    out = qm(x.to(device)).cpu()
    assert (out - model(x)).abs().mean() / model(x).abs().mean() < 0.1
