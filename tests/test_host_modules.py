"""Quantized convolution, embedding, activation and fused modules of the static workflow
(the cases of the reference's ``lucid/test/unit/quantization/test_static_ptq.py``,
``test_breadth.py``, ``test_module_breadth.py`` and ``test_safety.py``).  Every case runs on
the CPU with the oracle-backed stand-in for the kernel front end, and on a GPU with the
real kernels."""
import numpy as np
import pytest
import torch
from torch import nn

import lucid_b200 as lucid
import lucid_b200.nn.intrinsic as nni
import lucid_b200.quantization as Q
from lucid_b200 import _backend
from lucid_b200.nn import quantized as nnq


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


def _rel(a, b):
    a, b = a.detach().cpu().numpy(), b.detach().cpu().numpy()
    return float(np.abs(a - b).mean() / (np.abs(a).mean() + 1e-9))


class _ConvNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, 8, 3, padding=1, bias=False)
        self.bn = nn.BatchNorm2d(8)
        self.relu = nn.ReLU()
        self.pool = nn.AdaptiveAvgPool2d(1)
        self.flat = nn.Flatten()
        self.fc = nn.Linear(8, 10)

    def forward(self, x):
        return self.fc(self.flat(self.pool(self.relu(self.bn(self.conv(x))))))


# ---- fusion (test_static_ptq.py TestFusion) ------------------------------------------
def test_fuse_modules_patterns():
    torch.manual_seed(1)
    net = _ConvNet().eval()
    with torch.no_grad():
        net.bn.running_mean.normal_()
        net.bn.running_var.uniform_(0.5, 2.0)
    x = torch.randn(2, 3, 8, 8)
    want = net(x)
    fused = Q.fuse_modules(net, [["conv", "bn"]])
    assert torch.allclose(fused(x), want, atol=1e-4)
    assert isinstance(fused.bn, nn.Identity) and isinstance(net.bn, nn.BatchNorm2d)  # not in place
    fused = Q.fuse_modules(net, [["conv", "bn", "relu"]])
    assert isinstance(fused.conv, nni.ConvReLU2d)
    assert isinstance(fused.bn, nn.Identity) and isinstance(fused.relu, nn.Identity)
    assert torch.allclose(fused(x), want, atol=1e-4)
    seq = nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Conv1d(2, 2, 3), nn.ReLU())
    fused = Q.fuse_modules(seq, [["0", "1"], ["2", "3"]])
    assert isinstance(fused[0], nni.LinearReLU) and isinstance(fused[2], nni.ConvReLU1d)
    assert list(fused._modules) == ["0", "1", "2", "3"]
    with pytest.raises(ValueError, match="unsupported fusion pattern"):
        Q.fuse_modules(net, [["bn", "relu"]])


# ---- convolutions (test_static_ptq.py TestConvPTQ, TestSequentialOrderPreserved) ------
def test_conv_net_quantizes_with_fusion(device):
    torch.manual_seed(3)
    net = _ConvNet().eval()
    fused = Q.fuse_modules(net, [["conv", "bn", "relu"]])
    prepared = Q.prepare(nnq.QuantWrapper(fused))
    for _ in range(8):
        prepared(torch.randn(4, 3, 8, 8))
    qm = Q.convert(prepared)
    assert isinstance(qm.module.conv, nnq.ConvReLU2d) and isinstance(qm.module.fc, nnq.Linear)
    assert qm.module.conv.weight_int8.dtype is torch.int8
    xe = torch.randn(8, 3, 8, 8)
    assert _rel(net(xe), qm(xe.to(device))) < 0.05
    # the fused layer's grid is the post-ReLU one: non-negative outputs only
    assert float(qm.module.conv(xe.to(device)).min()) >= 0.0


def test_convert_keeps_child_order(device):
    torch.manual_seed(5)
    model = nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.BatchNorm2d(4), nn.ReLU()).eval()
    prepared = Q.prepare(nnq.QuantWrapper(model))
    for _ in range(4):
        prepared(torch.randn(2, 3, 8, 8))
    qm = Q.convert(prepared).to(device)  # the BatchNorm between the quantized layers stays a float module
    assert list(qm.module._modules.keys()) == ["0", "1", "2"]
    assert isinstance(qm.module[0], nnq.Conv2d)
    assert qm(torch.randn(2, 3, 8, 8).to(device)).shape == (2, 4, 8, 8)


def _convert_single(layer, x, device):
    model = nn.Sequential(layer).eval()
    want = model(x).detach()
    model.qconfig = Q.get_default_qconfig()
    Q.prepare(model, inplace=True)
    model(x)
    Q.convert(model, inplace=True)
    return want, model(x.to(device)).cpu()


# test_safety.py TestQuantizedConvKeepsThePaddingSpec
@pytest.mark.parametrize("rank", [1, 2, 3])
def test_conv_padding_spec_survives(device, rank):
    torch.manual_seed(rank)
    cls = {1: nn.Conv1d, 2: nn.Conv2d, 3: nn.Conv3d}[rank]
    x = torch.randn(1, 2, *([8] * rank))
    f, q = _convert_single(cls(2, 4, 3, padding="same"), x, device)
    assert tuple(f.shape) == tuple(q.shape) == (1, 4) + (8,) * rank
    f, q = _convert_single(cls(2, 4, 3, padding="valid"), x, device)
    assert tuple(f.shape) == tuple(q.shape) == (1, 4) + (6,) * rank
    f, q = _convert_single(cls(2, 4, 3, padding=1, padding_mode="reflect"), x, device)
    assert float((f - q).abs().max()) < 0.2  # dropping the mode gives about 1
    f, q = _convert_single(cls(2, 4, 3, padding=1), x, device)
    assert tuple(f.shape) == tuple(q.shape) and float((f - q).abs().max()) < 0.2


# test_module_breadth.py
@pytest.mark.parametrize("rank", [1, 2, 3])
def test_direct_conv_int_kernel_size(device, rank):
    q = {1: nnq.Conv1d, 2: nnq.Conv2d, 3: nnq.Conv3d}[rank](2, 4, 3, 1, 1, 1, 1, True)
    assert tuple(q.weight_int8.shape) == (4, 2) + (3,) * rank
    x = torch.randn(1, 2, *([6] * rank))
    assert tuple(q(x.to(device)).shape) == (1, 4) + (6,) * rank


@pytest.mark.parametrize("rank", [1, 2, 3])
def test_conv_transpose_quantizes(device, rank):
    torch.manual_seed(rank)
    ct = {1: nn.ConvTranspose1d, 2: nn.ConvTranspose2d, 3: nn.ConvTranspose3d}[rank]
    shape = {1: (2, 8, 8), 2: (2, 8, 8, 8), 3: (2, 8, 4, 4, 4)}[rank]
    m = nn.Sequential(ct(8, 4, 3, stride=2, padding=1, output_padding=1)).eval()
    x = torch.randn(*shape)
    want = m(x)
    prepared = Q.prepare(m, Q.get_default_qconfig_mapping())
    for _ in range(6):
        prepared(torch.randn(*shape))
    qm = Q.convert(prepared)
    assert isinstance(qm[0], {1: nnq.ConvTranspose1d, 2: nnq.ConvTranspose2d, 3: nnq.ConvTranspose3d}[rank])
    assert qm[0].weight_int8.dtype is torch.int8 and qm[0].weight_scale.shape == (4,)
    got = qm(x.to(device))
    assert got.shape == want.shape and _rel(want, got) < 0.05


@pytest.mark.parametrize("float_cls,q_cls", [(nn.Sigmoid, nnq.Sigmoid), (nn.Hardswish, nnq.Hardswish),
                                             (nn.Hardsigmoid, nnq.Hardsigmoid), (nn.Tanh, nnq.Tanh),
                                             (nn.ELU, nnq.ELU), (nn.LeakyReLU, nnq.LeakyReLU)])
def test_activation_quantizes(device, float_cls, q_cls):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(64, 64), float_cls()).eval()
    x = torch.randn(8, 64)
    want = m(x).detach()
    prepared = Q.prepare(m, Q.get_default_qconfig_mapping())
    for _ in range(5):
        prepared(torch.randn(8, 64))
    qm = Q.convert(prepared)
    assert isinstance(qm[1], q_cls)
    got = qm(x.to(device)).cpu()
    assert float((want - got).abs().max() / (want.abs().max() + 1e-9)) < 0.1
    # requantized: every output sits on the calibrated grid
    codes = got / qm[1].scale.cpu() + qm[1].zero_point.cpu()
    assert float((codes - codes.round()).abs().max()) < 1e-3


def test_leaky_relu_and_elu_carry_their_parameter(device):
    m = nn.Sequential(nn.Linear(8, 8), nn.LeakyReLU(negative_slope=0.2), nn.ELU(alpha=0.7)).eval()
    prepared = Q.prepare(m, Q.get_default_qconfig_mapping())
    for _ in range(3):
        prepared(torch.randn(4, 8))
    qm = Q.convert(prepared)
    assert qm[1].negative_slope == pytest.approx(0.2) and qm[2].alpha == pytest.approx(0.7)


# ---- embeddings (test_breadth.py, test_module_breadth.py TestQuantizedEmbeddingBag) ----
def test_quantized_embedding(device):
    torch.manual_seed(0)
    emb = nn.Embedding(100, 32).eval()
    idx = torch.tensor([[1, 5, 20], [3, 8, 50]])
    want = emb(idx)
    q = nnq.Embedding.from_float(emb)
    assert q.weight_int8.dtype is torch.int8 and q.weight_int8.shape == (100, 32)
    got = q(idx.to(device))
    assert got.shape == (2, 3, 32) and _rel(want, got) < 0.02
    packed = q.weight_int8.numel() + 4 * q.weight_scale.numel()
    assert packed < 100 * 32 * 4 / 2
    qm = Q.convert(Q.prepare(nn.Sequential(nn.Embedding(50, 16))))  # converts without calibration
    assert isinstance(qm[0], nnq.Embedding)
    with pytest.raises(TypeError):
        q(torch.randn(3).to(device))


def test_quantized_embedding_bag(device):
    torch.manual_seed(0)
    for mode in ("mean", "sum", "max"):
        m = nn.Sequential(nn.EmbeddingBag(50, 16, mode=mode))
        idx = torch.tensor([1, 5, 9, 3, 7, 2, 8])
        off = torch.tensor([0, 3, 5])
        want = m[0](idx, off).detach()
        qm = Q.convert(m)
        assert isinstance(qm[0], nnq.EmbeddingBag) and qm[0].weight_int8.dtype is torch.int8
        got = qm[0](idx.to(device), off.to(device)).cpu()
        assert float((want - got).abs().max() / (want.abs().max() + 1e-9)) < 0.05
    bag = nnq.EmbeddingBag.from_float(nn.EmbeddingBag(50, 16, mode="sum"))
    two_d = bag(torch.tensor([[1, 2, 3], [4, 5, 6]]).to(device)).cpu()
    flat = bag(torch.tensor([1, 2, 3, 4, 5, 6]).to(device), torch.tensor([0, 3]).to(device)).cpu()
    assert torch.equal(two_d, flat)
    w = torch.tensor([0.5, 2.0, 1.0, 1.0, 1.0, 0.0])
    weighted = bag(torch.tensor([1, 2, 3, 4, 5, 6]).to(device), torch.tensor([0, 3]).to(device), w.to(device)).cpu()
    rows = nnq.Embedding.from_float(nn.Embedding(50, 16))
    rows.load_state_dict(bag.state_dict())
    r = rows(torch.tensor([1, 2, 3, 4, 5, 6]).to(device)).cpu() * w[:, None]
    assert torch.allclose(weighted, torch.stack([r[:3].sum(0), r[3:].sum(0)]), rtol=1e-5, atol=1e-6)
    with pytest.raises(NotImplementedError):
        bag(torch.tensor([1]), torch.tensor([0]), compressed_indices_mapping=torch.tensor([0]))
    with pytest.raises(ValueError):
        bag(torch.tensor([1, 2]).to(device))


def test_stub_passes_integer_indices(device):
    stub = nnq.QuantStub()
    idx = torch.tensor([1, 2, 3])
    assert torch.equal(stub(idx), idx)
    quant = nnq.Quantize(torch.tensor(0.05), torch.tensor(0.0))
    assert torch.equal(quant(idx.to(device)).cpu(), idx)


def test_quantized_namespace_matches_the_reference():
    names = ["Linear", "QuantizedLinearMLX", "Conv1d", "Conv2d", "Conv3d", "ConvTranspose1d", "ConvTranspose2d",
             "ConvTranspose3d", "Embedding", "EmbeddingBag", "LinearReLU", "ConvReLU1d", "ConvReLU2d", "ConvReLU3d",
             "QuantStub", "DeQuantStub", "Quantize", "DeQuantize", "QuantWrapper", "FloatFunctional", "QFunctional",
             "Sigmoid", "Hardswish", "Hardsigmoid", "Tanh", "ELU", "LeakyReLU"]
    for name in names:
        assert name in nnq.__all__ and isinstance(getattr(nnq, name), type), name
    assert lucid.nn.intrinsic is nni


# ---- convert leaves no qconfig behind (test_convert_strips_qconfig.py) ---------------
def _with_qconfig(model):
    return [n for n, m in model.named_modules() if hasattr(m, "qconfig")]


@pytest.mark.parametrize("inplace", [False, True])
def test_convert_strips_qconfig(device, inplace):
    model = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Sequential(nn.Linear(8, 4), nn.Tanh()))
    model.qconfig = Q.get_default_qconfig()
    prepared = Q.prepare(model)
    prepared(torch.randn(2, 8))
    assert "" in _with_qconfig(prepared)
    converted = Q.convert(prepared, inplace=inplace)
    assert _with_qconfig(converted) == [] and (converted is prepared) is inplace
    assert isinstance(converted[0], nnq.Linear) and isinstance(converted[2][1], nnq.Tanh)
    assert converted(torch.randn(2, 8).to(device)).shape == (2, 4)


def test_excluded_embedding_stays_float_and_qint4_recipe_reaches_the_table(device):
    model = nn.Sequential(nn.Embedding(10, 4), nn.Linear(4, 4))
    model.qconfig = Q.get_default_qconfig()
    model[0].qconfig = None
    prepared = Q.prepare(model)
    prepared(torch.tensor([1, 2]))
    converted = Q.convert(prepared)
    assert type(converted[0]) is nn.Embedding and isinstance(converted[1], nnq.Linear)
    assert _with_qconfig(converted) == []
    from lucid_b200.quantization.observer import PerChannelMinMaxObserver

    model = nn.Sequential(nn.Embedding(10, 4))
    model.qconfig = Q.QConfig(activation=Q.get_default_qconfig().activation,
                              weight=PerChannelMinMaxObserver.with_args(ch_axis=0, qscheme=Q.per_channel_symmetric,
                                                                        qdtype=Q.qint4))
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")  # prepare(): nothing to observe in a weight-only model
        converted = Q.convert(Q.prepare(model))
    codes = converted[0].weight_int8
    assert isinstance(converted[0], nnq.Embedding) and int(codes.min()) >= -8 and int(codes.max()) <= 7
    assert converted[0](torch.tensor([3, 4]).to(device)).shape == (2, 4)


# ---- quantization-aware training (test_qat.py, test_safety.py TestQConfigGuards) --------
class _QatNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.quant = nnq.QuantStub()
        self.fc1 = nn.Linear(16, 32)
        self.act = nn.ReLU()
        self.fc2 = nn.Linear(32, 4)
        self.dequant = nnq.DeQuantStub()

    def forward(self, x):
        return self.dequant(self.fc2(self.act(self.fc1(self.quant(x)))))


def test_prepare_qat_trains_through_the_ste_and_converts(device):
    import lucid_b200.nn.qat as nnqat

    torch.manual_seed(2)
    float_net = _QatNet()
    qat = Q.prepare_qat(float_net).to(device)
    assert isinstance(qat.fc1, nnqat.Linear) and qat.training and type(float_net.fc1) is nn.Linear
    assert isinstance(qat.fc1.weight_fake_quant, Q.FakeQuantize)
    assert isinstance(qat.quant.activation_post_process, Q.FakeQuantize)
    w0 = qat.fc1.weight.detach().clone()
    opt = torch.optim.SGD(qat.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(2)
    for _ in range(5):
        loss = (qat(torch.randn(16, 16, generator=g).to(device)) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert not torch.allclose(w0, qat.fc1.weight.detach())  # the gradient reached the float weight
    qat.eval()
    qm = Q.convert(qat)
    assert isinstance(qm.fc1, nnq.Linear) and qm.fc1.weight_int8.dtype is torch.int8
    assert isinstance(qm.quant, nnq.Quantize) and isinstance(qm.dequant, nnq.DeQuantize)
    x = torch.randn(64, 16, generator=g).to(device)
    with torch.no_grad():
        want, got = qat(x).cpu(), qm(x).cpu()
    assert float((want - got).abs().mean() / (want.abs().mean() + 1e-9)) < 0.1


def test_qat_layers_need_a_qconfig_and_cover_conv_and_embedding(device):
    import lucid_b200.nn.qat as nnqat

    with pytest.raises(ValueError, match="qconfig"):
        nnqat.Linear(8, 8)
    with pytest.raises(ValueError, match="qconfig"):
        nnqat.Conv2d(3, 8, 3)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Conv2d(2, 4, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(4 * 6 * 6, 5))
    fused = Q.fuse_modules(model, [["0", "1"]])
    qat = Q.prepare_qat(fused).to(device)
    assert isinstance(qat[0], nnqat.ConvReLU2d) and isinstance(qat[3], nnqat.Linear)
    x = torch.randn(3, 2, 6, 6).to(device)
    qat(x).sum().backward()
    assert qat[0].weight.grad is not None and float(qat[0].weight.grad.abs().sum()) > 0
    qat.eval()
    qm = Q.convert(qat)
    assert isinstance(qm[0], nnq.ConvReLU2d) and isinstance(qm[3], nnq.Linear)
    with torch.no_grad():
        assert _rel(qat(x), qm(x)) < 0.1
    emb = Q.prepare_qat(nn.Sequential(nn.Embedding(20, 8))).to(device)
    assert isinstance(emb[0], nnqat.Embedding)
    idx = torch.tensor([1, 5, 7]).to(device)
    emb(idx).sum().backward()
    assert emb[0].weight.grad is not None
    qe = Q.convert(emb.eval())
    assert isinstance(qe[0], nnq.Embedding)
    with torch.no_grad():
        assert _rel(emb(idx), qe(idx)) < 0.02


# ---- trainable Conv + BatchNorm fusion (test_qat.py TestConvBnReLUQAT, test_qat_fused.py) ----
def test_fuse_modules_qat_trains_batchnorm_and_converts(device):
    import lucid_b200.nn.intrinsic.qat as nniqat

    torch.manual_seed(4)
    net = _ConvNet()
    qcfg = Q.get_default_qat_qconfig()
    fused = Q.fuse_modules_qat(net, [["conv", "bn", "relu"]], qcfg)
    assert isinstance(fused.conv, nniqat.ConvBnReLU2d) and isinstance(fused.bn, nn.Identity)
    assert isinstance(net.bn, nn.BatchNorm2d)  # a copy was fused
    qat = Q.prepare_qat(fused, qcfg).to(device)
    assert isinstance(qat.conv, nniqat.ConvBnReLU2d) and type(qat.conv.conv) is nn.Conv2d
    w, b = qat.conv._fold()
    assert w.shape == (8, 3, 3, 3) and b.shape == (8,)
    mean0 = qat.conv.bn.running_mean.clone()
    opt = torch.optim.SGD(qat.parameters(), lr=0.01)
    for _ in range(4):
        loss = (qat(torch.randn(2, 3, 8, 8).to(device)) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert qat.conv.conv.weight.grad is not None and qat.conv.bn.weight.grad is not None
    assert not torch.equal(mean0, qat.conv.bn.running_mean)  # batch statistics kept updating
    qat.conv.freeze_bn_stats()
    frozen = qat.conv.bn.running_mean.clone()
    qat.train()
    qat(torch.randn(2, 3, 8, 8).to(device))
    assert torch.equal(frozen, qat.conv.bn.running_mean) and not qat.conv.bn.training
    qat.eval()
    qm = Q.convert(qat)
    assert isinstance(qm.conv, nnq.ConvReLU2d) and qm.conv.weight_int8.dtype is torch.int8
    x = torch.randn(4, 3, 8, 8).to(device)
    with torch.no_grad():
        assert qm(x).shape == (4, 10) and _rel(qat(x), qm(x)) < 0.1
    with pytest.raises(ValueError, match="qconfig"):
        nniqat.ConvBn2d(nn.Conv2d(3, 8, 3), nn.BatchNorm2d(8))
    with pytest.raises(ValueError, match="running statistics"):
        nniqat.ConvBn2d(nn.Conv2d(3, 8, 3), nn.BatchNorm2d(8, track_running_stats=False), qconfig=qcfg)
    with pytest.raises(ValueError, match="unsupported pattern"):
        Q.fuse_modules_qat(net, [["bn", "relu"]], qcfg)
