"""Parity on the five benchmark configurations, by name.  C1, C2 and C5 also have dedicated
cases in test_gpu_qlinear.py / test_gpu_quant.py; here every configuration is exercised
through the public module API and every quantized Linear inside it is checked against the
oracle on exactly the tensors it saw."""
import numpy as np
import pytest
import torch
from torch import nn

import lucid_b200.quantization as Q
from lucid_b200.nn import quantized as nnq
from lucid_b200.nn.quantized import dynamic as nnqd
from oracle import oracle as O

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-6


def boundary_rows(m: int, count: int = 512) -> np.ndarray:
    """Row sample for a full-size product: the first and last rows, both sides of every 128- and
    256-row tile edge near the ends and the middle, and seeded random rows up to `count`."""
    if m <= count:
        return np.arange(m)
    fixed = {0, 1, m - 2, m - 1}
    for edge in (128, 256, 512, m // 2, m - 256, m - 128):
        fixed.update({edge - 1, edge})
    rnd = np.random.default_rng(m).choice(m, size=count - len(fixed), replace=False)
    return np.unique(np.concatenate([np.fromiter(fixed, dtype=np.int64), rnd]))


def check_dynamic_linears(model, x, sample_rows: int | None = None):
    """Run `model(x)`; for each dynamic Linear compare its output with the oracle's integer
    formulation evaluated on the input that layer received (codes exact, fp32 rtol 1e-5).
    The kernels always run on all rows; `sample_rows` limits the oracle's float64 product to a
    boundary-covering sample of them (activation ranges still come from the whole tensor)."""
    seen = []
    hooks = [m.register_forward_hook(lambda mod, args, out: seen.append((mod, args[0].detach(), out.detach())))
             for m in model.modules() if isinstance(m, nnqd.Linear)]
    with torch.no_grad():
        y = model(x)
    for h in hooks:
        h.remove()
    assert seen
    for mod, xin, out in seen:
        x2 = xin.reshape(-1, mod.in_features).float().cpu().numpy()
        wq = mod.weight_int8.cpu().numpy()
        sw = mod.weight_scale.cpu().numpy()
        b = None if mod.bias is None else mod.bias.cpu().numpy()
        rows = None if sample_rows is None else boundary_rows(x2.shape[0], sample_rows)
        _, y_o, _, _, _ = O.dynamic_linear_int(x2, wq, sw, b, mod.act_scheme, O.QDtype(
            mod.act_qdtype.name, 8, mod.act_qdtype.signed, mod.act_qdtype.quant_min, mod.act_qdtype.quant_max,
            mod.act_qdtype.storage), rows=rows)
        got = out.reshape(-1, mod.out_features).cpu().numpy()
        np.testing.assert_allclose(got if rows is None else got[rows], y_o, rtol=RTOL, atol=ATOL)
    return y, len(seen)


def test_config1_single_dynamic_linear_module():
    x, w, b = O.synth_config1()
    lin = nn.Linear(1024, 4096)
    with torch.no_grad():
        lin.weight.copy_(torch.tensor(w))
        lin.bias.copy_(torch.tensor(b))
    narrow = Q.QDtype("qint8", 8, True, -127, 127, "int8")  # scale = absmax/127, clamp [-127,127]
    q = Q.quantize_dynamic(lin, dtype=narrow).set_activation_scheme("tensor_symmetric", narrow)
    wq_o, sw_o, _ = O.quantize_weight_per_channel(w, O.qint8_narrow)
    np.testing.assert_array_equal(q.weight_int8.cpu().numpy(), wq_o)
    np.testing.assert_array_equal(q.weight_scale.cpu().numpy(), sw_o)
    _, n = check_dynamic_linears(q, torch.tensor(x, device="cuda"))
    assert n == 1


def test_config3_encoder_every_linear():
    """One post-norm encoder layer of the benchmark's shape family (d 512, 8 heads, FFN 2048):
    six dynamic int8 Linears, each checked on the activations it actually received."""
    torch.manual_seed(0)
    D, H, FF = 512, 8, 2048

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v, self.o = (nn.Linear(D, D) for _ in range(4))
            self.linear1, self.linear2 = nn.Linear(D, FF), nn.Linear(FF, D)
            self.norm1, self.norm2 = nn.LayerNorm(D), nn.LayerNorm(D)

        def forward(self, x):
            b, s, _ = x.shape
            with nnqd.share_quantized_input():
                q, k, v = [m(x).view(b, s, H, D // H).transpose(1, 2) for m in (self.q, self.k, self.v)]
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, D)
            x = self.norm1(x + self.o(a))
            return self.norm2(x + self.linear2(torch.nn.functional.gelu(self.linear1(x))))

    model = Layer().cuda().eval()
    for m in model.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, 0.0, 0.02)
    qmodel = Q.quantize_dynamic(model)
    x = torch.randn(4, 64, D, device="cuda")
    y, n = check_dynamic_linears(qmodel, x)
    assert n == 6
    with torch.no_grad():
        ref = model(x)
    assert float((y - ref).abs().mean() / ref.abs().mean()) < 0.05


def test_config3_encoder_full_size():
    """The configuration as stated: 6 post-norm layers, d 512, 8 heads, FFN 2048, batch 32 x 256
    tokens (M = 8192 rows per Linear), every one of the 36 Linears dynamic int8.  All kernels run at
    full size; each Linear's output is checked against the oracle on 512 rows that cover the tile
    edges, with the activation range taken from the full [8192, K] tensor it received."""
    torch.manual_seed(3)
    D, H, FF, L, B, S = 512, 8, 2048, 6, 32, 256

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v, self.o = (nn.Linear(D, D) for _ in range(4))
            self.linear1, self.linear2 = nn.Linear(D, FF), nn.Linear(FF, D)
            self.norm1, self.norm2 = nn.LayerNorm(D), nn.LayerNorm(D)

        def forward(self, x):
            b, s, _ = x.shape
            with nnqd.share_quantized_input():
                q, k, v = [m(x).view(b, s, H, D // H).transpose(1, 2) for m in (self.q, self.k, self.v)]
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, D)
            x = self.norm1(x + self.o(a))
            return self.norm2(x + self.linear2(torch.nn.functional.gelu(self.linear1(x))))

    model = nn.Sequential(*[Layer() for _ in range(L)]).cuda().eval()
    for m in model.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, 0.0, 0.02)
    qmodel = Q.quantize_dynamic(model)
    x = torch.randn(B, S, D, device="cuda")
    y, n = check_dynamic_linears(qmodel, x, sample_rows=512)
    assert n == 36
    with torch.no_grad():
        ref = model(x)
    assert float((y - ref).abs().mean() / ref.abs().mean()) < 0.05


def test_config4_decode_mlp_module():
    torch.manual_seed(1)
    Hd, F = 4096, 14336
    gate, up, down = (nn.Linear(Hd, F, bias=False), nn.Linear(Hd, F, bias=False), nn.Linear(F, Hd, bias=False))
    for l in (gate, up, down):
        nn.init.normal_(l.weight, 0.0, 0.02)
    mlp = nnq.WeightOnlySwiGLU.from_float(gate, up, down)
    # weights: bit-exact per-channel symmetric int8 against the oracle
    wq_o, sw_o, _ = O.quantize_weight_per_channel(down.weight.detach().numpy())
    np.testing.assert_array_equal(mlp.down.weight_int8.cpu().numpy(), wq_o)
    np.testing.assert_array_equal(mlp.down.weight_scale.cpu().numpy(), sw_o)
    wg, wu = mlp._split(mlp.gate_up_int8)
    sg, su = mlp._split(mlp.gate_up_scale)
    from lucid_b200._C import ops
    from tolerances import abs_terms, assert_rounded_product

    for batch in (1, 4, 16):
        x = torch.randn(batch, Hd, device="cuda").to(torch.bfloat16)
        y = mlp(x)
        # stage 1: the fused gate / up / SwiGLU pass (deterministic, so this is the module's own h)
        h = ops.wo_swiglu_s8(x, mlp.gate_up_int8, mlp.gate_up_scale)
        g = (x.double() @ wg.double().T) * sg.double()
        u = (x.double() @ wu.double().T) * su.double()
        href = torch.nn.functional.silu(g) * u
        depth = (Hd / 32.0 + 32.0) * 2.0 ** -24
        extra = depth * (1.1 * abs_terms(x, wg, sg) * u.abs().cpu().numpy()
                         + g.abs().cpu().numpy() * abs_terms(x, wu, su)) + 4 * 2.0 ** -24 * href.abs().cpu().numpy()
        assert_rounded_product(h, href.cpu().numpy(), np.zeros_like(extra), Hd, torch.bfloat16, extra=extra)
        # stage 2: the down projection of exactly that h
        wd, sd = mlp.down.weight_int8, mlp.down.weight_scale
        ref = (h.double() @ wd.double().T) * sd.double()
        assert_rounded_product(y, ref.cpu().numpy(), abs_terms(h, wd, sd), F, torch.bfloat16)
    assert ops.wo_linear_status() == 0


def test_graphed_module_replays_the_quantized_forward():
    """A dynamic Linear captured in a CUDA graph returns the eager result for new inputs of the
    captured shape, sees in-place weight updates, and refuses other shapes."""
    import lucid_b200
    import lucid_b200.quantization as Q

    torch.manual_seed(0)
    lin = torch.nn.Linear(1024, 4096).cuda()
    qlin = Q.quantize_dynamic(lin)
    x = torch.randn(64, 1024, device="cuda")
    g = lucid_b200.cuda.make_graphed(qlin, x, clone_outputs=True)
    for _ in range(3):
        x = torch.randn(64, 1024, device="cuda")
        assert torch.equal(g(x), qlin(x))
    qlin.bias.add_(1.0)  # same storage: the replay reads the new values
    assert torch.equal(g(x), qlin(x))
    with pytest.raises(ValueError, match="captured for"):
        g(torch.randn(8, 1024, device="cuda"))


def test_sibling_layers_share_one_activation_quantization():
    """Inside a share_quantized_input() block q / k / v style siblings fed the same tensor reuse its
    codes; a new tensor, an in-place change or another grid does not; outside a block nothing is
    shared (writes that bypass torch's version counter could not be seen)."""
    from lucid_b200.nn.quantized.dynamic import share_quantized_input

    torch.manual_seed(0)
    a, b = (Q.quantize_dynamic(nn.Linear(256, 128).cuda()) for _ in range(2))
    x = torch.randn(64, 256, device="cuda")
    calls = []
    orig = nnqd.Linear._quantize_activations

    def counting(self, x2):
        calls.append(1)
        return orig(self, x2)

    nnqd.Linear._quantize_activations = counting
    try:
        ya0, yb0 = a(x), b(x)  # outside a block nothing is shared (each call quantizes inside the library)
        assert len(calls) == 0
        with share_quantized_input():
            ya, yb = a(x), b(x)
            assert len(calls) == 1
            x.mul_(2.0)  # in-place change: new version
            ya2 = a(x)
            assert len(calls) == 2
            a(x.clone())  # another tensor
            assert len(calls) == 3
            b.set_activation_scheme("token_symmetric")
            b(x)  # same tensor, other grid (replaces the entry)
            a(x)
            assert len(calls) == 5
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                a(x)  # same tensor on another stream: its codes were produced on the first one
            torch.cuda.current_stream().wait_stream(side)
            assert len(calls) == 6
        with share_quantized_input():
            a(x)  # a new block starts empty
        assert len(calls) == 7
    finally:
        nnqd.Linear._quantize_activations = orig
    assert torch.equal(ya, ya0) and torch.equal(yb, yb0)  # shared codes give the bits of independent quantization
    assert torch.equal(a(x), ya2)
