"""Benchmark of the int8 quantized-inference path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras] [--profile-case NAME]

Headline workload ("prefill"): the prefill-shaped dynamic int8 Linear, x fp32 [16384, 8192]
~N(0,1) quantized per token, W [28672, 8192] ~N(0,0.02) quantized per output channel, int32
accumulation, fp32 dequantized output; over N GPUs the weight is sharded by output
columns and the output shards are exchanged inside the GEMM epilogue by peer stores over
NVLink (symmetric memory), or with an NCCL all-gather (--gather nccl).  One step = quantize
activations + GEMM (+ all-gather).  metric: int8 qLinear TOPS = 2*M*N*K / step time,
whole job.  At N = 1 the line also carries the HBM-bound companions of the metric (the
[8192, 8192] quantize / dequantize roundtrip and the decode-shaped weight-only MLP) under
"extras", the roofline of the dominant kernel and a CPU baseline timed on this host.

Inputs are seeded synthetic tensors of the configured shapes and distributions.
Timing: CUDA events on the launching stream after >= 3 warm-up steps, barrier +
synchronize on both sides, max over ranks; inputs are larger than L2 (126 MB).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_PREFILL, N_PREFILL, K_PREFILL = 16384, 28672, 8192
NOMINAL_INT8_TOPS = 4500.0   # dense int8, datasheet
NOMINAL_HBM_GBS = 8000.0


# ----------------------------------------------------------------------------------------
# measured peaks and clocks
# ----------------------------------------------------------------------------------------
def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs."""

    BAD = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
           "hw_power_brake_slowdown": 0x80}
    NOTED = {"sw_power_cap": 0x4}

    def __init__(self, index: int) -> None:
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self) -> None:
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for name, bit in {**self.BAD, **self.NOTED}.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------
# CPU reference arm (the reference's own formulation, restated in oracle/, on host cores)
# ----------------------------------------------------------------------------------------
def cpu_prefill_reference(steps: int, warmup: int, sample_rows: int = 512) -> dict:
    """Times the reference's dynamic Linear forward (fake-quantize x per row, dequantize the
    whole weight, fp32 GEMM) on `sample_rows` rows of the prefill workload against the full
    [28672, 8192] weight, with all host threads NumPy's BLAS takes."""
    import numpy as np

    from oracle import oracle as O

    rng = np.random.default_rng(20260925)
    x = rng.standard_normal((sample_rows, K_PREFILL), dtype=np.float32)
    w = rng.standard_normal((N_PREFILL, K_PREFILL), dtype=np.float32)
    w *= np.float32(0.02)
    wq, sw, zw = O.quantize_weight_per_channel(w)
    del w
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        y = O.dynamic_linear_float(x, wq, sw, zw, None, "token_symmetric", O.qint8)
        float(y[0, 0])
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    ops = 2.0 * sample_rows * N_PREFILL * K_PREFILL
    return {"value": ops / t / 1e12, "unit": "TOPS", "cores": len(os.sched_getaffinity(0)), "kind": "port",
            "sample": f"{sample_rows} of {M_PREFILL} rows of x against the full W [{N_PREFILL},{K_PREFILL}], "
                      f"reference float formulation (per-forward weight dequantize + sgemm), median of {steps}",
            "seconds_per_sample": t}


def run_reference_arm(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps = max(1, min(args.steps, 3))
    warmup = max(1, min(args.warmup, 1))
    base = cpu_prefill_reference(steps, warmup)
    line = {
        "impl": "reference", "metric": "int8_qlinear_tops", "value": base["value"], "unit": "TOPS",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": base["seconds_per_sample"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "prefill_qlinear_16384x28672x8192_per_token_int8",
                   "note": "reference engine is Apple-only; its Python-level CPU formulation restated in "
                           "oracle/ is timed on a bounded row sample"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------------------
# GPU side
# ----------------------------------------------------------------------------------------
def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_loop(torch, fn, steps: int, warmup: int) -> float:
    """Average milliseconds per call, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = _events(torch)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def graph_time(torch, fn, reps: int = 4, replays: int = 10):
    """Milliseconds per call of `fn` when `reps` calls are captured in one CUDA graph and the
    graph is replayed: removes host launch overhead from latency-bound sequences."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                fn()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = _events(torch)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * replays)


def encoder_extras(torch, dev, gen) -> dict:
    """Post-norm transformer encoder (the reference's layer order, nn/modules/transformer.py:300-311)
    with explicit q/k/v/o Linears so that quantize_dynamic swaps all 36 of them; attention,
    LayerNorm, GELU and residual adds stay in fp32 torch ops."""
    import lucid_b200.quantization as Q
    from lucid_b200.nn.quantized.dynamic import Linear as DynLinear

    nn, F = torch.nn, torch.nn.functional
    D, H, FF, L, B, S = 512, 8, 2048, 6, 32, 256

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v, self.o = (nn.Linear(D, D) for _ in range(4))
            self.linear1, self.linear2 = nn.Linear(D, FF), nn.Linear(FF, D)
            self.norm1, self.norm2 = nn.LayerNorm(D), nn.LayerNorm(D)

        def forward(self, x):
            b, s, _ = x.shape
            q, k, v = (m(x).view(b, s, H, D // H).transpose(1, 2) for m in (self.q, self.k, self.v))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, D)
            x = self.norm1(x + self.o(a))
            return self.norm2(x + self.linear2(F.gelu(self.linear1(x))))

    model = nn.Sequential(*[Layer() for _ in range(L)]).to(dev).eval()
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, nn.Linear):
                m.weight.normal_(0.0, 0.02, generator=gen)
                m.bias.zero_()
    x = torch.randn(B, S, D, device=dev, generator=gen)
    qmodel = Q.quantize_dynamic(model)
    n_swapped = sum(isinstance(m, DynLinear) for m in qmodel.modules())
    res = {"quantized_linears": n_swapped, "tokens_per_forward": B * S,
           "linear_int8_GOP": 2 * B * S * (4 * D * D + 2 * D * FF) * L / 1e9}
    with torch.no_grad():
        ref = model(x)
        got = qmodel(x)
        res["mean_rel_err_vs_float"] = float((got - ref).abs().mean() / ref.abs().mean())
        for name, mod in (("int8_dynamic", qmodel), ("float32_torch", model)):
            ms = time_loop(torch, lambda: mod(x), 10, 3)
            res[name] = {"eager_ms": ms, "eager_tokens_per_s": B * S / ms * 1e3}
            try:
                gms = graph_time(torch, lambda: mod(x), reps=2, replays=10)
                res[name].update({"graph_ms": gms, "graph_tokens_per_s": B * S / gms * 1e3})
            except Exception as e:
                res[name]["graph_error"] = repr(e)[:200]
    return res


def dispatch_rows(torch, dev, width: int = 1024, n_iter: int = 20) -> list:
    """Row schema and timing contract of the reference's dispatch benchmark: bits in {4, 8},
    M in {1, 2, 8, 32}, N = K = width, group 64; paths packed / cached_dense / dequant_each_call;
    a call is timed with its output materialised (`.sum().item()`) and the device synchronised
    (tools/_bench_timing.py:33-52); a 1e-4 relative parity gate precedes timing."""
    from lucid_b200.quantization import _qgemm

    def cold_ms(call):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        call().sum().item()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3

    torch.manual_seed(20260920)
    rows = []
    with torch.no_grad():
        for bits in (4, 8):
            weight = torch.randn(width, width, device=dev)
            packed, scales, biases = _qgemm.quantize(weight, group_size=64, bits=bits)
            dense = _qgemm.dequantize(packed, scales, biases, group_size=64, bits=bits)
            for m in (1, 2, 8, 32):
                x = torch.randn(m, width, device=dev)
                calls = {
                    "packed": lambda: _qgemm.quantized_matmul(x, packed, scales, biases, transpose=True,
                                                              group_size=64, bits=bits),
                    "cached_dense": lambda: torch.matmul(x, dense.mT),
                    "dequant_each_call": lambda: torch.matmul(
                        x, _qgemm.dequantize(packed, scales, biases, group_size=64, bits=bits).mT),
                }
                expected, actual = calls["cached_dense"](), calls["packed"]()
                err = float((expected - actual).abs().max()) / max(float(expected.abs().max()), 1e-12)
                if not err <= 1e-4:
                    raise RuntimeError(f"parity failure for bits={bits}, M={m}: {err}")
                for name, call in calls.items():
                    first = cold_ms(call)
                    for _ in range(5):
                        call().sum().item()
                    samples = sorted(cold_ms(call) for _ in range(n_iter))
                    rows.append({"bits": bits, "m": m, "n": width, "k": width, "path": name,
                                 "first_ms": round(first, 4), "median_ms": round(statistics.median(samples), 4),
                                 "p5_ms": round(samples[int(n_iter * 0.05)], 4),
                                 "p95_ms": round(samples[min(n_iter - 1, int(n_iter * 0.95))], 4),
                                 "parity_relative_error": err})
    return rows


def extras_single_gpu(torch, ops, peaks) -> dict:
    """HBM-bound companions of the metric, measured on one GPU after the headline run."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    hbm = peaks["hbm_gbs"]
    g = torch.Generator(device=dev).manual_seed(20260922)
    # ---- standalone roundtrip: fp32 [8192, 8192] ~N(0,1), 0.1 % outliers x50 (268 MB > L2)
    x = torch.randn(8192, 8192, device=dev, generator=g)
    idx = torch.randint(0, x.numel(), (x.numel() // 1000,), device=dev, generator=g)
    x.view(-1)[idx] *= 50.0
    q, s, z = ops.dynamic_quantize_rows(x, True, -128, 127, True)
    cases = {
        "quantize_per_channel_fused": (lambda: ops.dynamic_quantize_rows(x, True, -128, 127, True),
                                       x.numel() * 5 + 8192 * 4),
        "quantize_per_tensor_fused": (lambda: ops.dynamic_quantize_tensor(x, True, -128, 127, True, 1e-8, torch.int8),
                                      x.numel() * 9),
        "dequantize_per_channel": (lambda: ops.dequantize(q, s, z, ch_axis=0), x.numel() * 5),
        "quantize_per_channel_given_scale": (lambda: ops.quantize(x, s, z, -128, 127, torch.int8, ch_axis=0),
                                             x.numel() * 5),
        # calibration pass of the histogram observer: 2048 bins over the data range
        "histc_2048_bins": (lambda: ops.histc(x, 2048, -60.0, 60.0), x.numel() * 4),
    }
    rt = {}
    for name, (fn, nbytes) in cases.items():
        ms = time_loop(torch, fn, 30, 5)
        gbs = nbytes / ms / 1e6
        rt[name] = {"ms": ms, "GB/s": gbs, "algorithmic_bytes": nbytes, "frac_of_measured_hbm": gbs / hbm,
                    "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS}
    out["roundtrip_8192x8192"] = rt
    del x, q, s, z
    # ---- int8 embedding table [131072, 4096] (537 MB > L2), 16384 looked-up tokens: 1 byte read
    # and 4 bytes written per element (the reference's formulation decodes the whole table first)
    try:
        V, D, n = 131072, 4096, 16384
        table = torch.randint(-128, 128, (V, D), dtype=torch.int8, device=dev, generator=g)
        ts = torch.rand(V, device=dev, generator=g) * 0.05 + 1e-3
        toks = [torch.randint(0, V, (n,), device=dev, generator=g) for _ in range(5)]  # 5 x 67 MB of rows rotate
        turn = [0]

        def next_tok():
            turn[0] += 1
            return toks[turn[0] % len(toks)]

        ms = time_loop(torch, lambda: ops.embedding_s8(table, ts, None, next_tok()), 30, 5)
        nbytes = n * D * 5 + n * 12
        bag_off = torch.arange(0, n, 32, device=dev)
        ms_bag = time_loop(torch, lambda: ops.embedding_bag_s8(table, ts, None, next_tok(), bag_off, "sum"), 30, 5)
        bag_bytes = n * D + (n // 32) * D * 4 + n * 12
        out["embedding_int8_131072x4096"] = {
            "lookup_16384_tokens": {"ms": ms, "GB/s": nbytes / ms / 1e6, "algorithmic_bytes": nbytes,
                                    "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm},
            "bag_sum_512_bags_of_32": {"ms": ms_bag, "GB/s": bag_bytes / ms_bag / 1e6, "algorithmic_bytes": bag_bytes,
                                       "frac_of_measured_hbm": bag_bytes / ms_bag / 1e6 / hbm},
            "decode_whole_table_then_gather_bytes": V * D * 5 + n * D * 8}
        del table, ts, toks, bag_off
    except Exception as e:  # noqa: BLE001
        out["embedding_int8_131072x4096"] = {"error": repr(e)[:200]}
    # ---- decode-shaped weight-only SwiGLU MLP: hidden 4096, FFN 14336, bf16 activations
    H, F = 4096, 14336
    sets = []
    for i in range(3):  # 3 x 176 MB of weights rotate so that no step finds its weights in L2
        ws = []
        quantized = []
        for (n, k) in ((F, H), (F, H), (H, F)):  # gate, up, down
            w = torch.randn(n, k, device=dev, generator=g) * 0.02
            quantized.append(ops.dynamic_quantize_rows(w, True, -128, 127, True)[:2])
            del w
        (wg, sg), (wu, su), (wd, sd) = quantized
        # gate and up rows interleaved so that one pass over both weights ends in silu(gate) * up
        ws = [(ops.interleave_gate_up(wg, wu), ops.interleave_gate_up(sg, su)), (wd, sd)]
        del quantized, wg, wu
        sets.append(ws)
    dec = {}
    for batch in (1, 4, 16):
        xb = torch.randn(batch, H, device=dev, generator=g).to(torch.bfloat16)
        counter = [0]
        overlap = [True]  # weights are constants: each kernel may prefetch them while the one before drains

        def mlp_step():
            (wgu, sgu), (wd, sd) = sets[counter[0] % 3]
            counter[0] += 1
            h = ops.wo_swiglu_s8(xb, wgu, sgu, overlap_previous=overlap[0])
            return ops.wo_linear_s8(h, wd, sd, overlap_previous=overlap[0])

        nbytes = 3 * H * F + (2 * F + H) * 4
        eager_ms = time_loop(torch, mlp_step, 60, 6)
        entry = {"eager_us": eager_ms * 1e3, "algorithmic_bytes": nbytes}
        try:  # one MLP = 3 kernels + 2 elementwise ops of ~10 us each: host launch cost matters
            ms = graph_time(torch, mlp_step, reps=6, replays=10)
            entry["timing"] = ("CUDA graph of 6 MLPs (2 kernels each: fused gate/up/SwiGLU, down) over 3 rotating "
                               "weight sets, programmatic dependent launch between kernels")
        except Exception as e:
            ms, entry["graph_error"] = eager_ms, repr(e)[:200]
        entry.update({"us": ms * 1e3, "GB/s": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / hbm})
        try:  # the same graph with every kernel fully serialised behind its predecessor
            overlap[0] = False
            entry["us_without_launch_overlap"] = graph_time(torch, mlp_step, reps=6, replays=10) * 1e3
        except Exception as e:
            entry["serialised_graph_error"] = repr(e)[:200]
        dec[f"batch_{batch}"] = entry
    out["decode_mlp_4096x14336_w8a16"] = dec
    del sets
    # ---- small transformer encoder, every Linear dynamic int8 (6 layers, d 512, 8 heads, FFN 2048)
    try:
        out["encoder_6x512_b32_s256"] = encoder_extras(torch, dev, g)
    except Exception as e:  # reported, never hidden
        out["encoder_6x512_b32_s256"] = {"error": repr(e)[:300]}
    # ---- the reference's own dispatch benchmark rows (tools/bench_quantized_dispatch.py:26-75)
    try:
        out["quantized_dispatch_rows"] = dispatch_rows(torch, dev)
    except Exception as e:
        out["quantized_dispatch_rows"] = {"error": repr(e)[:300]}
    # ---- the single dynamic Linear (x [64,1024], W [4096,1024]) through the module API
    try:
        import lucid_b200.quantization as Q

        lin = torch.nn.Linear(1024, 4096).to(dev)
        with torch.no_grad():
            lin.weight.normal_(0, 0.02, generator=g)
            lin.bias.normal_(0, 0.01, generator=g)
        qlin = Q.quantize_dynamic(lin)
        x1 = torch.randn(64, 1024, device=dev, generator=g)
        # a fresh tensor object per call, as in real use (the layer reuses the codes of an input it
        # has just seen, which a loop over one tensor object would turn into a no-op)
        ms = time_loop(torch, lambda: qlin(x1.detach()), 200, 20)
        entry = {"us_per_forward": ms * 1e3, "TOPS": 2 * 64 * 4096 * 1024 / ms / 1e9,
                 "note": "eager: host-bound (two launches per forward, their output allocations and argument checks)"}
        try:  # the same module captured in a CUDA graph (one launch per forward, input copied in)
            import lucid_b200

            gl = lucid_b200.cuda.make_graphed(qlin, x1)
            assert torch.equal(gl(x1), qlin(x1))
            gms = time_loop(torch, lambda: gl(x1), 400, 40)
            entry.update({"graphed_us_per_forward": gms * 1e3, "graphed_TOPS": 2 * 64 * 4096 * 1024 / gms / 1e9})
            # device time alone: ten forwards in one graph (per-tensor quantize kernel + GEMM each)
            dms = graph_time(torch, lambda: qlin(x1.detach()), reps=10, replays=20)
            entry.update({"device_us_per_forward": dms * 1e3, "device_TOPS": 2 * 64 * 4096 * 1024 / dms / 1e9})
        except Exception as e:
            entry["graphed_error"] = repr(e)[:200]
        out["single_dynamic_linear_64x4096x1024"] = entry
    except Exception as e:  # reported, never hidden
        out["single_dynamic_linear_64x4096x1024"] = {"error": repr(e)[:200]}
    return out


def run_profile_case(args) -> int:
    """A small, fixed case of one kernel (inputs larger than L2, a few hundred MB on the
    device) run a handful of times: the target of `ncu --set full` captures."""
    import torch

    from lucid_b200._C import ops

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1)
    case = args.profile_case
    if case == "gemm":
        M, N, K = 4096, 7168, 8192
        a = torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8, generator=g)
        b = torch.randint(-128, 128, (N, K), device=dev, dtype=torch.int8, generator=g)
        sx, sw = torch.rand(M, device=dev), torch.rand(N, device=dev)
        fn = lambda: ops.qlinear_i8(a, b, sx, sw)  # noqa: E731
    elif case == "histc":
        x = torch.randn(8192, 8192, device=dev, generator=g)
        fn = lambda: ops.histc(x, 2048, -6.0, 6.0)  # noqa: E731
    elif case == "embedding":
        table = torch.randint(-128, 128, (131072, 4096), dtype=torch.int8, device=dev, generator=g)
        ts = torch.rand(131072, device=dev, generator=g) * 0.05 + 1e-3
        toks = [torch.randint(0, 131072, (16384,), device=dev, generator=g) for _ in range(5)]
        turn = [0]

        def fn():
            turn[0] += 1
            return ops.embedding_s8(table, ts, None, toks[turn[0] % 5])
    elif case == "embedding_bag":
        table = torch.randint(-128, 128, (131072, 4096), dtype=torch.int8, device=dev, generator=g)
        ts = torch.rand(131072, device=dev, generator=g) * 0.05 + 1e-3
        toks = [torch.randint(0, 131072, (16384,), device=dev, generator=g) for _ in range(5)]
        off = torch.arange(0, 16384, 32, device=dev)
        turn = [0]

        def fn():
            turn[0] += 1
            return ops.embedding_bag_s8(table, ts, None, toks[turn[0] % 5], off, "sum")
    elif case == "merge":
        x = torch.randn(8192, 8192, device=dev, generator=g)
        y = torch.randn(8192, 8192, device=dev, generator=g)
        fn = lambda: ops.fake_quantize_merge(x, y, "add_relu", 0.05, 12.0, 0, 255)  # noqa: E731
    elif case == "gemm_shortk":
        M, N, K = 8192, 2048, 512  # an encoder FFN projection: little K per output, epilogue-heavy
        a = torch.randint(0, 256, (M, K), device=dev, dtype=torch.uint8, generator=g)
        b = torch.randint(-128, 128, (N, K), device=dev, dtype=torch.int8, generator=g)
        sx, sw, bias = torch.rand((), device=dev), torch.rand(N, device=dev), torch.randn(N, device=dev)
        zx, wsum = torch.tensor(7.0, device=dev), ops.rowsum_s8(b)
        fn = lambda: ops.qlinear_i8(a, b, sx, sw, bias=bias, zx=zx, wsum=wsum)  # noqa: E731
    elif case == "gemm_small":
        a = torch.randint(-128, 128, (64, 1024), device=dev, dtype=torch.int8, generator=g)
        b = torch.randint(-128, 128, (4096, 1024), device=dev, dtype=torch.int8, generator=g)
        sx, sw = torch.rand(64, device=dev), torch.rand(4096, device=dev)
        fn = lambda: ops.qlinear_i8(a, b, sx, sw)  # noqa: E731
    elif case in ("quantize_rows", "quantize_tensor", "dequantize", "quantize_given_scale"):
        x = torch.randn(8192, 8192, device=dev, generator=g)
        q, s, z = ops.dynamic_quantize_rows(x, True, -128, 127, True)
        fn = {"quantize_rows": lambda: ops.dynamic_quantize_rows(x, True, -128, 127, True),
              "quantize_tensor": lambda: ops.dynamic_quantize_tensor(x, True, -128, 127, True, 1e-8, torch.int8),
              "dequantize": lambda: ops.dequantize(q, s, z, ch_axis=0),
              "quantize_given_scale": lambda: ops.quantize(x, s, z, -128, 127, torch.int8, ch_axis=0)}[case]
    elif case == "wo_gemv":
        ws = []
        for _ in range(4):
            w = torch.randn(14336, 4096, device=dev, generator=g) * 0.02
            wq, sw, _ = ops.dynamic_quantize_rows(w, True, -128, 127, True)
            ws.append((wq, sw))
        xb = torch.randn(int(args.profile_batch), 4096, device=dev, generator=g).to(torch.bfloat16)
        i = [0]

        def fn():
            wq, sw = ws[i[0] % 4]
            i[0] += 1
            return ops.wo_linear_s8(xb, wq, sw)
    else:
        raise SystemExit(f"unknown profile case {case!r}")
    for _ in range(6):
        fn()
    torch.cuda.synchronize()
    print(f"profile case {case}: ok")
    return 0


def run_ours(args) -> int:
    import torch
    import torch.distributed as dist

    from lucid_b200._C import ops  # fails loudly if liblucid_cuda.so is missing
    import lucid_b200.quantization as Q

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference "
                         "for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    M, N, K = M_PREFILL, N_PREFILL, K_PREFILL
    if N % world:
        raise SystemExit(f"N={N} does not split over {world} ranks")
    n_local = N // world

    # seeded synthetic data: x replicated on every rank, W rows [rank*n_local, (rank+1)*n_local)
    gx = torch.Generator(device=dev).manual_seed(20260925)
    x = torch.randn(M, K, device=dev, generator=gx)
    gw = torch.Generator(device=dev).manual_seed(20260926 + rank)
    lin = torch.nn.Linear(K, n_local, bias=False, device=dev)
    with torch.no_grad():
        lin.weight.normal_(0.0, 0.02, generator=gw)
    qlin = Q.quantize_dynamic(lin, inplace=True).set_activation_scheme("token_symmetric")
    del lin
    torch.cuda.empty_cache()
    wq, _ = qlin._cache.get(qlin.weight_int8)
    sw = qlin.weight_scale
    # ---- output exchange at N > 1 ------------------------------------------------------
    # "fused": every rank's GEMM epilogue stores its column slice straight into every rank's
    # [M, N] result (peer stores over NVLink through symmetric memory), so the all-gather is
    # part of the kernel; "nccl": local shard + ncclAllGather, the plain baseline.
    gathered = None
    gather_mode, gather_note, out_ptrs, symm_hdl, full = "none", "", None, None, None
    if world > 1:
        gather_mode = args.gather
        if gather_mode in ("auto", "fused"):
            try:
                import torch.distributed._symmetric_memory as symm

                full = symm.empty((M, N), dtype=torch.float32, device=dev)
                symm_hdl = symm.rendezvous(full, dist.group.WORLD)
                order = [(rank + i) % world for i in range(world)]  # own buffer first, peers rotated
                out_ptrs = [int(symm_hdl.buffer_ptrs[r]) + rank * n_local * 4 for r in order]
                gather_mode = "fused"
            except Exception as e:  # reported in the JSON line, never silent
                if args.gather == "fused":
                    raise
                gather_mode, gather_note = "nccl", f"symmetric memory unavailable: {repr(e)[:120]}"
        if gather_mode == "nccl":
            gathered = torch.empty((world, M, n_local), dtype=torch.float32, device=dev)

    gemm_ms = []

    def step(record: bool = False):
        xq, sx, _ = ops.dynamic_quantize_rows(x, True, -128, 127, True, 1e-8, torch.int8, pad_rows_to_16=True)
        if record:
            a, b = _events(torch)
            a.record()
        if gather_mode == "fused":
            ops.qlinear_i8_into(xq, wq, sx, sw, out_ptrs, N)
            y = full
        else:
            y = ops.qlinear_i8(xq, wq, sx, sw)
        if record:
            b.record()
            gemm_ms.append((a, b))
        if gather_mode == "fused":
            symm_hdl.barrier()  # every rank's slices have landed in this rank's result
        elif gather_mode == "nccl":
            dist.all_gather_into_tensor(gathered.view(-1), y.view(-1))
        return y

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    e0, e1 = _events(torch)
    with ClockSampler(local) as clocks:
        sync_all()
        e0.record()
        for _ in range(args.steps):
            step(record=True)
        e1.record()
        sync_all()
    total_ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(total_ms.item()) / args.steps
    gemm_avg_ms = sum(a.elapsed_time(b) for a, b in gemm_ms) / len(gemm_ms)
    value = 2.0 * M * N * K / ms_per_step / 1e9

    # ---- N > 1: check the exchange, and time the GEMM phase without it ------------------
    exchange_verified, gemm_only_ms = None, None
    cp_module = None
    if world > 1:
        from lucid_b200.nn.quantized.column_parallel import ColumnParallelLinear

        xq, sx, _ = ops.dynamic_quantize_rows(x, True, -128, 127, True, 1e-8, torch.int8, pad_rows_to_16=True)
        y_local = ops.qlinear_i8(xq, wq, sx, sw)
        result = step()
        sync_all()
        if gather_mode == "fused":
            mine = result[:, rank * n_local:(rank + 1) * n_local]
            whole = result
        else:
            mine = gathered[rank]
            whole = gathered
        ok_local = bool(torch.equal(mine, y_local))
        checksum = whole.view(torch.int32).sum(dtype=torch.int64).reshape(1)
        sums = [torch.zeros_like(checksum) for _ in range(world)]
        dist.all_gather(sums, checksum)
        flags = torch.tensor([int(ok_local)], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        exchange_verified = bool(flags.item()) and all(int(v) == int(sums[0]) for v in sums)
        t = torch.tensor([time_loop(torch, lambda: ops.qlinear_i8(xq, wq, sx, sw), 5, 2)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gemm_only_ms = float(t.item())
        del y_local
        cp_module = ColumnParallelLinear(qlin, N, gather="fused" if gather_mode == "fused" else "nccl")

    # ---- end to end through the module API with host buffers --------------------------
    from lucid_b200.nn.quantized.streaming import forward_from_host

    x_host = x.cpu().pin_memory()
    y_host = torch.empty((M, N), dtype=torch.float32).pin_memory() if rank == 0 else None
    x_dev = torch.empty_like(x)

    def e2e_step():
        if world == 1:  # chunked: H2D of chunk i+1, layer on chunk i and D2H of chunk i-1 overlap
            forward_from_host(qlin, x_host, y_host, chunk_rows=2048)
            return
        x_dev.copy_(x_host, non_blocking=True)
        y = cp_module(x_dev)
        if rank == 0:
            y_host.copy_(y, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    sync_all()
    f0, f1 = _events(torch)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    sync_all()
    e2e_ms = torch.tensor([f0.elapsed_time(f1)], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(e2e_ms.item()) / e2e_steps

    if rank == 0:
        int8_peak = 2.0 * peaks["bf16_tflops"]
        achieved = 2.0 * M * n_local * K / gemm_avg_ms / 1e9
        line = {
            "metric": "int8_qlinear_tops", "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8xs8->s32",
            "data": "synthetic",
            "config": {"workload": "prefill_qlinear_16384x28672x8192_per_token_int8", "M": M, "N": N, "K": K,
                       "activation_quant": "dynamic per-token symmetric int8 (absmax/127.5, [-128,127])",
                       "weight_quant": "per-output-channel symmetric int8", "output": "fp32",
                       "parallelism": f"column-parallel x{world}" + (
                           "" if world == 1 else " + all-gather fused into the GEMM epilogue (peer stores)"
                           if gather_mode == "fused" else " + NCCL all-gather"),
                       "gather": gather_mode, "gather_note": gather_note,
                       "l2": "inputs exceed L2 (x 537 MB, W 235 MB, y 1879 MB vs 126 MB)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                         "frac": achieved / int8_peak,
                         # dram__bytes_read+write of a 1/16-size launch of the same kernel (same K and tile
                         # shape: profiles/qlinear_i8_pair_gemm_4096x7168x8192.md) scaled by the ops ratio
                         "traffic": 3.41e9 if world == 1 else None,
                         "kernel": "qlinear_i8_pair_kernel", "kernel_ms": gemm_avg_ms,
                         "peak_source": f"2 x bf16_tflops ({peaks['source']}, burst): tcgen05 issues dense int8 at "
                                        "twice the bf16 rate; no int8 figure is measured by the driver",
                         "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS},
            "e2e": {"value": 2.0 * M * N * K / e2e_ms_per_step / 1e9, "unit": "TOPS",
                    "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4,
                    "ms_per_step": e2e_ms_per_step, "api": "lucid_b200.nn.quantized.streaming.forward_from_host(dynamic.Linear, ...), 2048-row chunks" if world == 1 else
                           "lucid_b200.nn.quantized.column_parallel.ColumnParallelLinear.forward"},
            "gpu_launches": args.steps * 2,
            "exchange": None if world == 1 else {
                "mode": gather_mode, "bytes_out_per_gpu": (world - 1) * M * n_local * 4,
                "GB/s_out_per_gpu_during_gemm_kernel": (world - 1) * M * n_local * 4 / gemm_avg_ms / 1e6,
                "nvlink_peer_copy_peak_GB/s": 770.0, "verified_bit_identical_on_all_ranks": exchange_verified,
                "gemm_phase_only": {"ms": gemm_only_ms, "aggregate_TOPS": 2.0 * M * N * K / gemm_only_ms / 1e9,
                                    "note": "same shard GEMM writing only the local buffer (no exchange), max over ranks"},
                "note": "fused: the GEMM kernel's duration includes the peer stores, so at large N it is "
                        "bound by NVLink, not by the tensor cores" if gather_mode == "fused" else
                        "nccl: the exchange runs after the GEMM kernel"},
            "clocks": clocks.summary(),
        }
        if world == 1:
            del x_host, y_host, x_dev
            torch.cuda.empty_cache()
        if world == 1 and not args.no_extras:
            try:  # library comparator (cuBLASLt through torch), for context only
                a8 = wq[:8192]
                t = time_loop(torch, lambda: torch._int_mm(a8, a8.t()), 5, 2)
                line["library_int8_gemm_tops_8192x8192x8192"] = 2 * 8192.0 ** 3 / t / 1e9
            except Exception as e:
                line["library_int8_gemm_tops_8192x8192x8192"] = f"unavailable: {repr(e)[:80]}"
            line["extras"] = extras_single_gpu(torch, ops, peaks)
            line["cpu_baseline"] = {k: v for k, v in cpu_prefill_reference(3, 1).items() if k != "seconds_per_sample"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline workload only: skip the companion workloads and the CPU baseline")
    ap.add_argument("--profile-case", default=None,
                    help="run a small fixed case of one kernel (gemm, quantize_rows, quantize_tensor, "
                         "dequantize, quantize_given_scale, histc, merge, embedding, embedding_bag, gemm_small, gemm_shortk, wo_gemv) for a profiler capture; prints no bench line")
    ap.add_argument("--profile-batch", default=4)
    ap.add_argument("--gather", choices=("auto", "fused", "nccl"), default="auto",
                    help="N > 1: how output shards are exchanged (auto = fused if symmetric memory works)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.profile_case:
        return run_profile_case(args)
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.abspath(__file__),
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--gather", args.gather]
        return subprocess.call(cmd)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
