"""The scratch-free global-range entry point, lc_observe_tensor_static_f32.

It exists for hosts that cannot hand the library any scratch memory (an allocator that
is closed to plug-ins, a binding without a CUDA allocator): the ticket and the per-CTA
partials live in a static device array inside the library.  The test calls it through
the C ABI twice in a row -- the second call finds the first call's leftovers in the
shared array -- and requires the same min, max, scale and zero-point, bit for bit, as
the workspace entry point lc_observe_tensor_f32 gives on the same input.  The file name
sorts last so that a run stopping at the first failure has already run everything else.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(capi, x, spec, accumulate, seed_minmax):
    """Run both entry points on `x`; returns ((min,max,scale,zp) static, same for workspace)."""
    sym, qmin, qmax, signed = spec
    dev = x.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    ws = torch.zeros(int(capi.lib.lc_observe_tensor_workspace_bytes()), dtype=torch.uint8, device=dev)
    out = []
    for static in (True, False):
        mn = torch.full((), seed_minmax[0], device=dev)
        mx = torch.full((), seed_minmax[1], device=dev)
        sc = torch.empty((), device=dev)
        zp = torch.empty((), device=dev)
        if static:
            rc = capi.lib.lc_observe_tensor_static_f32(x.data_ptr(), x.numel(), mn.data_ptr(), mx.data_ptr(),
                                                       accumulate, sym, qmin, qmax, signed, 1e-8, sc.data_ptr(),
                                                       zp.data_ptr(), stream)
        else:
            rc = capi.lib.lc_observe_tensor_f32(x.data_ptr(), x.numel(), mn.data_ptr(), mx.data_ptr(), accumulate,
                                                sym, qmin, qmax, signed, 1e-8, sc.data_ptr(), zp.data_ptr(),
                                                ws.data_ptr(), ws.numel(), stream)
        capi.check(rc)
        torch.cuda.synchronize()
        out.append(tuple(float(t) for t in (mn, mx, sc, zp)))
    return out


def test_static_scratch_entry_point_matches_workspace_entry_point():
    import lucid_b200._C as capi

    torch.manual_seed(7)
    dev = torch.device("cuda", 0)
    # two calls in a row on different inputs and sizes: the second one starts from the
    # first one's contents of the shared array
    a = torch.randn(3_000_001, device=dev) * 3.0          # odd length: vector body + scalar tail
    b = torch.randn(8192, 1024, device=dev) - 0.5          # many CTAs, different range
    first = _call_pair(capi, a, (0, 0, 255, 0), accumulate=0, seed_minmax=(0.0, 0.0))
    second = _call_pair(capi, b, (1, -128, 127, 1), accumulate=1, seed_minmax=(float("inf"), float("-inf")))
    for static, workspace in (first, second):
        assert static == workspace                           # exact: min/max and IEEE qparams
    assert first[0][0] == float(a.min()) and first[0][1] == float(a.max())
    assert second[0][0] == float(b.min()) and second[0][1] == float(b.max())
    # a small third call right behind them, back on the first input's layout
    c = torch.tensor([-2.0, 5.0, 0.25], device=dev)
    third_static, third_ws = _call_pair(capi, c, (0, 0, 255, 0), accumulate=0, seed_minmax=(0.0, 0.0))
    assert third_static == third_ws and third_static[:2] == (-2.0, 5.0)
    assert third_static[2] == float(np.float32(7.0) / np.float32(255.0))


def test_static_scratch_entry_point_rejects_oversized_and_bad_input():
    import lucid_b200._C as capi

    dev = torch.device("cuda", 0)
    x = torch.zeros(16, device=dev)
    mn = torch.zeros((), device=dev)
    limit = int(capi.lib.lc_observe_tensor_static_max_elems())
    assert limit == 1 << 30
    rc = capi.lib.lc_observe_tensor_static_f32(x.data_ptr(), limit + 1, mn.data_ptr(), mn.data_ptr(), 0, 0, 0, 255,
                                               0, 1e-8, None, None, None)
    assert rc == capi.LC_ERR_UNSUPPORTED and "exceed the limit" in capi.last_error()
    rc = capi.lib.lc_observe_tensor_static_f32(None, 4, mn.data_ptr(), mn.data_ptr(), 0, 0, 0, 255, 0, 1e-8,
                                               None, None, None)
    assert rc == capi.LC_ERR_INVALID_ARG
