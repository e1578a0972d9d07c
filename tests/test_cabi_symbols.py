"""CPU checks of the C-ABI boundary: the shared library loads, exports every
symbol include/lucid_cuda.h declares, and rejects bad arguments without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "lucid_cuda.h")


@pytest.fixture(scope="module")
def capi():
    from lucid_b200._C import build as B

    B.build()
    import lucid_b200._C as capi

    return capi


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lc_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = declared_symbols()
    for required in ("lc_quantize_f32", "lc_dequantize", "lc_qlinear_i8", "lc_wo_linear_s8",
                     "lc_observe_tensor_f32", "lc_group_matmul"):
        assert required in names


def test_library_exports_every_declared_symbol(capi):
    lib = ctypes.CDLL(capi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in lucid_cuda.h but not exported"
    assert set(declared_symbols()) == set(capi.SIGNATURES), "ctypes table out of sync with the header"


def test_version_and_error_text(capi):
    assert capi.lib.lc_version() >= 100
    rc = capi.lib.lc_quantize_f32(None, 1, 1, 8, None, 0, None, 0, 1.0, 0.0, -128, 127, None, capi.LC_S8, None)
    assert rc == capi.LC_ERR_INVALID_ARG
    assert "null pointer" in capi.last_error()
    with pytest.raises(capi.LucidCudaError):
        capi.check(rc)


def test_argument_validation_without_gpu(capi):
    L = capi.lib
    # empty tensors are a no-op success
    assert L.lc_quantize_f32(None, 0, 1, 0, None, 0, None, 0, 1.0, 0.0, -128, 127, None, capi.LC_S8, None) == 0
    # group format rejects unsupported bit widths and ragged K
    assert L.lc_group_quantize_f32(None, 4, 64, 64, 3, None, None, None, None) == capi.LC_ERR_UNSUPPORTED
    assert L.lc_group_quantize_f32(None, 4, 65, 64, 8, None, None, None, None) == capi.LC_ERR_INVALID_ARG
    # the GEMM wants 16-byte row pitches
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    p = (p + 15) // 16 * 16
    rc = L.lc_qlinear_i8(p, 0, 24, p, 32, 1, 1, 24, p, 0, None, None, None, None, p, capi.LC_F32, 1, None, None)
    assert rc == capi.LC_ERR_UNSUPPORTED and "16-byte" in capi.last_error()
    rc = L.lc_wo_linear_s8(p, 99, 1, 16, 16, p, 16, 1, None, None, p, 1, 0, None)
    assert rc == capi.LC_ERR_UNSUPPORTED
    # activations that do not start on a 16-byte boundary are refused before anything is launched
    rc = L.lc_group_matmul(p + 2, capi.LC_BF16, 1, 64, p, p, p, 1, 64, 8, p, None)
    assert rc == capi.LC_ERR_UNSUPPORTED and "16-byte aligned" in capi.last_error()
    # the new entry points validate their arguments the same way
    assert L.lc_wo_gemm_digits(p, 24, p, p, 32, 1, 1, 24, None, None, None, None, 0, None, None, 0, 255, p, 1, None, 0,
                               None) == capi.LC_ERR_UNSUPPORTED
    assert L.lc_wo_gemm_16(p, capi.LC_BF16, 3, 96, p, 32, 1, 1, 32, None, None, None, None, 0, None, None, 0, 255, p,
                           capi.LC_F32, 1, None, 0, None) == capi.LC_ERR_INVALID_ARG  # several terms need K % 64 == 0
    assert L.lc_peer_barrier(None, 0, 1, 1, 1000, None, None) == capi.LC_ERR_INVALID_ARG
    assert L.lc_dynamic_linear_workspace_bytes(64, 1024) >= 64 * 1024
    assert L.lc_wo_digit_rows(33) == 256


def test_fast_bindings_agree_with_ctypes(capi):
    """The CPython module built beside the library serves the per-layer entry points: it is bound to the
    addresses ctypes resolved, returns the library's own status codes, and refuses arguments of the wrong
    number or kind before anything is called."""
    fast, L = capi.fast, capi.lib
    assert fast is not None, "lucid_b200/_C/_fastcall was not built"
    for name in capi.FAST_ENTRY_POINTS:
        assert capi.entry(name[3:]) is getattr(fast, name[3:])
    assert capi.entry("quantize_f32") is not None and not hasattr(fast, "quantize_f32")  # everything else: ctypes
    buf = ctypes.create_string_buffer(64)
    p = (ctypes.addressof(buf) + 15) // 16 * 16
    cases = {
        "dynamic_linear_f32": (p, 0, -1, 0, 0, 0, 0, 0, 1e-8, p, 0, 0, None, None, None, p, 0, 0, p, 0, 0, None, None),
        "group_matmul_ex": (p + 2, capi.LC_BF16, 1, 64, p, p, p, 1, 64, 8, p, 0, None, 0, None),
        "wo_linear_s8_ex": (p, 99, 1, 16, 16, p, 16, 1, None, None, 0, None, None, -128, 127, p, 1, 0, None, 0, None),
        "wo_swiglu_s8_ex": (p, 99, 1, 16, 16, p, 16, 16, None, None, p, 8, 0, None, 0, None),
    }
    for name, args in cases.items():
        expected = getattr(L, "lc_" + name)(*args)
        message = capi.last_error()
        assert expected != capi.LC_OK
        assert getattr(fast, name)(*args) == expected and capi.last_error() == message, name
        with pytest.raises(TypeError):
            getattr(fast, name)(*args[:-1])
        with pytest.raises(TypeError):
            getattr(fast, name)("x", *args[1:])
    with pytest.raises(KeyError):
        fast.bind("lc_quantize_f32", 0)


def test_ops_refuse_cpu_tensors(capi):
    import torch

    from lucid_b200._C import ops

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.quantize(torch.zeros(4), 0.1, 0.0, -128, 127, torch.int8)
