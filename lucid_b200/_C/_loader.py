"""ctypes loader for liblucid_cuda.so, the C-ABI shim declared in include/lucid_cuda.h.

Plays the role of the reference's ``lucid._C.engine.quantized`` submodule
(``lucid/_C/bindings/bind_quantized.cpp:17-27``) for the CUDA device.  The
library is required: importing this module fails loudly when it has not been
built (``python -m lucid_b200._C.build``); there is no Python or CPU fallback.
A ctypes call releases the GIL for its duration, so a host thread that waits on
the GPU does not block other Python threads.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblucid_cuda.so")

LC_OK = 0
LC_ERR_INVALID_ARG, LC_ERR_UNSUPPORTED, LC_ERR_CUDA, LC_ERR_TIMEOUT, LC_ERR_WORKSPACE = -1, -2, -3, -4, -5
LC_F32, LC_BF16, LC_F16, LC_S8, LC_U8, LC_S16, LC_S32 = range(7)
LC_QLINEAR_WAIT_TEST = 256
LC_QLINEAR_MULTICAST_OUT = 512


class LucidCudaError(RuntimeError):
    """A liblucid_cuda entry point returned a non-zero status."""

    def __init__(self, code: int, message: str) -> None:
        super().__init__(f"liblucid_cuda error {code}: {message}")
        self.code = code


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m lucid_b200._C.build` "
        "(needs nvcc; there is no CPU fallback for the quantized CUDA path)"
    )

lib = C.CDLL(LIB_PATH)

_p, _i32, _i64, _f = C.c_void_p, C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); mirrors include/lucid_cuda.h declaration by declaration
SIGNATURES = {
    "lc_version": (_i32, []),
    "lc_last_error": (_i32, [C.c_char_p, _i32]),
    "lc_stream_capture_id": (_i32, [_p, C.POINTER(C.c_uint64)]),
    "lc_device_info": (_i32, [_i32, C.POINTER(_i32), C.POINTER(_i32)]),
    "lc_observe_tensor_workspace_bytes": (_i64, []),
    "lc_observe_tensor_f32": (_i32, [_p, _i64, _p, _p, _i32, _i32, _i32, _i32, _i32, _f, _p, _p, _p, _i64, _p]),
    "lc_observe_tensor_static_max_elems": (_i64, []),
    "lc_observe_tensor_static_f32": (_i32, [_p, _i64, _p, _p, _i32, _i32, _i32, _i32, _i32, _f, _p, _p, _p]),
    "lc_fake_quantize_merge_f32": (_i32, [_p, _p, _f, _i32, _i64, _p, _p, _f, _f, _f, _i32, _i32, _p, _p]),
    "lc_histc_workspace_bytes": (_i64, [_i32]),
    "lc_histc_f32": (_i32, [_p, _i64, _i32, C.c_double, C.c_double, _p, _i32, _p, _i64, _p]),
    "lc_observe_channel_f32": (_i32, [_p, _i64, _i64, _i64, _p, _p, _i32, _p]),
    "lc_calculate_qparams_f32": (_i32, [_p, _p, _i64, _i32, _i32, _i32, _i32, _f, _p, _p, _p]),
    "lc_quantize_f32": (_i32, [_p, _i64, _i64, _i64, _p, _i64, _p, _i64, _f, _f, _i32, _i32, _p, _i32, _p]),
    "lc_dequantize": (_i32, [_p, _i32, _i64, _i64, _i64, _p, _i64, _p, _i64, _f, _f, _p, _i32, _p]),
    "lc_fake_quantize_f32": (_i32, [_p, _i64, _i64, _i64, _p, _i64, _p, _i64, _f, _f, _f, _i32, _i32, _p, _p, _p]),
    "lc_dynamic_quantize_rows_f32": (_i32, [_p, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f, _p, _i32, _i64, _p, _p, _p]),
    "lc_dynamic_quantize_tensor_f32": (_i32, [_p, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f, _p, _i32, _i64, _p, _p, _p, _p, _i64, _p]),
    "lc_qlinear_i8": (_i32, [_p, _i32, _i64, _p, _i64, _i64, _i64, _i64, _p, _i32, _p, _p, _p, _p, _p, _i32, _i64, _p, _p]),
    "lc_qlinear_i8_ex": (_i32, [_p, _i32, _i64, _p, _i64, _i64, _i64, _i64, _p, _i32, _p, _p, _p, _p, _p, _i32, _i64, _p, _i32, _p]),
    "lc_qlinear_i8_multi": (_i32, [_p, _i32, _i64, _p, _i64, _i64, _i64, _i64, _p, _i32, _p, _p, _p, _p,
                                   C.POINTER(C.c_void_p), _i32, _i32, _i64, _p, _i32, _p]),
    "lc_qlinear_check_status": (_i32, [_p, _i32, _p]),
    "lc_peer_barrier": (_i32, [C.POINTER(C.c_void_p), _i32, _i32, C.c_uint32, _i64, _p, _p]),
    "lc_copy_2d_async": (_i32, [_p, _i64, _p, _i64, _i64, _i64, _p]),
    "lc_dynamic_linear_workspace_bytes": (_i64, [_i64, _i64]),
    "lc_dynamic_linear_f32": (_i32, [_p, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f, _p, _i64, _i64, _p, _p, _p, _p, _i32,
                                     _i64, _p, _i64, _i32, _p, _p]),
    "lc_rowsum_s8": (_i32, [_p, _i64, _i64, _i64, _p, _p]),
    "lc_wo_gemm_16": (_i32, [_p, _i32, _i32, _i64, _p, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _i32, _p, _p, _i32, _i32,
                             _p, _i32, _i64, _p, _i32, _p]),
    "lc_wo_digit_rows": (_i64, [_i64]),
    "lc_split_f32_digits": (_i32, [_p, _i64, _i64, _i64, _p, _i64, _p, _p, _p]),
    "lc_wo_gemm_digits": (_i32, [_p, _i64, _p, _p, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _i32, _p, _p, _i32, _i32, _p,
                                 _i64, _p, _i32, _p]),
    "lc_widen_s8": (_i32, [_p, _i64, _i64, _i64, _p, _i32, _i64, _p]),
    "lc_split_f32_bf16x3": (_i32, [_p, _i64, _i64, _i64, _p, _i64, _p, _p]),
    "lc_wo_linear_s8": (_i32, [_p, _i32, _i64, _i64, _i64, _p, _i64, _i64, _p, _p, _p, _i64, _i32, _p]),
    "lc_wo_linear_s8_ex": (_i32, [_p, _i32, _i64, _i64, _i64, _p, _i64, _i64, _p, _p, _i32, _p, _p, _i32, _i32, _p, _i64,
                                  _i32, _p, _i64, _p]),
    "lc_wo_linear_workspace_bytes": (_i64, [_i64]),
    "lc_wo_swiglu_s8_ex": (_i32, [_p, _i32, _i64, _i64, _i64, _p, _i64, _i64, _p, _p, _p, _i64, _i32, _p, _i64, _p]),
    "lc_wo_swiglu_s8": (_i32, [_p, _i32, _i64, _i64, _i64, _p, _i64, _i64, _p, _p, _p, _i64, _i32, _p]),
    "lc_wo_linear_status": (_i32, [C.POINTER(_i32), _i32]),
    "lc_group_quantize_f32": (_i32, [_p, _i64, _i64, _i32, _i32, _p, _p, _p, _p]),
    "lc_group_dequantize": (_i32, [_p, _p, _p, _i64, _i64, _i32, _i32, _p, _p]),
    "lc_group_matmul_ex": (_i32, [_p, _i32, _i64, _i64, _p, _p, _p, _i64, _i32, _i32, _p, _i32, _p, _i64, _p]),
    "lc_group_matmul": (_i32, [_p, _i32, _i64, _i64, _p, _p, _p, _i64, _i32, _i32, _p, _p]),
    "lc_embedding_s8_f32": (_i32, [_p, _p, _p, _p, _i64, _i64, _i64, _p, _p, _p]),
    "lc_embedding_bag_s8_f32": (_i32, [_p, _p, _p, _p, _i64, _p, _i64, _p, _i64, _i64, _i32, _i64, _i32, _p, _p, _p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library lacks a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


# The four entry points a decode-time forward calls once per layer, behind a CPython module that spares
# ctypes' marshalling (about 3 us per call with twenty arguments); ctypes serves them when the module has
# not been built.  Same arguments, same status code.
FAST_ENTRY_POINTS = ("lc_dynamic_linear_f32", "lc_group_matmul_ex", "lc_wo_linear_s8_ex", "lc_wo_swiglu_s8_ex")
try:
    from . import _fastcall as fast
except ImportError:
    fast = None
else:
    for _name in FAST_ENTRY_POINTS:
        fast.bind(_name, C.cast(getattr(lib, _name), C.c_void_p).value)


def entry(name: str):
    """The callable for ``lc_<name>``: the fast binding when there is one, else the ctypes function."""
    if fast is not None and "lc_" + name in FAST_ENTRY_POINTS:
        return getattr(fast, name)
    return getattr(lib, "lc_" + name)


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib.lc_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc: int) -> None:
    """Raise :class:`LucidCudaError` for a non-zero status."""
    if rc != LC_OK:
        raise LucidCudaError(rc, last_error())
