"""Error bounds shared by the GPU parity tests of the weight-only kernels."""
import numpy as np
import torch

_MANTISSA = {torch.bfloat16: 7, torch.float16: 10, torch.float32: 23}
_MIN_EXP = {torch.bfloat16: -126, torch.float16: -14, torch.float32: -126}


def assert_rounded_product(y, ref64, abs_terms64, K, dtype, extra=0.0):
    """`y` (output type `dtype`) against the float64 value `ref64` of the same expression:
    one unit in the last place of the output type at |ref| (a correctly rounded result is within
    half of one; the second half covers the fp32 -> 16-bit double rounding), plus the a-priori bound
    of fp32 accumulation, depth * 2^-24 * sum_k |x_k| * |operand_k| * scale, where the kernels add
    at most K/32 + 32 partial sums one after the other (lane- and warp-split K, 16 per mma)."""
    ref = np.asarray(ref64, dtype=np.float64)
    got = y.detach().double().cpu().numpy() if isinstance(y, torch.Tensor) else np.asarray(y, dtype=np.float64)
    expo = np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** _MIN_EXP[dtype])))
    ulp = 2.0 ** (expo - _MANTISSA[dtype])
    depth = K / 32.0 + 32.0
    tol = ulp + depth * 2.0 ** -24 * np.asarray(abs_terms64, dtype=np.float64) + extra
    bad = np.abs(got - ref) > tol
    assert not bad.any(), (f"{int(bad.sum())} of {bad.size} outputs off by more than 1 ulp + accumulation bound; "
                           f"worst {float((np.abs(got - ref) / tol).max()):.2f} x tolerance")


def abs_terms(x, wq, sw, offset=128.0):
    """sum_k |x[b,k]| * (|wq[n,k]| + offset) * sw[n] in float64: the magnitude the accumulation error
    scales with (the streaming kernel multiplies offset-binary bytes, hence the 128)."""
    xa = torch.as_tensor(x).double().abs()
    wa = torch.as_tensor(wq).double().abs() + offset
    return ((xa @ wa.T) * torch.as_tensor(sw).double()[None, :]).cpu().numpy()
