"""Writes tests/golden/quant_golden.npz and linear_golden.npz.

The reference engine cannot be imported on Linux, so these vectors are the
oracle's outputs on seeded inputs, produced after the oracle passed the
reference's known-answer tests (tests/test_oracle_golden.py) and the
torch.quantize_per_tensor cross-check.  Run from the repo root:
    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    # the reference's bit-exact rounding case: default_rng(0), [64,256], ch_axis=1
    x = np.random.default_rng(0).standard_normal((64, 256)).astype(np.float32)
    s1, z1 = O.calculate_qparams(*O.minmax_channel(x, 1), True, O.qint8)
    s0, z0 = O.calculate_qparams(*O.minmax_channel(x, 0), True, O.qint8)
    st, zt = O.calculate_qparams(*O.minmax_tensor(x), False, O.quint8)
    ss, zs = O.calculate_qparams(*O.minmax_tensor(x), True, O.qint8)
    fq, mask = O.fake_quantize(x, s1, z1, -128, 127, ch_axis=1)
    np.savez_compressed(
        os.path.join(HERE, "quant_golden.npz"),
        meta=json.dumps({"seed": 0, "shape": [64, 256]}),
        x=x,
        scale_ch1=s1, q_ch1=O.quantize(x, s1, z1, O.qint8, ch_axis=1),
        scale_ch0=s0, q_ch0=O.quantize(x, s0, z0, O.qint8, ch_axis=0),
        dq_ch0=O.dequantize(O.quantize(x, s0, z0, O.qint8, ch_axis=0), s0, z0, ch_axis=0),
        qparams_affine=np.array([st, zt], np.float32), q_affine=O.quantize(x, st, zt, O.quint8),
        qparams_sym=np.array([ss, zs], np.float32), q_sym=O.quantize(x, ss, zs, O.qint8),
        fq_ch1=fq, mask_ch1=mask,
        q_pyfloat=O.quantize(x, 0.05, 0.0, O.qint8),
    )
    # a small dynamic Linear in the three activation modes
    r = np.random.default_rng(1)
    xa = r.standard_normal((48, 160)).astype(np.float32)
    w = (r.standard_normal((72, 160)) * 0.02).astype(np.float32)
    b = (r.standard_normal(72) * 0.01).astype(np.float32)
    wq, sw, zw = O.quantize_weight_per_channel(w)
    out = {"x": xa, "w": w, "b": b, "wq": wq, "sw": sw}
    for mode, qd in (("tensor_affine", O.quint8), ("tensor_symmetric", O.qint8), ("token_symmetric", O.qint8)):
        acc, y, xq, sx, zx = O.dynamic_linear_int(xa, wq, sw, b, mode, qd)
        out[f"acc_{mode}"] = acc
        out[f"y_{mode}"] = y
        out[f"xq_{mode}"] = xq
        out[f"sx_{mode}"] = np.asarray(sx, np.float32)
        out[f"zx_{mode}"] = np.asarray(zx, np.float32)
    out["y_reference_float"] = O.dynamic_linear_reference(xa, wq, sw, zw, b)
    np.savez_compressed(os.path.join(HERE, "linear_golden.npz"), **out)
    print("wrote golden fixtures")


if __name__ == "__main__":
    main()
