"""``lucid.backends``: engine selection for the quantized Linear layers.

Mirrors ``lucid/backends/__init__.py:57-108``: ``backends.quantized.engine`` keeps
the reference's three values and gains ``"cuda_int8"``:

* ``"reference"`` / ``"cuda_int8"`` -- ``convert`` / ``quantize_dynamic`` build the
  sidecar int8 modules (``nn.quantized.Linear`` / ``nn.quantized.dynamic.Linear``),
  whose forwards here run on the tcgen05 int8 GEMM or the weight-only GEMV;
* ``"mlx_group"`` -- they build ``QuantizedLinearMLX`` (group-wise affine
  weight-only format) as the reference does when its MLX engine is selected;
* ``"auto"`` -- the int8 modules.  (The reference's ``auto`` picks its MLX kernel
  when that engine is compiled in; on this backend the tensor-core int8 path is the
  faster default and the group-wise format stays one assignment away.)
"""
from __future__ import annotations

from typing import final as _final

_ENGINES = ("auto", "mlx_group", "reference", "cuda_int8")


@_final
class _QuantizedBackend:
    _engine: str = "auto"

    @property
    def available(self) -> bool:
        """True when the CUDA kernel library is built and a CUDA device is present."""
        try:
            import torch

            from lucid_b200 import _C  # noqa: F401

            return torch.cuda.is_available()
        except ImportError:
            return False

    @property
    def engine(self) -> str:
        return self._engine

    @engine.setter
    def engine(self, value: str) -> None:
        if value not in _ENGINES:
            raise ValueError(
                "quantized.engine must be 'auto'/'mlx_group'/'reference'/'cuda_int8', " f"got {value!r}"
            )
        self._engine = value

    def use_mlx(self) -> bool:
        """Whether converters should build the group-wise weight-only module."""
        return self._engine == "mlx_group"


@_final
class _CudaBackend:
    """Knobs of the CUDA device backend (the reference exposes ``metal`` / ``accelerate``)."""

    deterministic: bool = True  # every kernel on this path is run-to-run deterministic
    benchmark: bool = False


quantized = _QuantizedBackend()
cuda = _CudaBackend()

__all__ = ["quantized", "cuda"]
