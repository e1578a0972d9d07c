"""Column-parallel dynamic int8 Linear over several GPUs of one node.

The reference has no multi-device path; this is the N-sharded form of its dynamic Linear
(``lucid/nn/quantized/dynamic/linear.py:85-109``).  Rank r keeps output rows
``[r*N/P, (r+1)*N/P)`` of the quantized weight, the input is replicated and quantized
locally, K is not split, so every output column is bit-identical to the single-GPU result.
The shards are exchanged either

* ``"fused"``: inside the GEMM epilogue -- each rank stores its tiles straight into the
  ``[M, N]`` result buffer of every rank (peer stores over NVLink through symmetric
  memory), then a device-side barrier; or
* ``"nccl"`` / ``"gloo"``: a plain all-gather of the local ``[M, N/P]`` shard.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized.dynamic.linear import Linear as DynamicLinear
from lucid_b200.quantization._qscheme import QDtype, qint8


def shard_rows(out_features: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open row range of ``rank``; ``out_features`` must divide evenly."""
    if out_features % world:
        raise ValueError(f"out_features={out_features} does not split over {world} ranks")
    per = out_features // world
    return rank * per, (rank + 1) * per


class ColumnParallelLinear(nn.Module):
    def __init__(self, shard: DynamicLinear, out_features: int, group=None, gather: str = "auto") -> None:
        super().__init__()
        self.shard = shard
        self.out_features = out_features
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if gather not in ("auto", "fused", "nccl", "gloo"):
            raise ValueError(f"gather must be auto/fused/nccl/gloo, got {gather!r}")
        self.gather = gather
        self._symm = None  # (rows, buffer, handle, destination pointers)

    @classmethod
    def from_float(cls, mod: nn.Module, group=None, dtype: QDtype = qint8, act_scheme: str = "token_symmetric",
                   gather: str = "auto") -> "ColumnParallelLinear":
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        lo, hi = shard_rows(mod.out_features, world, rank)
        local = nn.Linear(mod.in_features, hi - lo, bias=mod.bias is not None)
        with torch.no_grad():
            local.weight.copy_(mod.weight[lo:hi])
            if mod.bias is not None:
                local.bias.copy_(mod.bias[lo:hi])
        shard = DynamicLinear.from_float(local, dtype).set_activation_scheme(act_scheme)
        return cls(shard, mod.out_features, group, gather)

    # -- fused exchange ------------------------------------------------------------------
    def _symmetric_buffer(self, rows: int, device):
        if self._symm is None or self._symm[0] != rows:
            import torch.distributed._symmetric_memory as symm

            buf = symm.empty((rows, self.out_features), dtype=torch.float32, device=device)
            hdl = symm.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            per = self.out_features // self.world
            order = [(self.rank + i) % self.world for i in range(self.world)]
            ptrs = [int(hdl.buffer_ptrs[r]) + self.rank * per * 4 for r in order]
            self._symm = (rows, buf, hdl, ptrs)
        return self._symm[1:]

    def _forward_fused(self, x2: torch.Tensor) -> torch.Tensor:
        ops = _backend.ops()
        sh = self.shard
        buf, hdl, ptrs = self._symmetric_buffer(x2.shape[0], x2.device)
        wq, wsum = sh._cache.get(sh.weight_int8)
        xq, sx, zx = sh._quantize_activations(x2)
        ops.qlinear_i8_into(xq, wq, sx, sh.weight_scale, ptrs, self.out_features, bias=sh.bias, zx=zx,
                            wsum=wsum if zx is not None else None)
        hdl.barrier()
        return buf

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        mode = self.gather
        if mode == "auto":
            mode = "fused" if x.is_cuda else "gloo"
        if mode == "fused":
            x2 = x.reshape(-1, x.shape[-1]).float()
            return self._forward_fused(x2).reshape(*lead, self.out_features)
        y = self.shard(x)  # [..., N/P]
        y2 = y.reshape(-1, y.shape[-1]).contiguous()
        parts = [torch.empty_like(y2) for _ in range(self.world)]
        dist.all_gather(parts, y2, group=self.group)
        return torch.cat(parts, dim=1).reshape(*lead, self.out_features)
