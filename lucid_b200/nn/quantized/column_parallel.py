"""Column-parallel dynamic int8 Linear over several GPUs of one node.

The reference has no multi-device path; this is the N-sharded form of its dynamic Linear
(``lucid/nn/quantized/dynamic/linear.py:85-109``).  Rank r keeps output rows
``[r*N/P, (r+1)*N/P)`` of the quantized weight, the input is replicated and quantized
locally, K is not split, so every output column is bit-identical to the single-GPU result.
Every rank ends up with the whole ``[M, N]`` fp32 result.  The shards are exchanged by one of

* ``"fused"``: inside the GEMM epilogue -- each rank stores its tiles straight into the result
  buffer of every rank (plain peer stores over NVLink through symmetric memory);
* ``"multimem"``: inside the GEMM epilogue, one ``multimem.st`` per tile segment to the
  buffer's multicast address; the NVSwitch replicates it into every rank's buffer;
* ``"copy"``: the GEMM runs in row bands into this rank's buffer, and while band i+1 is being
  computed the copy engines push band i's column block into the peers' buffers
  (``cudaMemcpy2DAsync`` on a second stream);
* ``"nccl"`` / ``"gloo"``: a plain all-gather of the local ``[M, N/P]`` shard (the baseline).

The first three write into symmetric-memory result buffers and synchronise the ranks with this
library's own barrier kernel (``lc_peer_barrier``), whose device-side wait is bounded: a peer that
never arrives costs about a second and an error from :meth:`check`, not a hung GPU.

Result lifetime: the module owns TWO result buffers and alternates between them, and every
forward begins with a barrier.  The tensor returned by forward n is therefore valid until forward
n + 2 starts on this rank's stream (enqueue its consumers before that); keep a ``clone()`` to hold
it longer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from lucid_b200 import _backend
from lucid_b200.nn.quantized.dynamic.linear import Linear as DynamicLinear
from lucid_b200.quantization._qscheme import QDtype, qint8

_SYMMETRIC_MODES = ("fused", "multimem", "copy")


def shard_rows(out_features: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open row range of ``rank``; ``out_features`` must divide evenly."""
    if out_features % world:
        raise ValueError(f"out_features={out_features} does not split over {world} ranks")
    per = out_features // world
    return rank * per, (rank + 1) * per


class _Exchange:
    """Symmetric-memory state of one (rows, device): two result buffers, the flag arrays of the
    barrier, a status word, and the raw addresses of every rank's copies."""

    def __init__(self, rows: int, out_features: int, device, group, rank: int, world: int) -> None:
        import torch.distributed._symmetric_memory as symm

        grp = group if group is not None else dist.group.WORLD
        self.rows = rows
        self.buffers, self.handles = [], []
        for _ in range(2):
            buf = symm.empty((rows, out_features), dtype=torch.float32, device=device)
            self.buffers.append(buf)
            self.handles.append(symm.rendezvous(buf, grp))
        self.flags = symm.empty((world,), dtype=torch.int32, device=device)
        self.flags.zero_()
        flag_handle = symm.rendezvous(self.flags, grp)
        self.flag_ptrs = [int(flag_handle.buffer_ptrs[r]) for r in range(world)]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.turn = 0
        self.side = torch.cuda.Stream(device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every rank's flags are zero before anyone's first epoch can land

    def multicast_ptr(self, which: int) -> int:
        return int(getattr(self.handles[which], "multicast_ptr", 0) or 0)


class ColumnParallelLinear(nn.Module):
    def __init__(self, shard: DynamicLinear, out_features: int, group=None, gather: str = "auto",
                 band_rows: int = 4096) -> None:
        super().__init__()
        self.shard = shard
        self.out_features = out_features
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if gather not in ("auto", "nccl", "gloo") + _SYMMETRIC_MODES:
            raise ValueError(f"gather must be one of auto/fused/multimem/copy/nccl/gloo, got {gather!r}")
        self.gather = gather
        self.band_rows = band_rows
        self._exchange: _Exchange | None = None

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

    # -- exchange through symmetric memory ---------------------------------------------------
    def _state(self, rows: int, device) -> _Exchange:
        if self._exchange is None or self._exchange.rows != rows:
            self._exchange = _Exchange(rows, self.out_features, device, self.group, self.rank, self.world)
        return self._exchange

    def _barrier(self, ex: _Exchange, device) -> None:
        ex.epoch += 1
        _backend.ops().peer_barrier(ex.flag_ptrs, self.rank, ex.epoch, status=ex.status, device=device)

    def check(self) -> None:
        """Synchronise and raise if a bounded device-side wait of this module ran out (a peer that
        never reached a barrier, or a GEMM role that gave up)."""
        if self._exchange is not None:
            _backend.ops().qlinear_check_status(self._exchange.status)

    def _forward_symmetric(self, x2: torch.Tensor, mode: str) -> torch.Tensor:
        ops = _backend.ops()
        sh = self.shard
        ex = self._state(x2.shape[0], x2.device)
        which = ex.turn
        ex.turn ^= 1
        buf, hdl = ex.buffers[which], ex.handles[which]
        per = self.out_features // self.world
        col_bytes = self.rank * per * 4
        wq, wsum = sh._cache.get(sh.weight_int8, sh.weight_zero_point)
        xq, sx, zx = sh._quantize_activations(x2)
        kw = dict(bias=sh.bias, zx=zx, wsum=wsum if zx is not None else None, status=ex.status)
        # nobody's consumers still read this buffer (their result n - 2) once every rank is here
        self._barrier(ex, x2.device)
        if mode == "multimem":
            mc = ex.multicast_ptr(which)
            if not mc:
                raise RuntimeError("gather='multimem' needs a multicast mapping of the result buffer (NVLS); "
                                   "this process group has none")
            ops.qlinear_i8_into(xq, wq, sx, sh.weight_scale, [mc + col_bytes], self.out_features, multicast=True, **kw)
        elif mode == "fused":
            order = [(self.rank + i) % self.world for i in range(self.world)]  # own buffer first, peers rotated
            ptrs = [int(hdl.buffer_ptrs[r]) + col_bytes for r in order]
            ops.qlinear_i8_into(xq, wq, sx, sh.weight_scale, ptrs, self.out_features, **kw)
        else:  # "copy": GEMM band by band into the own buffer, copy engines push finished bands to the peers
            rows, pitch = x2.shape[0], self.out_features * 4
            own = int(hdl.buffer_ptrs[self.rank]) + col_bytes
            main = torch.cuda.current_stream(x2.device)
            per_row = sx.numel() == rows and rows != 1
            for r0 in range(0, rows, self.band_rows):
                r1 = min(rows, r0 + self.band_rows)
                ops.qlinear_i8_into(xq[r0:r1], wq, sx[r0:r1] if per_row else sx, sh.weight_scale,
                                    [own + r0 * pitch], self.out_features, **kw)
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(ex.side):
                    ex.side.wait_event(done)
                    for i in range(1, self.world):
                        peer = (self.rank + i) % self.world
                        ops.copy_2d(int(hdl.buffer_ptrs[peer]) + col_bytes + r0 * pitch, pitch, own + r0 * pitch, pitch,
                                    per * 4, r1 - r0, x2.device)
            main.wait_stream(ex.side)
        self._barrier(ex, x2.device)  # every rank's column blocks have landed in this rank's buffer
        return buf

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        mode = self.gather
        if mode == "auto":
            mode = "fused" if x.is_cuda else "gloo"
        if mode in _SYMMETRIC_MODES:
            x2 = x.reshape(-1, x.shape[-1]).float()
            return self._forward_symmetric(x2, mode).reshape(*lead, self.out_features)
        y = self.shard(x)  # [..., N/P]
        y2 = y.reshape(-1, y.shape[-1]).contiguous()
        parts = [torch.empty_like(y2) for _ in range(self.world)]
        dist.all_gather(parts, y2, group=self.group)
        return torch.cat(parts, dim=1).reshape(*lead, self.out_features)
