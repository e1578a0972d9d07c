"""Host-to-host forward of a quantized Linear over row chunks.

When activations start and results end in host memory, the PCIe copies dwarf the GEMM.
``forward_from_host`` cuts the batch into row chunks and runs three stages on three
streams -- host-to-device copy of chunk i+1, the layer on chunk i, device-to-host copy
of chunk i-1 -- so the two copy directions (PCIe is full duplex) and the compute overlap.
Only layers whose activation grid is per row (``act_scheme == "token_symmetric"``) give
the same result chunked as whole, so others are rejected.

With a process group (one rank per GPU, every rank holding the same ``x_host`` and its own shard
of a column-parallel layer) a rank uploads only its 1/P of every chunk's rows and the ranks
all-gather the chunk over NVLink, so the host delivers the activations once instead of P times.
"""
from __future__ import annotations

import torch


def forward_from_host(module, x_host: torch.Tensor, out_host: torch.Tensor, chunk_rows: int = 2048,
                      device: torch.device | None = None, group=None) -> torch.Tensor:
    """``out_host[:] = module(x_host)`` with pinned 2-D ``x_host`` / ``out_host``; returns ``out_host``.
    The call returns once all work is enqueued; the current stream waits for the last copy.
    ``group``: see the module docstring; chunks whose row count the group size does not divide are
    uploaded whole by every rank."""
    if getattr(module, "act_scheme", None) != "token_symmetric":
        raise ValueError("forward_from_host needs a per-row activation grid (act_scheme='token_symmetric'): "
                         "a per-tensor range over a chunk differs from the range over the whole batch")
    if x_host.dim() != 2 or out_host.dim() != 2 or x_host.shape[0] != out_host.shape[0]:
        raise ValueError("x_host and out_host must be 2-D with the same number of rows")
    if not (x_host.is_pinned() and out_host.is_pinned()):
        raise ValueError("x_host and out_host must be pinned host tensors")
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    rows, k = x_host.shape
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(cur)
    xbuf = [torch.empty((min(chunk_rows, rows), k), dtype=x_host.dtype, device=dev) for _ in range(2)]
    consumed = [None, None]  # event: the layer has read xbuf[b]
    world, rank = 1, 0
    if group is not None:
        import torch.distributed as dist

        world, rank = dist.get_world_size(group), dist.get_rank(group)
    piece = [torch.empty((-(-min(chunk_rows, rows) // world), k), dtype=x_host.dtype, device=dev) for _ in range(2)] \
        if world > 1 else None
    for i, r0 in enumerate(range(0, rows, chunk_rows)):
        r1 = min(rows, r0 + chunk_rows)
        b = i & 1
        with torch.cuda.stream(s_in):
            if consumed[b] is not None:
                s_in.wait_event(consumed[b])
            n = r1 - r0
            if world > 1 and n % world == 0:
                part = n // world
                piece[b][:part].copy_(x_host[r0 + rank * part: r0 + (rank + 1) * part], non_blocking=True)
                dist.all_gather_into_tensor(xbuf[b][:n], piece[b][:part], group=group)
            else:
                xbuf[b][:n].copy_(x_host[r0:r1], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(s_in)
        cur.wait_event(arrived)
        y = module(xbuf[b][: r1 - r0])
        consumed[b] = torch.cuda.Event()
        consumed[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(consumed[b])
            out_host[r0:r1].copy_(y, non_blocking=True)
            y.record_stream(s_out)
    cur.wait_stream(s_out)
    return out_host
