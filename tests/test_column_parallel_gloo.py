"""N > 1 host logic on CPU: two gloo ranks, each with an oracle-backed stand-in for the
kernels, run the column-parallel dynamic Linear; the gathered result must equal the
unsharded one bit for bit (K is not split, so sharding changes no arithmetic)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lucid_b200 import _backend
    from tests import fake_ops

    cpu = torch.device("cpu")
    _backend.ops = lambda: fake_ops
    _backend.on_cuda = lambda t: t.to(cpu)
    _backend.cuda_device = lambda index=None: cpu
    from lucid_b200.nn.quantized.column_parallel import ColumnParallelLinear, shard_rows
    from lucid_b200.nn.quantized.dynamic import Linear as DynLinear

    torch.manual_seed(0)  # same float layer and input on every rank
    lin = nn.Linear(48, 64)
    x = torch.randn(3, 5, 48)
    for scheme in ("token_symmetric", "tensor_affine"):
        cp = ColumnParallelLinear.from_float(lin, act_scheme=scheme, gather="gloo")
        assert shard_rows(64, world, rank) == (rank * 32, rank * 32 + 32)
        assert tuple(cp.shard.weight_int8.shape) == (32, 48)
        y = cp(x)
        full = DynLinear.from_float(lin).set_activation_scheme(scheme)(x)
        assert y.shape == (3, 5, 64)
        assert torch.equal(y, full), f"rank {rank}: sharded result differs ({scheme})"
    with pytest.raises(ValueError):
        shard_rows(10, 3, 0)
    np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([1]))
    dist.destroy_process_group()


def test_column_parallel_two_gloo_ranks(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok_{r}.npy") for r in range(world))
