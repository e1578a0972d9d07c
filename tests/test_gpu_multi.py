"""Multi-GPU plumbing: the bounded barrier between ranks and the copy-engine block copy on one GPU
(a peer that never arrives is simulated by a flag nobody writes: the wait runs out, nothing hangs),
and the column-parallel Linear on two GPUs when the box has them."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lucid_b200._C import ops

    return ops


def test_peer_barrier_wait_is_bounded(ops):
    """World of two whose second rank never shows up: this rank's wait for it gives up after the
    cycle budget, the status word maps to LC_ERR_TIMEOUT, and the GPU keeps working."""
    from lucid_b200._C import LC_ERR_TIMEOUT, LucidCudaError

    mine = torch.zeros(2, dtype=torch.int32, device="cuda")
    absent = torch.zeros(2, dtype=torch.int32, device="cuda")  # stands for the peer's array; the peer writes nothing
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.peer_barrier([mine.data_ptr(), absent.data_ptr()], 0, 1, status=status, wait_cycles=200_000)
    with pytest.raises(LucidCudaError) as info:
        ops.qlinear_check_status(status)
    assert info.value.code == LC_ERR_TIMEOUT and "peer never arrived" in str(info.value)
    assert mine.tolist() == [1, 0] and absent.tolist() == [1, 0]  # this rank did publish its arrival
    # the "peer" arrives (its epoch lands in this rank's array): the same barrier now passes
    mine[1] = 2
    ops.peer_barrier([mine.data_ptr(), absent.data_ptr()], 0, 2, status=status, wait_cycles=200_000)
    ops.qlinear_check_status(status)
    assert mine.tolist() == [2, 2]
    # a world of one is a no-op barrier
    solo = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):
        ops.peer_barrier([solo.data_ptr()], 0, epoch, status=status)
    ops.qlinear_check_status(status)
    assert solo.item() == 3


def test_copy_2d_moves_a_column_block(ops):
    src = torch.arange(6 * 10, device="cuda", dtype=torch.float32).reshape(6, 10)
    dst = torch.zeros(6, 10, device="cuda")
    ops.copy_2d(dst.data_ptr() + 3 * 4, 40, src.data_ptr() + 3 * 4, 40, 4 * 4, 5, src.device)
    torch.cuda.synchronize()
    want = torch.zeros(6, 10, device="cuda")
    want[:5, 3:7] = src[:5, 3:7]
    assert torch.equal(dst, want)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist
    from torch import nn

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from lucid_b200.nn.quantized.column_parallel import ColumnParallelLinear
    from lucid_b200.nn.quantized.dynamic import Linear as DynLinear

    torch.manual_seed(0)  # the same float layer and inputs on every rank
    lin = nn.Linear(512, 1024)
    xs = [torch.randn(700, 512) for _ in range(3)]
    full = DynLinear.from_float(lin).set_activation_scheme("token_symmetric").to(dev)
    want = [full(x.to(dev)).clone() for x in xs]
    cp = ColumnParallelLinear.from_float(lin, act_scheme="token_symmetric", gather="fused").to(dev)
    cp.band_rows = 256
    tried = []
    for mode in ("fused", "copy", "multimem"):
        cp.gather = mode
        try:
            y1 = cp(xs[0].to(dev))
            y2 = cp(xs[1].to(dev))  # y1 must survive one more forward (two result buffers)
            ok12 = torch.equal(y1, want[0]) and torch.equal(y2, want[1])
            y3 = cp(xs[2].to(dev))
            cp.check()
            assert ok12 and torch.equal(y3, want[2]) and torch.equal(y2, want[1]), f"rank {rank}: {mode} differs"
            tried.append(mode)
        except RuntimeError as e:
            if mode != "multimem" or "multicast" not in str(e):
                raise
    assert "fused" in tried and "copy" in tried
    # host-to-host streaming of this rank's column shard: uploading 1/P of every chunk and all-gathering it
    # gives the bits of uploading the whole chunk (700 rows: chunks of 256, 256 and an odd 188 -> whole upload)
    from lucid_b200.nn.quantized.streaming import forward_from_host

    xh = torch.cat([xs[0], xs[1][:68]]).pin_memory()  # 768 rows
    shard = cp.shard
    outs = []
    for grp, nrows in ((None, 768), (dist.group.WORLD, 768), (dist.group.WORLD, 700)):
        out = torch.empty((nrows, shard.out_features), dtype=torch.float32).pin_memory()
        forward_from_host(shard, xh[:nrows], out, chunk_rows=256, device=dev, group=grp)
        torch.cuda.synchronize(dev)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0][:700], outs[2]), f"rank {rank}: sharded upload differs"
    per = shard.out_features
    assert torch.equal(outs[0][:700].to(dev), want[0][:, rank * per:(rank + 1) * per]), f"rank {rank}: shard result differs"
    with open(os.path.join(out_dir, f"ok_{rank}"), "w") as f:
        f.write(",".join(tried))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_parallel_two_gpus(tmp_path):
    """Every exchange mode gives each rank the single-GPU result bit for bit, and a result stays
    intact while the next forward runs (the module alternates between two buffers)."""
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    mp.spawn(_two_gpu_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok_{r}") for r in range(world))
