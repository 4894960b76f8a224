"""Batch sharding across ranks, exercised with two gloo ranks on CPU: the
slices partition the batch, per-rank results reassemble to the unsharded
result, and the optional gather returns the full batch on every rank."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from flagdnn_b200.sharding import batch_slice, gather_batch, shard_batch


@pytest.mark.parametrize("n,world", [(256, 1), (256, 2), (256, 8), (1024, 8), (7, 2), (5, 8), (0, 4)])
def test_slices_partition_the_batch(n, world):
    edges = [batch_slice(n, r, world) for r in range(world)]
    assert edges[0][0] == 0 and edges[-1][1] == n
    for (b0, e0), (b1, e1) in zip(edges, edges[1:]):
        assert e0 == b1
    sizes = [e - b for b, e in edges]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        batch_slice(n, world, world)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_total, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)  # same seed on every rank: replicated filter
        x = torch.randn(n_total, 6, 9, 9, generator=g)
        w = torch.randn(4, 6, 3, 3, generator=g)
        b = torch.randn(4, generator=g)
        x_local = shard_batch(x, rank, world)
        # the per-rank compute leg is the CPU oracle here; on GPUs it is the native library
        y_local = oracle.conv2d_torch_cpu(x_local, w, b, 1, 1, 1, 1, relu=True)
        y_all = gather_batch(y_local, n_total)
        y_ref = oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1, relu=True)
        torch.testing.assert_close(y_all, y_ref, rtol=0, atol=1e-6)
        # timing reduction used by the benchmark: max over ranks
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_total", [8, 7])
def test_two_rank_sharded_run_reassembles(tmp_path, n_total):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_total, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def _worker_partner_leaves(rank, world, port, result_dir):
    """Rank 1 leaves between steps (after a completed gather, with nothing in flight); rank 0's next gather must
    end with an error within the process group's timeout instead of waiting forever."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    y_local = torch.full((2, 3), float(rank))
    first = gather_batch(y_local, 4)                      # step 1: both ranks take part
    assert first.shape == (4, 3) and first[:2].eq(0).all() and first[2:].eq(1).all()
    if rank == 1:
        open(os.path.join(result_dir, "left1"), "w").close()
        os._exit(0)                                       # gone: no further collective, no clean shutdown
    t0 = time.monotonic()
    try:
        gather_batch(y_local, 4)                          # step 2: the partner never joins
        outcome = "returned"
    except Exception as exc:                              # gloo reports a timeout or a closed connection
        outcome = f"error:{type(exc).__name__}"
    took = time.monotonic() - t0
    with open(os.path.join(result_dir, "rank0"), "w") as fh:
        fh.write(f"{outcome} {took:.1f}")
    os._exit(0)                                           # the group cannot be torn down cleanly without its partner


def test_gather_with_a_departed_rank_fails_within_the_timeout(tmp_path):
    world = 2
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker_partner_leaves, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode is not None, "a rank is still waiting: the departed partner hung it"
    assert os.path.exists(tmp_path / "left1")
    outcome, took = open(tmp_path / "rank0").read().split()
    assert outcome.startswith("error:"), outcome
    assert float(took) < 60.0
