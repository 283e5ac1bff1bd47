"""Multi-rank host logic on CPU (gloo, world_size 2): shard ranges cover the batch, the gather to
rank 0 reassembles it in order, and unequal shard sizes work."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, systems, q):
    sys.path.insert(0, os.path.join(ROOT, "learned-dynamics_b200"))
    from ld_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    b, e = sharding.shard_range(systems, rank, world)
    full = torch.arange(systems * 4 * 3, dtype=torch.float32).reshape(systems, 4, 3)
    out = sharding.gather_positions(full[b:e].clone(), systems)
    if rank == 0:
        q.put(bool(torch.equal(out, full)))
    else:
        assert out is None
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("systems", [16, 7])
def test_gather_reassembles_batch(systems):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + systems
    procs = [ctx.Process(target=_worker, args=(r, 2, port, systems, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_shard_ranges_partition():
    sys.path.insert(0, os.path.join(ROOT, "learned-dynamics_b200"))
    from ld_b200 import sharding
    for systems in (1, 7, 16, 1024):
        for world in (1, 2, 3, 8):
            rs = [sharding.shard_range(systems, r, world) for r in range(world)]
            assert rs[0][0] == 0 and rs[-1][1] == systems
            assert all(rs[i][1] == rs[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in rs]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.noise_seed(5, 3) != sharding.noise_seed(3, 5)
