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


def _noise_worker(rank, world, port, systems, nodes, q):
    sys.path.insert(0, os.path.join(ROOT, "learned-dynamics_b200"))
    from ld_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    b, e = sharding.shard_range(systems, rank, world)
    x = torch.zeros(e - b, nodes, 3)
    for step in range(3):   # a three-step "rollout": x += 0.1 * noise(system, step)
        x = sharding.shard_noise(tuple(x.shape), b, 777, step, "cpu", base=x, scale=0.1)
    out = sharding.gather_positions(x, systems)
    if rank == 0:
        full = torch.zeros(systems, nodes, 3)
        for step in range(3):
            full = sharding.shard_noise(tuple(full.shape), 0, 777, step, "cpu", base=full, scale=0.1)
        q.put(bool(torch.equal(out, full)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("systems", [8, 5])
def test_sharded_noise_equals_single_rank_noise(systems):
    """noise keyed by (global system, step): the gathered result of two ranks is bit-identical to one rank's"""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000) + systems
    procs = [ctx.Process(target=_noise_worker, args=(r, 2, port, systems, 6, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_counter_noise_is_standard_normal_and_keyed():
    sys.path.insert(0, os.path.join(ROOT, "learned-dynamics_b200"))
    from ld_b200 import sharding
    z = sharding.counter_noise_torch(0, 1 << 20, 777, 0)
    assert torch.isfinite(z).all()
    assert abs(z.mean().item()) < 5e-3 and abs(z.std().item() - 1.0) < 5e-3
    assert abs((z[:-1] * z[1:]).mean().item()) < 5e-3                     # neighbouring elements uncorrelated
    assert abs(z.pow(4).mean().item() - 3.0) < 0.05                        # Gaussian fourth moment
    assert torch.equal(sharding.counter_noise_torch(1000, 64, 777, 0), z[1000:1064])
    assert not torch.equal(sharding.counter_noise_torch(0, 64, 777, 1), z[:64])
    assert not torch.equal(sharding.counter_noise_torch(0, 64, 778, 0), z[:64])
