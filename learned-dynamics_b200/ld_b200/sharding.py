"""Batch sharding across GPUs: independent systems are split into contiguous ranges, one per rank.
Nothing crosses ranks inside a step (node ids are b*N+i, cells and group norms are per system);
one gather of the final positions to rank 0 ends a rollout."""
import torch
import torch.distributed as dist


def shard_range(systems, rank, world):
    """contiguous [begin, end) of system indices owned by `rank`; sizes differ by at most one"""
    base, extra = divmod(systems, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def noise_seed(global_system_index, step, base_seed=777):
    """per-(system, step) seed: results do not depend on the number of ranks"""
    return (base_seed * 1000003 + global_system_index) * 1000003 + step


def gather_positions(x_local, systems, dst=0):
    """[systems_local, N, 3] on every rank -> [systems, N, 3] on rank `dst` (None elsewhere)"""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x_local
    world, rank = dist.get_world_size(), dist.get_rank()
    sizes = [shard_range(systems, r, world) for r in range(world)]
    most = max(e - b for b, e in sizes)
    # collectives want equal shapes: pad the shorter shards by one system
    local = x_local.contiguous()
    if local.shape[0] < most:
        pad = torch.zeros((most - local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        local = torch.cat([local, pad], dim=0)
    if rank == dst:
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.gather(local, parts, dst=dst)
        return torch.cat([p[: e - b] for p, (b, e) in zip(parts, sizes)], dim=0)
    dist.gather(local, None, dst=dst)
    return None
