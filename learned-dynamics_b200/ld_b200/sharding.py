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


_M1, _M2 = -4658895280553007687, -7723592293110705685      # 0xBF58476D1CE4E5B9, 0x94D049BB133111EB as int64
_K1 = -7046029254386353131                                  # 0x9E3779B97F4A7C15 as int64


def _wrap64(v):
    """Python integer -> the int64 with the same low 64 bits"""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(x, k):
    """logical right shift of int64 tensors (torch's >> is arithmetic)"""
    return (x >> k) & ((1 << (64 - k)) - 1)


def counter_noise_torch(first_element, count, seed, step, device="cpu"):
    """N(0,1) values number first_element .. first_element+count-1 of the noise field of (seed, step): the arithmetic of
    ld_counter_noise in torch integer operations (64-bit wrapping multiply, splitmix64 finaliser, Box-Muller).
    Element numbering of a batch [systems, nodes, 3]: ((system * nodes) + node) * 3 + component, so a shard's values
    are a contiguous range and do not depend on how the batch is split over ranks."""
    key = _wrap64(seed * 0x9E3779B97F4A7C15 + step * 0xBF58476D1CE4E5B9)
    x = torch.arange(first_element, first_element + count, dtype=torch.int64, device=device) + key
    x = (x ^ _lsr(x, 30)) * _M1
    x = (x ^ _lsr(x, 27)) * _M2
    x = x ^ _lsr(x, 31)
    u1 = (_lsr(x, 40) + 1).to(torch.float32) * (1.0 / 16777216.0)
    u2 = (_lsr(x, 16) & 0xFFFFFF).to(torch.float32) * (1.0 / 16777216.0)
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)


def shard_noise(shape, first_system, seed, step, device, base=None, scale=1.0):
    """base + scale * noise for the systems [first_system, first_system + shape[0]) of a batch whose per-system shape is
    shape[1:] (one kernel launch on a CUDA device). The values are those a single rank owning the whole batch draws."""
    per = 1
    for d in shape[1:]:
        per *= d
    count, first = shape[0] * per, first_system * per
    dev = torch.device(device)
    if dev.type != "cuda":
        z = counter_noise_torch(first, count, seed, step, dev).reshape(shape)
        return z * scale if base is None else base + scale * z
    from ._lib import lib, check, ptr, stream_ptr, KERNEL_TIMER
    out = torch.empty(shape, dtype=torch.float32, device=dev)
    if base is not None:
        base = base.contiguous()
        assert base.shape == out.shape and base.dtype == torch.float32
    with KERNEL_TIMER.region("counter_noise"):
        check(lib().ld_counter_noise(ptr(out), ptr(base), float(scale), first, count, seed, step, stream_ptr(dev)))
    return out


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
