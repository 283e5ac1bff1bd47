"""Rollout plumbing on the GPU: counter-based noise (identical whatever the sharding), fixed-capacity graph builds
(identical to the ordinary build, overflow reported), and a sharded rollout of the l<=2 denoiser that matches the
unsharded one bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_counter_noise_kernel_matches_torch_and_shards():
    from ld_b200 import sharding
    shape = (7, 33, 3)
    full = sharding.shard_noise(shape, 0, 777, 5, "cuda")
    want = sharding.counter_noise_torch(0, 7 * 33 * 3, 777, 5).reshape(shape)
    assert (full.cpu() - want).abs().max().item() < 2e-6      # same integers; logf / cosf differ in the last bit
    lo = sharding.shard_noise((3, 33, 3), 0, 777, 5, "cuda")
    hi = sharding.shard_noise((4, 33, 3), 3, 777, 5, "cuda")
    assert torch.equal(torch.cat([lo, hi]), full)              # a shard draws exactly its part of the full batch
    base = torch.randn(shape, device="cuda")
    fused = sharding.shard_noise(shape, 0, 777, 5, "cuda", base=base, scale=0.25)
    assert torch.allclose(fused, base + 0.25 * full, atol=1e-6)


@pytest.mark.parametrize("box", [None, (12.0, 12.0, 12.0)])
def test_rollout_graph_cache_equals_ordinary_build(box):
    from ld_b200 import graph as G, graph_layers as GL
    gen = torch.Generator().manual_seed(3)
    if box is None:
        pos = torch.cumsum(torch.randn(6, 200, 3, generator=gen) / 3 ** 0.5, dim=1).cuda()
    else:
        pos = (torch.rand(6, 200, 3, generator=gen) * 12.0).cuda()
    cache = G.RolloutGraphCache(margin=1.25)
    with torch.no_grad():
        for step in range(4):
            p = pos + 0.05 * step * torch.randn(pos.shape, generator=gen).cuda()
            want = GL.Graph.radius_graph(3.0, box, p)
            got = GL.Graph.radius_graph(3.0, box, p, cache=cache)
            E = want.src32.numel()
            assert int(got.num_edges_dev.item()) == E
            assert torch.equal(got.row_ptr, want.row_ptr)
            assert torch.equal(got.src32[:E], want.src32) and torch.equal(got.dst32[:E], want.dst32)
            assert torch.equal(got.rij[:E], want.rij)
            assert torch.equal(got.src, want.src)             # the int64 view is trimmed to the edge count
    cache.finish()


def test_rollout_graph_cache_reports_overflow():
    from ld_b200 import graph as G, graph_layers as GL, _lib
    gen = torch.Generator().manual_seed(4)
    pos = (torch.rand(2, 400, 3, generator=gen) * 10.0).cuda()
    cache = G.RolloutGraphCache(margin=1.05)
    with torch.no_grad():
        GL.Graph.radius_graph(2.0, (10.0,) * 3, pos, cache=cache)
        dense = pos * 0.5 + 2.5                                # same box, eight times the density: far more edges
        GL.Graph.radius_graph(2.0, (10.0,) * 3, dense, cache=cache)
        with pytest.raises(_lib.HotpathError) as err:
            cache.finish()
    assert err.value.status == _lib.LD_ERR_CAPACITY
    # the buffers were grown: the next build fits
    with torch.no_grad():
        g = GL.Graph.radius_graph(2.0, (10.0,) * 3, dense, cache=cache)
        cache.finish()
        want = GL.Graph.radius_graph(2.0, (10.0,) * 3, dense)
    assert int(g.num_edges_dev.item()) == want.src32.numel()


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_sharded_rollout_is_bit_identical_to_unsharded(precision):
    """three steps of the l<=2 denoiser on 6 systems in one batch, and as shards of 4 + 2 systems with the noise keyed by
    the global system index: the same positions bit for bit (what makes the 1/2/4/8-GPU results identical)"""
    from ld_b200 import bee, painn, sharding
    torch.manual_seed(11)
    dims = (64, 32, 32, 64)
    dn = bee.set_precision(bee.BeeDenoiser(4.0, *dims, ntypes=5, depth=2).cuda(), precision)
    gen = torch.Generator().manual_seed(12)
    x_all = torch.cumsum(torch.randn(6, 96, 3, generator=gen) / 3 ** 0.5, dim=1).cuda()
    types = torch.randint(0, 5, (96,), generator=gen).cuda()

    def rollout(begin, end, cached):
        if cached:
            painn.enable_rollout_graphs(dn)
        else:
            dn.graph_cache = None
        x = x_all[begin:end].clone()
        for step in range(3):
            noise = sharding.shard_noise(tuple(x.shape), begin, 777, step, "cuda")
            x = dn.generate(x, noise, 0.05, None, types)
        if cached:
            painn.finish_rollout_graphs(dn)
        return x

    whole = rollout(0, 6, cached=False)
    parts = torch.cat([rollout(0, 4, cached=True), rollout(4, 6, cached=True)])
    assert torch.equal(whole, parts)
