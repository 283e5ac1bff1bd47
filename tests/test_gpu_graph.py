"""Radius graph on the GPU (through the C ABI) against the brute-force CPU oracle: bit-exact as
sorted (i, j, shift) sets; r_ij exact."""
import pytest
import torch

from oracle import reference_math as R

pytestmark = pytest.mark.gpu


def _gpu_graph(pos, cutoff, box, mode=0, **kw):
    from ld_b200 import graph as G
    B, N, _ = pos.shape
    b = G.RadiusGraphBuilder(B, N, cutoff, box, mode=mode, **kw)
    g = b.build(pos.cuda(), want_shift=True, want_rij=True)
    G.check_status_flags(b.status) if torch.isfinite(pos).all() else None
    return g, b


def _canon(src, dst, shift, rij):
    """sort edges by (src, dst); returns int64 keys + aligned payloads"""
    key = src.long() * (1 << 32) + dst.long()
    order = torch.argsort(key)
    return key[order], shift[order], rij[order]


def _assert_same(pos, cutoff, box, mode=0, **kw):
    from ld_b200 import graph as G
    g, _ = _gpu_graph(pos, cutoff, box, mode, **kw)
    o = R.radius_graph(pos, cutoff, box, mode)
    assert g["E"] == o["E"], (g["E"], o["E"])
    Nt = pos.shape[0] * pos.shape[1]
    row_ptr = g["row_ptr"].cpu()
    assert row_ptr[0] == 0 and row_ptr[-1] == g["E"]
    assert torch.equal((row_ptr[1:] - row_ptr[:-1]), o["degree"])
    src, dst = g["src"].cpu(), g["dst"].cpu()
    assert torch.all(src[1:] >= src[:-1]), "src must be non-decreasing"
    k1, s1, r1 = _canon(src, dst, G.unpack_shift(g["shift"]).cpu(), g["rij"].cpu())
    k2, s2, r2 = _canon(o["src"], o["dst"], o["shift"], o["rij"])
    assert torch.equal(k1, k2)
    assert torch.equal(s1, s2)
    assert torch.equal(r1, r2), "r_ij must be bit-identical to the oracle's float32 boxwrap"
    B = pos.shape[0]
    cum = torch.tensor([int(row_ptr[(b + 1) * pos.shape[1]]) for b in range(B)], dtype=torch.int32)
    assert torch.equal(g["edge_counts"].cpu(), cum)
    return g


def test_reference_known_answer(golden):
    k = golden["graph_kat"]
    g = _assert_same(k["positions"], k["r0"], k["box"])
    from ld_b200 import graph as G
    deg = G.segment_sum(torch.ones(g["E"], device="cuda"), g["row_ptr"], 5)
    assert torch.allclose(deg.cpu()[None], k["degrees"])


@pytest.mark.parametrize("mode", [0, 1])
def test_periodic_small_boxes(mode):
    gen = torch.Generator().manual_seed(11)
    box = (16.0, 16.0, 16.0)
    pos = torch.rand(3, 700, 3, generator=gen) * 16.0
    _assert_same(pos, 2.5, box, mode)


def test_periodic_anisotropic_and_outside_box():
    gen = torch.Generator().manual_seed(12)
    box = (30.5, 33.5, 36.5)  # the reference's own test box (extensions/neighbour_grid/test.py:11)
    pos = (torch.rand(20, 60, 3, generator=gen) * 3 - 1) * torch.tensor(box)
    _assert_same(pos, 7.0, box, 0)
    _assert_same(pos, 7.0, box, 1)


def test_periodic_few_cells():
    gen = torch.Generator().manual_seed(13)
    pos = torch.rand(2, 300, 3, generator=gen) * 10
    _assert_same(pos, 4.0, (8.5, 9.0, 12.5), 0)   # 2, 2 and 3 cells per axis
    _assert_same(pos, 4.9, (10.0, 10.0, 10.0), 0)  # 2 cells per axis


def test_open_polymers():
    gen = torch.Generator().manual_seed(14)
    pos = torch.cumsum(torch.randn(8, 64, 3, generator=gen) / 3 ** 0.5, dim=1)
    _assert_same(pos, 3.0, None)
    pos = torch.cumsum(torch.randn(4, 512, 3, generator=gen) / 3 ** 0.5, dim=1)
    _assert_same(pos, 5.0, None)
    _assert_same(pos, 5.0, None, open_cells_cap=8)  # coarsened grid must give the same graph


def test_edge_cases():
    gen = torch.Generator().manual_seed(15)
    # one node per system, two coincident nodes, all nodes in one cell, empty batch
    _assert_same(torch.rand(5, 1, 3, generator=gen), 1.0, (4.0, 4.0, 4.0))
    p = torch.zeros(1, 2, 3)
    g = _assert_same(p, 1.0, None)
    assert g["E"] == 2
    _assert_same(torch.rand(2, 40, 3, generator=gen) * 0.1, 1.0, (5.0, 5.0, 5.0))
    _assert_same(torch.rand(2, 40, 3, generator=gen) * 0.1, 1.0, None)
    from ld_b200 import graph as G
    b = G.RadiusGraphBuilder(0, 10, 1.0, (4.0, 4.0, 4.0))
    g = b.build(torch.zeros(0, 10, 3, device="cuda"))
    assert g["E"] == 0


def test_errors_and_flags():
    from ld_b200 import graph as G, _lib
    with pytest.raises(_lib.HotpathError) as e:
        G.RadiusGraphBuilder(1, 10, 3.0, (5.0, 5.0, 5.0))
    assert e.value.status == _lib.LD_ERR_BOX_TOO_SMALL
    pos = torch.rand(1, 50, 3)
    pos[0, 7, 1] = float("nan")
    b = G.RadiusGraphBuilder(1, 50, 0.3, (1.0, 1.0, 1.0))
    b.build(pos.cuda())
    with pytest.raises(RuntimeError, match="NaN"):
        G.check_status_flags(b.status)
    # fixed capacity smaller than E raises the capacity flag and writes nothing past the end
    pos = torch.rand(1, 200, 3)
    b = G.RadiusGraphBuilder(1, 200, 0.3, (1.0, 1.0, 1.0))
    g = b.build(pos.cuda())
    cap = g["E"] // 2
    src = torch.full((cap + 8,), -7, dtype=torch.int32, device="cuda")
    dst = torch.full((cap + 8,), -7, dtype=torch.int32, device="cuda")
    b.status.zero_()
    b.build_fixed(pos.cuda(), cap, src, dst)
    assert int(b.status.item()) & _lib.LD_FLAG_CAPACITY
    assert (src[cap:] == -7).all() and (dst[cap:] == -7).all()


def test_deterministic_order():
    gen = torch.Generator().manual_seed(16)
    pos = (torch.rand(4, 2000, 3, generator=gen) * 12.0).cuda()
    from ld_b200 import graph as G
    b = G.RadiusGraphBuilder(4, 2000, 2.0, (12.0, 12.0, 12.0))
    g1 = b.build(pos)
    g2 = b.build(pos)
    assert torch.equal(g1["dst"], g2["dst"]) and torch.equal(g1["rij"], g2["rij"])


def test_benchmark_config_1_all_systems_and_full_properties():
    """32 periodic boxes L=16 x 4096 uniform particles, cutoff 2.5: all 32 systems bit-exact against the brute-force
    oracle (edge set, lattice shifts, displacements), then size-independent properties (symmetry, degree sums)."""
    gen = torch.Generator().manual_seed(1001)
    pos = torch.rand(32, 4096, 3, generator=gen) * 16.0
    box = (16.0, 16.0, 16.0)
    from ld_b200 import graph as G
    b = G.RadiusGraphBuilder(32, 4096, 2.5, box)
    g = b.build(pos.cuda(), want_shift=True)
    G.check_status_flags(b.status)
    o = R.radius_graph(pos, 2.5, box)
    assert g["E"] == o["E"]
    k1, s1, r1 = _canon(g["src"].cpu(), g["dst"].cpu(), G.unpack_shift(g["shift"]).cpu(), g["rij"].cpu())
    k2, s2, r2 = _canon(o["src"], o["dst"], o["shift"], o["rij"])
    assert torch.equal(k1, k2) and torch.equal(s1, s2) and torch.equal(r1, r2)
    per_system = torch.bincount(o["src"].long() // 4096, minlength=32)
    assert torch.equal(torch.cumsum(per_system, 0).to(torch.int32), g["edge_counts"].cpu())
    # symmetry of the whole batch: the multiset of (min,max) pairs has every pair exactly twice
    s, d = g["src"].long(), g["dst"].long()
    fwd = torch.sort(s * (1 << 32) + d).values
    bwd = torch.sort(d * (1 << 32) + s).values
    assert torch.equal(fwd, bwd)
    assert (s // 4096 == d // 4096).all(), "edges never cross systems"
    assert abs(g["E"] / (32 * 4096) - 65.4) < 1.0  # mean degree of the uniform density-1 box
    # every reported displacement is within the cutoff and antisymmetric
    assert (g["rij"].norm(dim=1) <= 2.5 * (1 + 1e-6)).all()
