"""Fused l<=2 message layer against the reference's own Messages output (tests/golden) and against
the unfused op sequence on the same GPU. FP32; the radial basis is a degree-7 polynomial with
cancelling coefficients of order 1e3, so the bar is 1e-4 relative (max-norm) here."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def close(a, b, rel):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    scale = max(b.abs().max().item(), 1e-30)
    assert err <= rel * scale, f"max abs err {err:.3e} vs scale {scale:.3e} (rel {err / scale:.2e})"


def test_messages_against_reference_golden(golden):
    from ld_b200 import bee, graph_layers as GL
    p, m = golden["painn"], golden["bee_messages"]
    da, dv, dd, chan = m["dims"]
    mes = bee.Messages(p["r0"], da, dv, dd, chan)
    mes.load_state_dict(m["state"])
    mes.cuda()
    B, N = m["x_a"].shape[:2]
    graph = GL.Graph(p["src"].cuda(), p["dst"].cuda(), None, B, N)
    args = (graph, p["r_ij"].cuda(), m["x_a"].cuda(), m["x_v"].cuda(), m["x_d"].cuda())
    with torch.no_grad():
        fused = mes(*args)
    unfused = mes._forward_unfused(*args)
    for got, ref, want in zip(fused, unfused, m["out"]):
        close(ref, want, 1e-4)
        close(got, want, 1e-4)


@pytest.mark.parametrize("dims,B,N,r0,box", [((128, 64, 32, 128), 2, 200, 3.0, (9.0, 9.0, 9.5)), ((64, 32, 16, 96), 3, 50, 5.0, None),
                                             ((32, 8, 8, 32), 1, 6, 1.0, None)])
def test_messages_fused_vs_unfused(dims, B, N, r0, box):
    """benchmark config 2 widths (128, 64, 32, chan 128) in the first row"""
    from ld_b200 import bee, graph_layers as GL
    torch.manual_seed(sum(dims))
    mes = bee.Messages(r0, *dims).cuda()
    g = torch.Generator().manual_seed(7)
    if box is None:
        pos = torch.cumsum(torch.randn(B, N, 3, generator=g) / 3 ** 0.5, dim=1)
    else:
        pos = torch.rand(B, N, 3, generator=g) * torch.tensor(box)
    da, dv, dd, _ = dims
    x_a, x_v, x_d = torch.randn(B, N, da, generator=g), torch.randn(B, N, dv, 3, generator=g), torch.randn(B, N, dd, 3, 3, generator=g)
    with torch.no_grad():
        graph = GL.Graph.radius_graph(r0, box, pos.cuda())
        fused = mes(graph, graph.rij, x_a.cuda(), x_v.cuda(), x_d.cuda())
    unfused = mes._forward_unfused(graph, graph.rij, x_a.cuda(), x_v.cuda(), x_d.cuda())
    for got, ref in zip(fused, unfused):
        close(got, ref, 1e-4)


def test_bee_denoiser_vs_oracle():
    from ld_b200 import bee
    from oracle import reference_math as R
    torch.manual_seed(3)
    dims = (32, 16, 8, 32)
    ref = R.OBeeDenoiser(3.0, *dims, ntypes=5, depth=2)
    mine = bee.BeeDenoiser(3.0, *dims, ntypes=5, depth=2)
    mine.load_state_dict(ref.state_dict())
    mine.cuda()
    g = torch.Generator().manual_seed(9)
    B, N = 3, 48
    x0 = torch.cumsum(torch.randn(B, N, 3, generator=g) / 3 ** 0.5, dim=1)
    noise = torch.randn(B, N, 3, generator=g)
    types = torch.randint(0, 5, (N,), generator=g)
    x1 = x0 + 0.3 * noise
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    with torch.no_grad():
        want_v = ref(x0, x1, None, types)
        got_v = mine(x0.cuda(), x1.cuda(), None, types.cuda(), counter)
    assert want_v.abs().max() > 1e-3
    close(got_v, want_v, 2e-4)
    assert int(counter.item()) == ref.edges_last
    close(mine.generate(x0.cuda(), noise.cuda(), 0.3, None, types.cuda()), ref.generate(x0, noise, 0.3, None, types), 2e-4)


@pytest.mark.parametrize("dims,B,N,r0,box", [((128, 64, 32, 128), 2, 300, 3.0, (9.0, 9.0, 9.5)), ((64, 32, 16, 96), 3, 50, 5.0, None),
                                             ((128, 8, 8, 32), 1, 6, 1.0, None), ((128, 64, 32, 128), 8, 256, 5.0, None),
                                             ((64, 32, 32, 128), 3, 40, 0.9, None), ((64, 32, 32, 64), 2, 20, 0.01, None)])
def test_messages_tensor_core_vs_fp32(dims, B, N, r0, box):
    """scalar channel on tcgen05 (BF16 operands) against the FP32 fused kernels: 2e-2 relative. The last rows cover
    many tiles and node segments, a sparse graph with nodes without neighbours, and a graph without any edge."""
    from ld_b200 import bee, graph_layers as GL, ops
    torch.manual_seed(sum(dims) + 1)
    mes = bee.Messages(r0, *dims).cuda()
    g = torch.Generator().manual_seed(8)
    if box is None:
        pos = torch.cumsum(torch.randn(B, N, 3, generator=g) / 3 ** 0.5, dim=1)
    else:
        pos = torch.rand(B, N, 3, generator=g) * torch.tensor(box)
    da, dv, dd, _ = dims
    x_a, x_v, x_d = torch.randn(B, N, da, generator=g), torch.randn(B, N, dv, 3, generator=g), torch.randn(B, N, dd, 3, 3, generator=g)
    with torch.no_grad():
        graph = GL.Graph.radius_graph(r0, box, pos.cuda())
        ref = mes(graph, graph.rij, x_a.cuda(), x_v.cuda(), x_d.cuda())
        bee.set_precision(mes, "bf16")
        got = mes(graph, graph.rij, x_a.cuda(), x_v.cuda(), x_d.cuda())
        got2 = mes(graph, graph.rij, x_a.cuda(), x_v.cuda(), x_d.cuda())
    torch.cuda.synchronize()
    assert int(ops.tc_status("cuda").item()) == 0
    for a, b in zip(got, ref):
        close(a, b, 2e-2)
    for a, b in zip(got, got2):
        assert torch.equal(a, b)  # fixed summation order: run-to-run identical


def test_bee_denoiser_bf16_vs_fp32():
    """whole l<=2 denoiser with the scalar channel and the node-level channel mixings on tcgen05; the
    BF16 rounding of every layer compounds over depth, so the bar for the network output is 5e-2"""
    from ld_b200 import bee, ops
    torch.manual_seed(4)
    dims = (128, 64, 32, 128)
    dn = bee.BeeDenoiser(3.0, *dims, ntypes=5, depth=3).cuda()
    g = torch.Generator().manual_seed(10)
    x0 = torch.cumsum(torch.randn(4, 64, 3, generator=g) / 3 ** 0.5, dim=1).cuda()
    x1 = x0 + 0.3 * torch.randn(4, 64, 3, generator=g).cuda()
    types = torch.randint(0, 5, (64,), generator=g).cuda()
    with torch.no_grad():
        ref = dn(x0, x1, None, types)
        got = bee.set_precision(dn, "bf16")(x0, x1, None, types)
    assert int(ops.tc_status("cuda").item()) == 0
    close(got, ref, 5e-2)


@pytest.mark.parametrize("dims,rows", [((128, 64, 32, 128), (3, 50)), ((16, 8, 8, 32), (1, 7)), ((64, 32, 16, 96), (2, 33))])
def test_self_tens_prods_fused_vs_reference_sequence(dims, rows):
    """node-local products: three stacked channel mixings + one product kernel + three concatenated Y maps against
    the reference's op sequence (six linears, Bee, thirteen Y maps) on the unfused kernels and against the oracle"""
    from ld_b200 import bee
    from oracle import reference_math as R
    torch.manual_seed(sum(dims))
    mod = bee.SelfTensProds(*dims).cuda()
    g = torch.Generator().manual_seed(3)
    da, dv, dd, _ = dims
    x_a, x_v, x_d = (torch.randn(*rows, da, generator=g), torch.randn(*rows, dv, 3, generator=g),
                     torch.randn(*rows, dd, 3, 3, generator=g))
    ref_mod = R.OSelfTensProds(*dims)
    ref_mod.load_state_dict(mod.state_dict())
    with torch.no_grad():
        ref = ref_mod(x_a, x_v, x_d)
        fused = mod(x_a.cuda(), x_v.cuda(), x_d.cuda())
    unfused = mod(x_a.cuda(), x_v.cuda(), x_d.cuda())   # autograd enabled: the reference's op sequence
    for a, b, c in zip(fused, unfused, ref):
        close(a, b.detach(), 2e-5)
        close(a, c, 5e-5)
