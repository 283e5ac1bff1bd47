"""Channel mixing, tensor products, gather / segment sums on the GPU against the CPU oracle.
Tolerance: 1e-5 relative (FP32 path), measured as max|a-b| / max|b| and as the reference's
avg_relative_diff (managan/utils.py:45-52)."""
import pytest
import torch

from oracle import reference_math as R

pytestmark = pytest.mark.gpu
REL = 1e-5


def close(a, b, rel=REL):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape
    if b.numel() == 0:
        return
    err = (a - b).abs().max().item()
    scale = max(b.abs().max().item(), 1e-30)
    assert err <= rel * scale, f"max abs err {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("inds", [0, 1, 2])
@pytest.mark.parametrize("shape", [(10, 117, 210), (1, 1, 1), (257, 64, 64), (33, 128, 7)])
def test_tensor_linear_forward_backward(inds, shape):
    from ld_b200.ops import tensor_linear
    rows, din, dout = shape
    g = torch.Generator().manual_seed(inds * 7 + rows)
    W = torch.randn(dout, din, generator=g)
    x = torch.randn(rows, din, *([3] * inds), generator=g)
    dy = torch.randn(rows, dout, *([3] * inds), generator=g)
    Wr, xr = W.clone().requires_grad_(True), x.clone().requires_grad_(True)
    yr = R.tensor_linear(inds, Wr, xr)
    yr.backward(dy)
    Wg, xg = W.cuda().requires_grad_(True), x.cuda().requires_grad_(True)
    yg = tensor_linear(inds, Wg, xg)
    yg.backward(dy.cuda())
    close(yg, yr)
    close(xg.grad, xr.grad)
    close(Wg.grad, Wr.grad, rel=2e-5)


def test_tensor_linear_leading_dims_strided_weight_and_empty():
    from ld_b200.ops import tensor_linear
    g = torch.Generator().manual_seed(5)
    Wbig = torch.randn(40, 60, generator=g)
    W = Wbig[::2, ::3]  # strided view, as the reference allows for W
    x = torch.randn(4, 9, 20, 3, generator=g)
    close(tensor_linear(1, W.cuda(), x.cuda()), R.tensor_linear(1, W, x))
    y = tensor_linear(2, torch.randn(5, 6).cuda(), torch.zeros(0, 6, 3, 3).cuda())
    assert y.shape == (0, 5, 3, 3)
    with pytest.raises(RuntimeError, match="channel dim"):
        tensor_linear(0, torch.randn(5, 6).cuda(), torch.zeros(3, 7).cuda())
    with pytest.raises(RuntimeError, match="contiguous"):
        tensor_linear(0, torch.randn(5, 6).cuda(), torch.zeros(6, 3).cuda().t())


def test_tensor_linear_many_rows():
    from ld_b200.ops import tensor_linear
    g = torch.Generator().manual_seed(6)
    W = torch.randn(64, 128, generator=g)
    x = torch.randn(20000, 128, 3, generator=g)
    close(tensor_linear(1, W.cuda(), x.cuda()), R.tensor_linear(1, W, x))


@pytest.mark.parametrize("rows,chan", [(10, 256), (1, 1), (333, 40), (0, 8)])
def test_bee_forward_backward(rows, chan):
    from ld_b200.codegen_tensor_products import Bee
    g = torch.Generator().manual_seed(rows + chan)
    ops = [torch.randn(rows, chan, *([3] * l), generator=g) for l in (0, 1, 2, 0, 1, 2)]
    ref_in = [t.clone().requires_grad_(True) for t in ops]
    gpu_in = [t.cuda().requires_grad_(True) for t in ops]
    yr = R.bee(*ref_in)
    yg = Bee.apply(*gpu_in)
    assert len(yg) == 13
    gy = [torch.randn(y.shape, generator=g) for y in yr]
    for a, b in zip(yg, yr):
        close(a, b)
    if rows == 0:
        return
    sum((y * q).sum() for y, q in zip(yr, gy)).backward()
    sum((y * q.cuda()).sum() for y, q in zip(yg, gy)).backward()
    for a, b in zip(gpu_in, ref_in):
        close(a.grad, b.grad, rel=2e-5)


def test_cow_forward_backward():
    from ld_b200.codegen_tensor_products import Cow0, Cow1
    g = torch.Generator().manual_seed(3)
    ops = [torch.randn(10, 256, *([3] * l), generator=g) for l in (0, 1, 0, 1)]
    for fn_gpu, fn_ref in ((Cow0.apply, R.cow0), (Cow1.apply, R.cow1)):
        ref_in = [t.clone().requires_grad_(True) for t in ops]
        gpu_in = [t.cuda().requires_grad_(True) for t in ops]
        yr, yg = fn_ref(*ref_in), fn_gpu(*gpu_in)
        gy = [torch.randn(y.shape, generator=g) for y in yr]
        for a, b in zip(yg, yr):
            close(a, b)
        sum((y * q).sum() for y, q in zip(yr, gy)).backward()
        sum((y * q.cuda()).sum() for y, q in zip(yg, gy)).backward()
        for a, b in zip(gpu_in, ref_in):
            close(a.grad, b.grad, rel=2e-5)


def test_products_against_reference_golden(golden):
    from ld_b200 import ops
    b = golden["bee"]
    for mine, ref in zip(ops.bee_fwd(*[t.cuda() for t in b["operands"]]), b["outputs"]):
        close(mine, ref)
    c = golden["cow"]
    for mine, ref in zip(ops.cow_o0_fwd(*[t.cuda() for t in c["operands"]]), c["o0"]):
        close(mine, ref)
    for mine, ref in zip(ops.cow_o1_fwd(*[t.cuda() for t in c["operands"]]), c["o1"]):
        close(mine, ref)


def test_operand_checks():
    from ld_b200 import ops
    t = lambda *s: torch.zeros(*s, device="cuda")
    with pytest.raises(RuntimeError, match="l_1: expected axis 2 to have size 3"):
        ops.bee_fwd(t(2, 4), t(2, 4, 2), t(2, 4, 3, 3), t(2, 4), t(2, 4, 3), t(2, 4, 3, 3))
    with pytest.raises(RuntimeError, match="r_0: expected axis 1 to have size chan"):
        ops.bee_fwd(t(2, 4), t(2, 4, 3), t(2, 4, 3, 3), t(2, 5), t(2, 4, 3), t(2, 4, 3, 3))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.bee_fwd(torch.zeros(2, 4), t(2, 4, 3), t(2, 4, 3, 3), t(2, 4), t(2, 4, 3), t(2, 4, 3, 3))


@pytest.mark.parametrize("feat", [(), (1,), (7,), (64,), (16, 3), (8, 3, 3), (130,)])
def test_gather_and_segment_sum(feat):
    from ld_b200 import graph_layers as GL
    g = torch.Generator().manual_seed(len(feat) + 40)
    B, N = 3, 50
    pos = torch.rand(B, N, 3, generator=g) * 6
    o = R.radius_graph(pos, 2.0, (6.0, 6.0, 6.0))
    graph = GL.Graph(o["src"].cuda(), o["dst"].cuda(), None, B, N)
    x = torch.randn(B, N, *feat, generator=g)
    xs, xd = GL.edges_read(graph, x.cuda())
    flat = x.reshape(B * N, *feat)
    close(xs, flat[o["src"].long()], rel=0)
    close(xd, flat[o["dst"].long()], rel=0)
    xe = torch.randn(o["E"], *feat, generator=g)
    got = GL.edges_reduce_src(graph, xe.cuda())
    want = R.edges_reduce_src(o["src"], xe, B * N).reshape(B, N, *feat)
    close(got, want, rel=2e-6)


def test_segment_sum_autograd_and_drop_in_module():
    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "learned-dynamics_b200", "dropin"))
    import torch_scatter
    g = torch.Generator().manual_seed(8)
    idx = torch.sort(torch.randint(0, 20, (300,), generator=g)).values
    x = torch.randn(300, 6, generator=g)
    xr = x.clone().requires_grad_(True)
    out_r = torch.zeros(25, 6).index_add_(0, idx, xr)
    w = torch.randn(25, 6, generator=g)
    (out_r * w).sum().backward()
    xg = x.cuda().requires_grad_(True)
    out_g = torch_scatter.segment_coo(xg, idx.cuda(), dim_size=25)
    (out_g * w.cuda()).sum().backward()
    close(out_g, out_r, rel=2e-6)
    close(xg.grad, xr.grad, rel=0)


def test_drop_in_neighbour_grid_module():
    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "learned-dynamics_b200", "dropin"))
    import neighbour_grid_cuda as ng
    gen = torch.Generator().manual_seed(9)
    box = (30.5, 33.5, 36.5)
    x = (torch.rand(20, 60, 3, generator=gen) * torch.tensor(box)).cuda()
    # the checks of extensions/neighbour_grid/test.py:13-46
    neighbours, counts = ng.get_neighbours(32, 32, 7., *box, x)
    assert neighbours.dtype == torch.int32 and counts.dtype == torch.int32
    adj = torch.zeros(20, 60, 60, dtype=torch.int8)
    nb, ct = neighbours.cpu(), counts.cpu()
    for b in range(20):
        for n in range(60):
            for j in range(ct[b, n]):
                adj[b, n, nb[b, n, j]] = 1
    assert (adj == adj.permute(0, 2, 1)).all()
    indices = torch.arange(60, device="cuda")[None, :, None].expand(20, -1, -1).contiguous().float()
    read = ng.edges_read(counts, neighbours, indices)
    mask = torch.arange(32, device="cuda")[None, None, :] < counts[:, :, None]
    assert ((neighbours[..., None] - read).abs() * mask[..., None]).sum() < 1e-4
    ones = torch.ones(20, 60, 7, device="cuda")
    red = ng.edges_reduce(counts, neighbours, ng.edges_read(counts, neighbours, ones))
    assert (red[:, :, 0] - counts).abs().sum() < 1e-4
    # bit-exact against the loops of neighbour_grid_kern.cu:226-306 (zero past the count; slots added in ascending order)
    feat = torch.randn(20, 60, 37, generator=gen).cuda()
    read = ng.edges_read(counts, neighbours, feat)
    want = torch.gather(feat[:, None].expand(-1, 60, -1, -1), 2, neighbours.long()[..., None].expand(-1, -1, -1, 37)) * mask[..., None]
    assert torch.equal(read, want)
    table = torch.randn(20, 60, 32, 37, generator=gen).cuda()
    acc = torch.zeros(20, 60, 37, device="cuda")
    for j in range(32):
        acc = torch.where(mask[:, :, j, None], acc + table[:, :, j], acc)
    assert torch.equal(ng.edges_reduce(counts, neighbours, table), acc)
    with pytest.raises(RuntimeError, match="neighboursmax dimension"):
        ng.edges_reduce(counts, neighbours, table[:, :, :16].contiguous())
    assert ng.edges_read(counts[:0], neighbours[:0], feat[:0]).shape == (0, 60, 32, 37)
    src, dst, ec = ng.get_edges(32, 64, 7., *box, x)
    assert src.dtype == torch.int32 and ec.shape == (20,) and int(ec[-1]) == src.numel() == int(counts.sum())
    with pytest.raises(RuntimeError, match="listmax"):
        ng.get_edges(48, 64, 7., *box, x)
    with pytest.raises(RuntimeError, match="overflow"):
        ng.get_neighbours(32, 2, 7., *box, x)


def test_group_norms_fused_against_reference_golden(golden):
    """ScalGroupNorm / TensGroupNorm as the fused statistics + apply kernels (no autograd) against outputs of the
    reference's own classes, and against the torch formulation used under autograd"""
    from ld_b200.painn import ScalGroupNorm
    from ld_b200.tensor_products import TensGroupNorm
    n = golden["norms"]
    sgn = ScalGroupNorm(16, 4, epsilon=1.).cuda()
    sgn.load_state_dict(n["sgn_state"])
    tgn1, tgn2 = TensGroupNorm(1, 8, 4).cuda(), TensGroupNorm(2, 8, 2).cuda()
    x, xv, xd = n["x"].cuda(), n["xv"].cuda(), n["xd"].cuda()
    with torch.no_grad():
        close(sgn(x), n["sgn_out"], rel=2e-5)
        close(tgn1(xv), n["tgn1_out"], rel=2e-5)
        close(tgn2(xd), n["tgn2_out"], rel=2e-5)
        fused = [sgn(x), tgn1(xv), tgn2(xd)]
    for a, b in zip(fused, [sgn(x), tgn1(xv), tgn2(xd)]):   # autograd enabled: torch formulation
        close(a, b, rel=2e-5)


@pytest.mark.parametrize("shape,groups,inds", [((3, 257, 64), 4, 0), ((2, 100, 32, 3), 8, 1), ((5, 33, 16, 3, 3), 2, 2), ((1, 1, 8), 8, 0)])
def test_group_norm_shapes(shape, groups, inds):
    from ld_b200 import ops
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g) * 3 + (0.7 if inds == 0 else 0.0)
    C = shape[2]
    gamma, beta = torch.randn(C, generator=g), torch.randn(C, generator=g)
    B, N = shape[0], shape[1]
    xg = x.reshape(B, N, groups, C // groups, -1)
    if inds == 0:
        mean = xg.mean([1, 3, 4], keepdim=True)
        var = ((xg - mean) ** 2).mean([1, 3, 4], keepdim=True)
        ref = beta + gamma * ((xg - mean) / torch.sqrt(1e-3 + var)).reshape(shape)
        got = ops.group_norm(x.cuda(), groups, 1e-3, gamma.cuda(), beta.cuda(), center=True)
    else:
        m2 = (xg ** 2).sum(-1, keepdim=True).mean([1, 3], keepdim=True)
        ref = gamma.reshape(C, *[1] * inds) * (xg / torch.sqrt(1e-3 + m2)).reshape(shape)
        got = ops.group_norm(x.cuda(), groups, 1e-3, gamma.cuda(), None, center=False)
    close(got, ref, rel=2e-5)


def _golden_radial():
    import os
    return torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_golden_radial.pt"),
                      weights_only=False)


def test_older_radial_encodings_against_reference_golden():
    """radial_encode_edge (archs/diffuser_atoms5.py:25-30) and layers_common.radial_encode (:122-126) on the GPU against
    the outputs of the reference's own functions and against the oracle on a larger seeded input"""
    from ld_b200 import layers_common as LC
    from oracle import reference_math as R
    g = _golden_radial()
    with torch.no_grad():
        close(LC.radial_encode_edge(g["r_vec"].cuda(), 8, 4.0), g["edge_n8_rmax4"], 1e-5)
        close(LC.radial_encode_edge(g["r_vec"].cuda(), 16, 2.5), g["edge_n16_rmax2p5"], 1e-5)
        close(LC.radial_encode(g["r_len"].cuda(), 8, 1.0), g["cos_n8"], 1e-5)
        close(LC.radial_encode(g["r_len"].cuda(), 12, 3.0), g["cos_n12"], 1e-5)
        gen = torch.Generator().manual_seed(11)
        r = torch.randn(4, 1000, 3, generator=gen)
        close(LC.radial_encode_edge(r.cuda(), 12, 3.0), R.radial_encode_edge(r, 12, 3.0), 1e-5)
        d = torch.rand(7, 333, generator=gen)
        close(LC.radial_encode(d.cuda(), 10, 1.0), R.radial_encode_cos(d, 10, 1.0), 1e-5)
        assert LC.radial_encode_edge(torch.zeros(0, 3, device="cuda"), 8, 1.0).shape == (0, 8)
    # with autograd the torch formulation runs; same values
    rg = g["r_vec"].cuda().requires_grad_(True)
    close(LC.radial_encode_edge(rg, 8, 4.0), g["edge_n8_rmax4"], 1e-5)


def test_vec_linear_against_reference_golden():
    """VecLinear (managan/layers_common.py:81-89): the reference's state dict loads, forward and gradients match"""
    from ld_b200 import layers_common as LC
    from oracle import reference_math as R
    g = _golden_radial()
    vl = LC.VecLinear(24, 40)
    vl.load_state_dict(g["veclinear_state"])
    vl.cuda()
    with torch.no_grad():
        close(vl(g["veclinear_in"].cuda()), g["veclinear_out"], 1e-5)
    x = g["veclinear_in"].cuda().requires_grad_(True)
    y = vl(x)
    cot = torch.randn(y.shape, generator=torch.Generator().manual_seed(2))
    gx, gw = torch.autograd.grad(y, (x, vl.W), cot.cuda())
    xr = g["veclinear_in"].clone().requires_grad_(True)
    Wr = g["veclinear_state"]["W"].clone().requires_grad_(True)
    rx, rw = torch.autograd.grad(R.vec_linear(Wr, xr), (xr, Wr), cot)
    close(gx, rx, 1e-5)
    close(gw, rw, 1e-5)
