"""The CPU oracle against vectors produced by the reference's own classes (tests/golden)."""
import torch

from oracle import reference_math as R

TOL = dict(rtol=1e-5, atol=1e-6)


def test_graph_known_answer(golden):
    k = golden["graph_kat"]
    g = R.radius_graph(k["positions"], k["r0"], k["box"])
    assert torch.all(g["src"][1:] >= g["src"][:-1])
    ones = torch.ones(g["E"])
    assert torch.allclose(R.edges_reduce_src(g["src"], ones, 5)[None], k["degrees"])
    x = torch.arange(5.).repeat(4).reshape(5, 4)
    sumprod = R.edges_reduce_src(g["src"], x[g["src"].long()] * x[g["dst"].long()], 5)[None]
    assert torch.allclose(sumprod, k["sumprod"])
    assert torch.all(g["rij"][0] ** 2 < 2.001 ** 2)


def test_radial_encodings(golden):
    r = golden["radial"]
    assert torch.allclose(R.radial_encode_painn(r["r"], 16, 3.0), r["painn_n16_r3"], **TOL)
    assert torch.allclose(R.radial_encode_painn(r["r"], 7, 5.0), r["painn_n7_r5"], **TOL)
    assert torch.allclose(R.radial_encode_8(r["r"], 4.0), r["jacobi8_r4"], rtol=1e-4, atol=1e-5)


def test_norms(golden):
    n = golden["norms"]
    sgn = R.OScalGroupNorm(16, 4, epsilon=1.)
    sgn.load_state_dict(n["sgn_state"])
    assert torch.allclose(sgn(n["x"]), n["sgn_out"], **TOL)
    assert torch.allclose(R.tens_sigmoid(1, n["xv"]), n["tens_sigmoid1"], **TOL)
    assert torch.allclose(R.tens_sigmoid(2, n["xd"]), n["tens_sigmoid2"], **TOL)


def test_products(golden):
    b = golden["bee"]
    for mine, ref in zip(R.bee(*b["operands"]), b["outputs"]):
        assert torch.allclose(mine, ref, **TOL)
    c = golden["cow"]
    for mine, ref in zip(R.cow0(*c["operands"]), c["o0"]):
        assert torch.allclose(mine, ref, **TOL)
    for mine, ref in zip(R.cow1(*c["operands"]), c["o1"]):
        assert torch.allclose(mine, ref, **TOL)


def test_painn_layers(golden):
    p = golden["painn"]
    n, r0 = p["n"], p["r0"]
    msg = R.OMessage(r0, n)
    msg.load_state_dict(p["message_state"])
    with torch.no_grad():
        a, v = msg(p["src"], p["dst"], p["x_a"], p["x_v"], p["r_ij"])
    assert torch.allclose(a, p["message_out"][0], rtol=1e-4, atol=1e-5)
    assert torch.allclose(v, p["message_out"][1], rtol=1e-4, atol=1e-5)
    upd = R.OUpdate(n)
    upd.load_state_dict(p["update_state"])
    with torch.no_grad():
        a, v = upd(p["x_a"], p["x_v"])
    assert torch.allclose(a, p["update_out"][0], rtol=1e-4, atol=1e-5)
    assert torch.allclose(v, p["update_out"][1], rtol=1e-4, atol=1e-5)
    blk = R.OBlock(r0, n)
    blk.load_state_dict(p["block_state"])
    with torch.no_grad():
        a, v = blk((p["src"], p["dst"], p["r_ij"]), (p["bond_src"], p["bond_dst"], p["r_ij_bond"]), p["x_a"], p["x_v"])
    assert torch.allclose(a, p["block_out"][0], rtol=1e-4, atol=1e-5)
    assert torch.allclose(v, p["block_out"][1], rtol=1e-4, atol=1e-5)


def test_oracle_graph_matches_golden_graph(golden):
    """the golden graph was built in float64 by the generator; same edge set expected here"""
    p = golden["painn"]
    g = R.radius_graph(p["pos"], p["r0"], None)
    assert torch.equal(g["src"].long(), p["src"]) and torch.equal(g["dst"].long(), p["dst"])
    assert torch.allclose(g["rij"], p["r_ij"], atol=1e-5)  # golden r_ij went through boxwrap with a 100-wide box


def test_periodic_graph_properties():
    gen = torch.Generator().manual_seed(3)
    box = (7.5, 8.0, 9.25)
    pos = torch.rand(2, 150, 3, generator=gen) * torch.tensor(box) * 3 - torch.tensor(box)  # also outside the box
    g = R.radius_graph(pos, 2.5, box)
    pairs = set(zip(g["src"].tolist(), g["dst"].tolist()))
    assert all((j, i) in pairs for (i, j) in pairs)
    # r_ij = x_j - x_i + shift*box, and |r_ij| <= cutoff up to rounding
    flat = pos.reshape(-1, 3)
    recon = flat[g["dst"].long()] - flat[g["src"].long()] + g["shift"].float() * torch.tensor(box)
    assert torch.allclose(recon, g["rij"], atol=2e-5)
    assert (g["rij"].norm(dim=1) <= 2.5 * (1 + 1e-5)).all()
    # reference-compatible mode never adds edges
    g1 = R.radius_graph(pos, 2.5, box, mode=1)
    pairs1 = set(zip(g1["src"].tolist(), g1["dst"].tolist()))
    assert pairs1 <= pairs


def test_bee_messages_layer(golden):
    p, m = golden["painn"], golden["bee_messages"]
    mes = R.OMessages(p["r0"], *m["dims"])
    mes.load_state_dict(m["state"])
    with torch.no_grad():
        out = mes(p["src"], p["dst"], p["r_ij"], m["x_a"], m["x_v"], m["x_d"])
    for mine, ref in zip(out, m["out"]):
        assert torch.allclose(mine, ref, rtol=1e-4, atol=1e-5)
    n = golden["norms"]
    for inds, key, x in ((1, "tgn1_out", n["xv"]), (2, "tgn2_out", n["xd"])):
        gn = R.OTensGroupNorm(inds, 8, 4 if inds == 1 else 2)
        assert torch.allclose(gn(x), n[key], rtol=1e-5, atol=1e-6)


def test_ant16_against_reference_einsums(golden):
    """outputs and all 29 gradients of the dense-weight products vs the reference's own einsum refimpl"""
    a = golden["ant16"]
    ins = [t.clone().requires_grad_(True) for t in a["inputs"]]
    outs = R.ant16(*ins)
    for mine, ref in zip(outs, a["outputs"]):
        assert torch.allclose(mine, ref, rtol=1e-5, atol=1e-5)
    grads = torch.autograd.grad(sum((y * c).sum() for y, c in zip(outs, a["cotangents"])), ins)
    for mine, ref in zip(grads, a["grads"]):
        assert torch.allclose(mine, ref, rtol=1e-5, atol=1e-5)


def test_avd_tensor_prods(golden):
    a = golden["avd_tensor_prods"]
    mod = R.OAVDFullTensorProds(*a["dims"])
    mod.load_state_dict(a["state"])
    with torch.no_grad():
        outs = mod(*a["inputs"])
    for mine, ref in zip(outs, a["out"]):
        assert torch.allclose(mine, ref, rtol=1e-5, atol=1e-5)


def test_meanflow_training_step(golden):
    """loss and every parameter gradient of one meanflow training step (Jacobian-vector product with
    create_graph, then backward) vs the reference's own Meanflow._diffuser_step on its own SE3ITO"""
    m = golden["meanflow_step"]
    L, B, N, _ = m["x"].shape
    dn = R.OSE3ITO(m["r0"], m["n"], N, 4, *m["blks"])
    dn.load_state_dict(m["state"])
    x_prev, z_0 = m["x"][:-1].reshape(-1, N, 3), m["x"][1:].reshape(-1, N, 3)
    bs, bd = R.chain_bonds(x_prev.shape[0], N)
    loss = R.meanflow_loss(dn, x_prev, z_0, m["z_1"], m["s"], m["t"], m["box"], m["types"], bs, bd)
    assert abs(loss.item() - m["loss"]) <= 1e-5 * abs(m["loss"])
    loss.backward()
    grads = {k: p.grad for k, p in dn.named_parameters() if p.grad is not None}
    assert set(grads) == set(m["grads"])
    for k, ref in m["grads"].items():
        scale = ref.abs().max().item()
        assert (grads[k] - ref).abs().max().item() <= 1e-4 * scale + 1e-9, k


def test_proximity_attention(golden):
    """open-space and periodic proximity attention with all five gradients vs the reference's refimpl"""
    p = golden["proxattn"]
    for box, ko, kg in ((None, "out", "grads"), (p["box"], "out_periodic", "grads_periodic")):
        ins = [t.clone().requires_grad_(True) for t in p["inputs"]]
        out = R.proxattn(*ins, p["r0sq"], box)
        assert torch.allclose(out, p[ko], rtol=1e-5, atol=1e-5)
        grads = torch.autograd.grad((out * p["cotangent"]).sum(), ins)
        for mine, ref in zip(grads, p[kg]):
            assert torch.allclose(mine, ref, rtol=1e-4, atol=1e-4)


def _golden_radial():
    import os
    return torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_golden_radial.pt"),
                      weights_only=False)


def test_older_radial_encodings_and_vec_linear():
    """radial_encode_edge (archs/diffuser_atoms5.py), radial_encode and VecLinear (managan/layers_common.py)"""
    g = _golden_radial()
    assert torch.allclose(R.radial_encode_edge(g["r_vec"], 8, 4.0), g["edge_n8_rmax4"], **TOL)
    assert torch.allclose(R.radial_encode_edge(g["r_vec"], 16, 2.5), g["edge_n16_rmax2p5"], **TOL)
    assert torch.allclose(R.radial_encode_cos(g["r_len"], 8, 1.0), g["cos_n8"], **TOL)
    assert torch.allclose(R.radial_encode_cos(g["r_len"], 12, 3.0), g["cos_n12"], **TOL)
    assert torch.allclose(R.vec_linear(g["veclinear_state"]["W"], g["veclinear_in"]), g["veclinear_out"], **TOL)


def test_reference_float32_rounding_of_the_polynomial_basis(golden):
    """The reference evaluates radial_encode_8 as a float32 power sum with coefficients up to 2.7e4; its stored output
    is therefore a few 1e-4 away from the exact value (basis functions are of size 1). The float64 oracle is the exact
    value; this pins it to the golden vector within the reference's own rounding, and shows that the float32 oracle
    (same formulation as the reference) carries an error of the same size."""
    r = golden["radial"]
    exact = R.radial_encode_8(r["r"].double(), 4.0)
    ref_err = (r["jacobi8_r4"].double() - exact).abs().max().item()
    f32_err = (R.radial_encode_8(r["r"], 4.0).double() - exact).abs().max().item()
    assert 1e-6 < ref_err < 5e-4 and f32_err < 5e-4
