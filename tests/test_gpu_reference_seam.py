"""The drop-in seam with the reference's UNCHANGED Python: with `dropin/` on the module path in place of the reference's
built extensions (neighbour_grid_cuda, tensor_ops_cuda, codegen_tensops_cuda, torch_scatter), the reference's own
managan.graph_layers / tensor_products / codegen_tensor_products / jacobi_radenc and archs.meanflow_painn8 /
archs.diffuser_atoms15 are imported as they are and run on this library's kernels; results are compared with the
golden vectors the same classes produced on the CPU (tests/golden).

Needs a checkout of the reference: set LD_REFERENCE_DIR (skipped otherwise). Only the reference's empty
`managan/seq2pdbchain` submodule (protein tables that are not in its repository) is stubbed."""
import importlib
import os
import sys
import types

import pytest
import torch

pytestmark = pytest.mark.gpu

REF = os.environ.get("LD_REFERENCE_DIR", "")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def reference():
    if not os.path.isdir(os.path.join(REF, "managan")):
        pytest.skip("LD_REFERENCE_DIR is not a checkout of the reference repository")
    added = [os.path.join(ROOT, "learned-dynamics_b200", "dropin"), REF]
    for p in added:
        sys.path.insert(0, p)
    sys.dont_write_bytecode = True
    for name, attrs in (("managan.seq2pdbchain", {}), ("managan.seq2pdbchain.amino_data", {"letter_code": {}, "structures": {}}),
                        ("managan.seq2pdbchain.amino_bonds", {"bond_graphs": {}})):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules.setdefault(name, m)
    # the reference wraps one MLP in torch.compile; run it eagerly here (no tracing compiler on the hot path)
    real_compile = torch.compile
    torch.compile = lambda f=None, **k: f if f is not None else (lambda g: g)
    try:
        mods = {n: importlib.import_module(n) for n in ("managan.graph_layers", "managan.tensor_products",
                                                        "managan.codegen_tensor_products", "managan.jacobi_radenc",
                                                        "archs.meanflow_painn8", "archs.diffuser_atoms15")}
    finally:
        torch.compile = real_compile
    # the extension modules the reference imported are this repository's
    import neighbour_grid_cuda, tensor_ops_cuda, codegen_tensops_cuda, torch_scatter
    for m in (neighbour_grid_cuda, tensor_ops_cuda, codegen_tensops_cuda, torch_scatter):
        assert os.path.join("learned-dynamics_b200", "dropin") in m.__file__, m.__file__
    yield mods
    for p in added:
        sys.path.remove(p)


def _close(a, b, rel):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape
    err = (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)
    assert err <= rel, f"max-norm relative error {err:.2e} > {rel:.0e}"


def test_reference_graph_on_dropin(reference, golden):
    """Graph.radius_graph of the reference (get_edges of the drop-in underneath) on the reference's own 5-node table
    (managan/graph_layers.py:80-124)"""
    gl = reference["managan.graph_layers"]
    k = golden["graph_kat"]
    pos = k["positions"].cuda()
    graph = gl.Graph.radius_graph(k["r0"], k["box"], pos)
    assert torch.all(graph.src[1:] >= graph.src[:-1])
    ones = torch.ones(graph.src.shape[0], device="cuda")
    assert torch.allclose(gl.edges_reduce_src(graph, ones).cpu(), k["degrees"])
    x = torch.arange(5.).repeat(4).reshape(5, 4).cuda()[None]
    x_src, x_dst = gl.edges_read(graph, x)
    assert torch.allclose(gl.edges_reduce_src(graph, x_src * x_dst).cpu(), k["sumprod"])


def test_reference_painn_block_on_dropin(reference, golden):
    """the reference's Block (archs/meanflow_painn8.py:102-125) with its own Message / Update / TensLinear / edges_*
    code, extension calls served by the drop-in modules, against the golden output of the same class"""
    painn, gl = reference["archs.meanflow_painn8"], reference["managan.graph_layers"]
    p = golden["painn"]
    n, r0 = p["n"], p["r0"]
    B, N = p["x_a"].shape[:2]
    blk = painn.Block(r0, n)
    blk.load_state_dict(p["block_state"])
    blk.cuda()
    graph = gl.Graph(p["src"].cuda(), p["dst"].cuda(), None, B, N)
    graph_bond = gl.Graph(p["bond_src"].cuda(), p["bond_dst"].cuda(), None, B, N)
    with torch.no_grad():
        out = blk((p["pos"].cuda(), graph, p["r_ij"].cuda(), graph_bond, p["r_ij_bond"].cuda(), p["x_a"].cuda(), p["x_v"].cuda(),
                   (100., 100., 100.)))
    _close(out[5], p["block_out"][0], 3e-5)
    _close(out[6], p["block_out"][1], 3e-5)
    # and with autograd: the reference's op sequence differentiates through the drop-in's backward kernels
    x_a = p["x_a"].cuda().requires_grad_(True)
    out = blk((p["pos"].cuda(), graph, p["r_ij"].cuda(), graph_bond, p["r_ij_bond"].cuda(), x_a, p["x_v"].cuda(), (100., 100., 100.)))
    (out[5].sum() + out[6].sum()).backward()
    assert torch.isfinite(x_a.grad).all() and x_a.grad.abs().max() > 0


def test_reference_l2_messages_on_dropin(reference, golden):
    """the reference's Messages layer (archs/diffuser_atoms15.py:227-253: radial_encode_8, TensLinear, Bee, segment_coo)
    on the drop-in, against the golden output of the same class (which carries the reference's own float32 rounding of
    the radial power sum: 5e-4)"""
    atoms15, gl = reference["archs.diffuser_atoms15"], reference["managan.graph_layers"]
    p, m = golden["painn"], golden["bee_messages"]
    B, N = m["x_a"].shape[:2]
    real_compile = torch.compile      # the layer wraps its edge MLP in torch.compile when it is constructed: keep it eager
    torch.compile = lambda f=None, **k: f if f is not None else (lambda g: g)
    try:
        mes = atoms15.Messages(p["r0"], *m["dims"])
    finally:
        torch.compile = real_compile
    mes.load_state_dict(m["state"])
    mes.cuda()
    graph = gl.Graph(p["src"].cuda(), p["dst"].cuda(), None, B, N)
    with torch.no_grad():
        out = mes(graph, p["r_ij"].cuda(), m["x_a"].cuda(), m["x_v"].cuda(), m["x_d"].cuda())
    for got, want in zip(out, m["out"]):
        _close(got, want, 5e-4)
