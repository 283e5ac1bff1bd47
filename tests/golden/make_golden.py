"""Generates tests/golden/*.pt by running the REFERENCE's own Python classes on CPU.

Run where a checkout of the reference is available:
    python tests/golden/make_golden.py /path/to/learned-dynamics      (or set LD_REFERENCE_DIR)
The reference cannot be imported as-is without a GPU (its extension modules are CUDA-only and
some modules create CUDA tensors at import time), so this script
  * registers stub modules for tensor_ops_cuda (the reference's own einsum form), torch_scatter
    (index_add_), neighbour_grid_cuda (unused: graphs are passed in), codegen_tensops_cuda
    (bee/cow forward = the reference's einsum refimpls, lifted from the `__main__` block of
    managan/codegen_tensor_products.py by AST), and for the empty seq2pdbchain submodule;
  * redirects device="cuda" in torch factory functions to the CPU;
and then calls the unmodified reference classes. Nothing from the reference is copied into the
repository: only inputs, weights and outputs are stored."""
import ast
import importlib
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LD_REFERENCE_DIR", "")
if not os.path.isdir(os.path.join(REF, "managan")):
    sys.exit("usage: make_golden.py /path/to/learned-dynamics (a checkout of the reference repository)")
OUT = os.path.dirname(os.path.abspath(__file__))
sys.dont_write_bytecode = True
sys.path.insert(0, REF)


def stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


for fn in ["zeros", "ones", "tensor", "arange", "eye", "empty", "randn", "rand", "linspace", "full"]:
    orig = getattr(torch, fn)

    def mk(orig):
        def f(*a, **k):
            if str(k.get("device", "")).startswith("cuda"):
                k["device"] = "cpu"
            return orig(*a, **k)
        return f
    setattr(torch, fn, mk(orig))
torch.compile = lambda f=None, **k: f if f is not None else (lambda g: g)


def tensor_linear(inds, W, x):
    idx = "ijk"[:inds]
    return torch.einsum(f"OI, ...I{idx} -> ...O{idx}", W, x)


def segment_coo(x, index, dim_size=None):
    out = torch.zeros(dim_size, *x.shape[1:], dtype=x.dtype)
    return out.index_add_(0, index, x)


# reference einsum definitions of the products, lifted from the __main__ block
src_text = open(os.path.join(REF, "managan/codegen_tensor_products.py")).read()
tree = ast.parse(src_text)
refimpl_ns = {"torch": torch}
from itertools import permutations
lc = torch.zeros(3, 3, 3)
for i, j, k in permutations(range(3)):
    lc[i, j, k] = ((i - j) / abs(i - j)) * ((j - k) / abs(j - k)) * ((k - i) / abs(k - i))
refimpl_ns["lc_ijk"] = lc
for node in ast.walk(tree):
    if isinstance(node, ast.FunctionDef) and node.name.endswith("_refimpl"):
        exec(compile(ast.Module(body=[node], type_ignores=[]), "<reference refimpl>", "exec"), refimpl_ns)

stub("tensor_ops_cuda", tensor_linear=tensor_linear)
stub("neighbour_grid_cuda")
stub("torch_scatter", segment_coo=segment_coo)
cg = types.ModuleType("codegen_tensops_cuda")
_names = ["set_kern_attributes"] + [f"ant16_{o}{s}_cuda" for o in ("o0", "o1", "o2", "oc") for s in ("", "_backward", "_backleft", "_wtsback")] + \
    ["bee_fwd_cuda", "bee_bwl_cuda", "bee_bwr_cuda"] + [f"cow_{o}_{s}_cuda" for o in ("o0", "o1") for s in ("fwd", "bwl", "bwr")]
for n in _names:
    setattr(cg, n, lambda *a, **k: None)
cg.bee_fwd_cuda = lambda *a: list(refimpl_ns["bee_refimpl"](*a))
cg.cow_o0_fwd_cuda = lambda *a: list(refimpl_ns["cow0_refimpl"](*a))
cg.cow_o1_fwd_cuda = lambda *a: list(refimpl_ns["cow1_refimpl"](*a))
sys.modules["codegen_tensops_cuda"] = cg
import managan  # noqa: E402
stub("managan.seq2pdbchain")
stub("managan.seq2pdbchain.amino_data", letter_code={}, structures={})
stub("managan.seq2pdbchain.amino_bonds", bond_graphs={})

painn = importlib.import_module("archs.meanflow_painn8")
atoms15 = importlib.import_module("archs.diffuser_atoms15")
gl = importlib.import_module("managan.graph_layers")
tp = importlib.import_module("managan.tensor_products")
lcm = importlib.import_module("managan.layers_common")
jr = importlib.import_module("managan.jacobi_radenc")
cgtp = importlib.import_module("managan.codegen_tensor_products")


def brute_graph(pos, r0, box):
    """all pairs within r0 (minimum image if box), sorted by (src, dst); float64 distances"""
    B, N, _ = pos.shape
    srcs, dsts = [], []
    for b in range(B):
        d = pos[b][None, :, :].double() - pos[b][:, None, :].double()
        if box is not None:
            bx = torch.tensor(box, dtype=torch.float64)
            d = d - bx * torch.round(d / bx)
        adj = (d.pow(2).sum(-1) <= r0 * r0) & ~torch.eye(N, dtype=torch.bool)
        i, j = torch.nonzero(adj, as_tuple=True)
        srcs.append(i + b * N)
        dsts.append(j + b * N)
    return torch.cat(srcs), torch.cat(dsts)


def get_edges(listmax, neighboursmax, cutoff, bx, by, bz, x):
    """stand-in for the extension's get_edges on CPU: same outputs, membership by float64 brute force"""
    src, dst = brute_graph(x.detach(), cutoff, (bx, by, bz))
    counts = torch.bincount(src // x.shape[1], minlength=x.shape[0])
    return src.to(torch.int32), dst.to(torch.int32), torch.cumsum(counts, 0).to(torch.int32)


sys.modules["neighbour_grid_cuda"].get_edges = get_edges
NTYPES = 4


class TypeEmbed(torch.nn.Module):
    """plain type-embedding table in place of ResidueAtomEmbed (protein metadata is out of scope);
    `metadata` is the int64 type index per atom"""

    def __init__(self, dim):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.randn(NTYPES, dim))

    def forward(self, metadata):
        return self.weight[metadata]


def chain_bond_graph(batch, metadata, device):
    """get_bond_graph for a linear chain: bonds (i, i+1) both ways, sorted by src, replicated over the batch"""
    atoms = metadata.shape[0]
    i = torch.arange(atoms - 1)
    bs, bd = torch.cat([i, i + 1]), torch.cat([i + 1, i])
    order = torch.argsort(bs, stable=True)
    return gl.expand_graph(gl.Graph(bs[order], bd[order], None, 1, atoms), batch)


class NoOptim:
    def zero_grad(self):
        pass

    def step(self):
        pass


def meanflow_training_step(g):
    """the reference's own Meanflow._diffuser_step (archs/meanflow_painn8.py:283-301) on its own
    SE3ITO, with the optimiser replaced by a no-op so that the parameter gradients stay readable; the
    random draws are replayed from the same seed and stored"""
    painn.ResidueAtomEmbed, painn.get_bond_graph = TypeEmbed, chain_bond_graph
    r0, n, B, N, L, box, sigma_0 = 2.5, 16, 2, 10, 2, (30., 30., 30.), 0.3
    torch.manual_seed(23)
    dn = painn.SE3ITO(r0, n, N, 1, 2)
    with torch.no_grad():   # the reference initialises the table to zeros; make it count
        for emb in (dn.cpainn_0.atom_embed, dn.cpainn_1.atom_embed):
            emb.weight.copy_(torch.randn(NTYPES, n, generator=g))
    types = torch.randint(0, NTYPES, (N,), generator=g)
    x = 10. + torch.cumsum(torch.randn(L, B, N, 3, generator=g) / 3 ** 0.5, dim=2)
    x[1] = x[0] + 0.2 * torch.randn(B, N, 3, generator=g)
    me = types_ns(dn=dn, box=box, sigma_0=sigma_0, config={"loss_wt": "ph"}, optim=NoOptim())
    for name in ("_get_pos_and_vel", "_get_jvp"):
        setattr(me, name, getattr(painn.Meanflow, name).__get__(me))
    torch.manual_seed(29)
    loss = painn.Meanflow._diffuser_step(me, x, types)
    grads = {k: p.grad.clone() for k, p in dn.named_parameters() if p.grad is not None}
    torch.manual_seed(29)   # replay _diffuser_step's draws (:288-290)
    x_prev = x[:-1].reshape((L - 1) * B, N, 3)
    z_1 = x_prev + sigma_0 * torch.randn_like(x_prev)
    t = torch.rand((L - 1) * B)
    s = t * (1 - torch.relu(4 * torch.rand((L - 1) * B) - 3))
    return {"r0": r0, "n": n, "box": box, "sigma_0": sigma_0, "types": types, "x": x, "z_1": z_1, "t": t, "s": s,
            "blks": (1, 2), "state": dn.state_dict(), "loss": loss, "grads": grads}


def types_ns(**kw):
    return types.SimpleNamespace(**kw)


def main():
    g = torch.Generator().manual_seed(20240)
    gold = {}
    # --- radial encodings -----------------------------------------------------------------------
    r = torch.randn(40, 3, generator=g) * 1.5
    gold["radial"] = {"r": r, "painn_n16_r3": painn.radial_encode(r, 16, 3.0), "painn_n7_r5": painn.radial_encode(r, 7, 5.0),
                      "jacobi8_r4": jr.radial_encode_8(r, 4.0)}
    # --- norms / activations --------------------------------------------------------------------
    x = torch.randn(3, 10, 16, generator=g)
    sgn = lcm.ScalGroupNorm(16, 4, epsilon=1.)
    with torch.no_grad():
        sgn.gamma.copy_(torch.randn(16, generator=g)); sgn.beta.copy_(torch.randn(16, generator=g))
    xv = torch.randn(3, 10, 8, 3, generator=g)
    xd = torch.randn(3, 10, 8, 3, 3, generator=g)
    tgn1, tgn2 = tp.TensGroupNorm(1, 8, 4), tp.TensGroupNorm(2, 8, 2)
    gold["norms"] = {"x": x, "sgn_state": sgn.state_dict(), "sgn_out": sgn(x).detach(), "xv": xv, "xd": xd,
                     "tgn1_out": tgn1(xv).detach(), "tgn2_out": tgn2(xd).detach(),
                     "tens_sigmoid1": tp.tens_sigmoid(1, xv), "tens_sigmoid2": tp.tens_sigmoid(2, xd)}
    # --- products -------------------------------------------------------------------------------
    ops = [torch.randn(6, 5, *([3] * l), generator=g) for l in (0, 1, 2, 0, 1, 2)]
    gold["bee"] = {"operands": ops, "outputs": [t.clone() for t in refimpl_ns["bee_refimpl"](*ops)]}
    c_ops = [ops[0], ops[1], ops[3], ops[4]]
    gold["cow"] = {"operands": c_ops, "o0": list(refimpl_ns["cow0_refimpl"](*c_ops)), "o1": list(refimpl_ns["cow1_refimpl"](*c_ops))}
    # --- PaiNN Message / Update / Block (n=16, 3 open polymers of 12 beads, r0=3, large box as in
    #     the reference's own graph test) ----------------------------------------------------------
    n, B, N, r0 = 16, 3, 12, 3.0
    pos = torch.cumsum(torch.randn(B, N, 3, generator=g) / 3 ** 0.5, dim=1)
    box = (100., 100., 100.)
    src, dst = brute_graph(pos, r0, None)
    graph = gl.Graph(src, dst, None, B, N)
    tbox = torch.tensor(box)
    pos_src, pos_dst = gl.edges_read(graph, pos)
    r_ij = gl.boxwrap(tbox, pos_dst - pos_src)
    i = torch.arange(N - 1)
    bs = torch.cat([i, i + 1]); bd = torch.cat([i + 1, i])
    order = torch.argsort(bs, stable=True)
    bs, bd = bs[order], bd[order]
    graph_bond = gl.expand_graph(gl.Graph(bs, bd, None, 1, N), B)
    flat = pos.reshape(-1, 3)
    r_ij_bond = flat[graph_bond.dst] - flat[graph_bond.src]
    x_a = torch.randn(B, N, n, generator=g)
    x_v = torch.randn(B, N, n, 3, generator=g)
    torch.manual_seed(7)
    msg = painn.Message(r0, n)
    upd = painn.Update(n)
    blk = painn.Block(r0, n)
    with torch.no_grad():
        m_a, m_v = msg(graph, x_a, x_v, r_ij)
        u_a, u_v = upd(x_a, x_v)
        out = blk((pos, graph, r_ij, graph_bond, r_ij_bond, x_a, x_v, box))
    gold["painn"] = {"n": n, "r0": r0, "pos": pos, "src": src, "dst": dst, "r_ij": r_ij, "bond_src": graph_bond.src,
                     "bond_dst": graph_bond.dst, "r_ij_bond": r_ij_bond, "x_a": x_a, "x_v": x_v,
                     "message_state": msg.state_dict(), "message_out": (m_a, m_v),
                     "update_state": upd.state_dict(), "update_out": (u_a, u_v),
                     "block_state": blk.state_dict(), "block_out": (out[5], out[6])}
    # --- Bee-path Messages (archs/diffuser_atoms15.py:227-253), dims (a,v,d)=(16,8,8), chan 16 ----
    torch.manual_seed(11)
    mes = atoms15.Messages(r0, 16, 8, 8, 16)
    y_a = torch.randn(B, N, 16, generator=g); y_v = torch.randn(B, N, 8, 3, generator=g); y_d = torch.randn(B, N, 8, 3, 3, generator=g)
    with torch.no_grad():
        B_a, B_v, B_d = mes(graph, r_ij, y_a, y_v, y_d)
    gold["bee_messages"] = {"dims": (16, 8, 8, 16), "x_a": y_a, "x_v": y_v, "x_d": y_d, "state": mes.state_dict(),
                            "out": (B_a, B_v, B_d)}
    # --- Ant16 dense-weight products: the reference's einsum refimpl (managan/codegen_tensor_products.py:112-133)
    #     with autograd gradients for seeded cotangents; (P, left) pairs in Ant16.forward's argument order ----
    nb, d0, d1, d2, dl = 5, 8, 6, 4, 3
    sfx = {0: (), 1: (3,), 2: (3, 3)}
    dims = {0: d0, 1: d1, 2: d2}
    order = ["000", "110", "220", "011", "101", "121", "211", "111", "022", "202", "112", "222", "212"]
    a_in = [torch.randn(nb, dims[r], *sfx[r], generator=g, requires_grad=True) for r in (0, 1, 2)]
    for name in order:
        rl, rr, ro = int(name[0]), int(name[1]), int(name[2])
        a_in.append(torch.randn(dims[ro], dl, dims[rr], generator=g, requires_grad=True))
        a_in.append(torch.randn(nb, dl, *sfx[rl], generator=g, requires_grad=True))
    a_out = refimpl_ns["ant16_refimpl"](*a_in)
    cot = [torch.randn(t.shape, generator=g) for t in a_out]
    a_grads = torch.autograd.grad(sum((y * c).sum() for y, c in zip(a_out, cot)), a_in)
    gold["ant16"] = {"inputs": [t.detach() for t in a_in], "outputs": [t.detach() for t in a_out], "cotangents": cot,
                     "grads": list(a_grads)}
    # --- AVDFullTensorProds (managan/tensor_products.py:250-265), dims (8, 6, 4), rank 5 -----------------
    torch.manual_seed(13)
    avd = tp.AVDFullTensorProds(8, 6, 4, 5)
    z_a, z_v, z_d = (torch.randn(2, 7, dims[r], *sfx[r], generator=g) for r in (0, 1, 2))
    with torch.no_grad():
        avd_out = avd(z_a, z_v, z_d)
    gold["avd_tensor_prods"] = {"dims": (8, 6, 4, 5), "inputs": (z_a, z_v, z_d), "state": avd.state_dict(), "out": avd_out}
    # --- one meanflow training step: loss and parameter gradients (JVP + double backward) ------------
    gold["meanflow_step"] = meanflow_training_step(g)
    # --- dense proximity attention: the reference's own torch definitions with autograd gradients --------
    pa = importlib.import_module("managan.triton_kernels.proxattn")
    pap = importlib.import_module("managan.triton_kernels.proxattn_periodic")
    Zp, Np, dp = 6, 37, 16
    pa_in = [torch.randn(Zp, Np, dp, generator=g, requires_grad=True) for _ in range(3)] + \
            [(2 * torch.rand(Zp, Np, 3, generator=g)).requires_grad_(True) for _ in range(2)]
    pa_r0sq = torch.tensor([0.2, 0.5, 1.3])
    pa_box = (1.7, 2.1, 2.6)
    pa_cot = torch.randn(Zp, Np, dp, generator=g)
    pa_out = pa.refimpl_proxattn(*pa_in, pa_r0sq)
    pa_grads = torch.autograd.grad((pa_out * pa_cot).sum(), pa_in)
    pap_out = pap.refimpl_proxattn(*pa_in, pa_r0sq, torch.tensor(pa_box))
    pap_grads = torch.autograd.grad((pap_out * pa_cot).sum(), pa_in)
    gold["proxattn"] = {"inputs": [t.detach() for t in pa_in], "r0sq": pa_r0sq, "box": pa_box, "cotangent": pa_cot,
                        "out": pa_out.detach(), "grads": list(pa_grads), "out_periodic": pap_out.detach(),
                        "grads_periodic": list(pap_grads)}
    # --- trajectory file image written by the reference's own save_state_to_file --------------------
    sf = importlib.import_module("managan.statefiles")
    pred = importlib.import_module("managan.predictor")
    import io
    traj = torch.randn(3, 2, 5, 3, generator=g)
    buf = io.BytesIO()
    sf.save_state_to_file(buf, pred.ModelState((5, 3), traj, metadata={"seq": "AG", "note": 7}))
    gold["statefile"] = {"x": traj, "shape": (5, 3), "metadata": {"seq": "AG", "note": 7},
                         "image": np.frombuffer(buf.getvalue(), dtype=np.uint8).copy()}
    # --- the reference's own hand-computed graph test (managan/graph_layers.py:80-124) ------------
    gold["graph_kat"] = {
        "positions": torch.tensor([[[0., 0., -1.], [1., 0., 0.], [3., 0., 0.], [2., 1., 0.], [8., 0., 0.]]]),
        "r0": 2.0, "box": (100., 100., 100.), "degrees": torch.tensor([[1., 3., 2., 2., 0.]]),
        "sumprod": torch.tensor([[0., 0., 2., 6.], [20., 0., 6., 8.], [18., 12., 0., 2.], [14., 12., 4., 0.], [0., 0., 0., 0.]])[None]}
    torch.save(gold, os.path.join(OUT, "reference_golden.pt"))
    print("wrote", os.path.join(OUT, "reference_golden.pt"), os.path.getsize(os.path.join(OUT, "reference_golden.pt")), "bytes")


if __name__ == "__main__":
    main()
