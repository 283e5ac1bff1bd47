"""TEST INFRASTRUCTURE ONLY - the CPU oracle. Never imported by the product package.

PyTorch-CPU restatement of the reference's own formulation of the hot path, used by tests/,
__graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs as the checker and
the timed CPU baseline. Each function names the reference lines it follows (paths inside
pb1729/learned-dynamics). Pinning: tests/golden/ holds outputs of the reference's own Python
classes (imported on CPU with stub extension modules by tests/golden/make_golden.py) and
tests/test_oracle_golden.py checks this file against them; the radius graph is pinned by the
hand-computed table in managan/graph_layers.py:80-124.

Substitutions: torch_scatter.segment_coo -> index_add_; tensor_ops_cuda.tensor_linear -> the
einsum of managan/tensor_products.py:12-24; neighbour_grid_cuda -> brute force over all pairs
(oracle/radius_graph_oracle.c) with a fixed float32 predicate."""
import ctypes
import math
import os

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .build_oracle import build as _build_c

_clib = None


def _c():
    global _clib
    if _clib is None:
        L = ctypes.CDLL(_build_c())
        L.oracle_radius_graph.restype = ctypes.c_longlong
        L.oracle_radius_graph.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                          ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong] + [ctypes.c_void_p] * 5
        _clib = L
    return _clib


# ---- radius graph -----------------------------------------------------------------------------
def _radius_graph_block(pos, cutoff, box, mode):
    """one call of the C brute force on pos [B,N,3] (numpy float32); node ids are local to the block"""
    B, N, _ = pos.shape
    periodic = 0 if box is None else 1
    boxarr = np.asarray(box if box is not None else (0, 0, 0), dtype=np.float32)
    deg = np.zeros(B * N, dtype=np.int32)
    E = _c().oracle_radius_graph(pos.ctypes.data, B, N, periodic, ctypes.c_float(cutoff), boxarr.ctypes.data, mode, 0,
                                 None, None, None, None, deg.ctypes.data)
    src = np.zeros(E, dtype=np.int32); dst = np.zeros(E, dtype=np.int32)
    shift = np.zeros(E, dtype=np.int32); rij = np.zeros((E, 3), dtype=np.float32)
    _c().oracle_radius_graph(pos.ctypes.data, B, N, periodic, ctypes.c_float(cutoff), boxarr.ctypes.data, mode, E,
                             src.ctypes.data, dst.ctypes.data, shift.ctypes.data, rij.ctypes.data, deg.ctypes.data)
    return src, dst, shift, rij, deg


def radius_graph(pos, cutoff, box=None, mode=0):
    """pos [B,N,3] float32 (CPU). Returns dict(src, dst, shift[E,3], rij[E,3], degree[B*N]) with
    edges ordered by (system, i, j). Membership: neighbour_grid_kern.cu:39-48, 95-150; edge order
    neighbour_grid.cpp:180-194; rij is graph_setup's boxwrap (managan/graph_layers.py:62-66).
    Systems are independent, so large batches are handed to the C routine one system per host thread."""
    pos = np.ascontiguousarray(pos.detach().cpu().numpy(), dtype=np.float32)
    B, N, _ = pos.shape
    if B > 1 and B * N * N > (1 << 24):
        from concurrent.futures import ThreadPoolExecutor
        _c()
        with ThreadPoolExecutor(max_workers=len(os.sched_getaffinity(0))) as pool:
            parts = list(pool.map(lambda b: _radius_graph_block(pos[b:b + 1], cutoff, box, mode), range(B)))
        src = np.concatenate([p[0] + b * N for b, p in enumerate(parts)])
        dst = np.concatenate([p[1] + b * N for b, p in enumerate(parts)])
        shift, rij, deg = (np.concatenate([p[k] for p in parts]) for k in (2, 3, 4))
    else:
        src, dst, shift, rij, deg = _radius_graph_block(pos, cutoff, box, mode)
    E = src.shape[0]
    sh = np.stack([((shift >> (8 * a)) & 0xFF).astype(np.int32) for a in range(3)], axis=1)
    sh = np.where(sh >= 128, sh - 256, sh)
    return {"src": torch.from_numpy(src), "dst": torch.from_numpy(dst), "shift": torch.from_numpy(sh),
            "rij": torch.from_numpy(rij), "degree": torch.from_numpy(deg), "E": int(E)}


def boxwrap(box, delta_pos):
    """managan/graph_layers.py:62-66"""
    return (delta_pos + 0.5 * box) % box - 0.5 * box


def edges_reduce_src(src, x_edge, num_nodes):
    """managan/graph_layers.py:54-59 with index_add_ in place of segment_coo"""
    out = torch.zeros((num_nodes,) + tuple(x_edge.shape[1:]), dtype=x_edge.dtype)
    return out.index_add_(0, src.long(), x_edge)


# ---- channel mixing -----------------------------------------------------------------------------
def tensor_linear(inds, W, x):
    """managan/tensor_products.py:12-24 (einsum form); extensions/tensor_ops/test.py:8-15"""
    idx = "ijk"[:inds]
    return torch.einsum(f"OI, ...I{idx} -> ...O{idx}", W, x)


# ---- l<=2 products ------------------------------------------------------------------------------
def levi_civita():
    from itertools import permutations
    e = torch.zeros(3, 3, 3)
    for i, j, k in permutations(range(3)):
        e[i, j, k] = ((i - j) / abs(i - j)) * ((j - k) / abs(j - k)) * ((k - i) / abs(k - i))
    return e


def bee(l_0, l_1, l_2, r_0, r_1, r_2):
    """managan/codegen_tensor_products.py:235-249; output order of Bee.forward (:66-69)"""
    lc = levi_civita().to(l_0.dtype)
    y_000 = torch.einsum("bc, bc -> bc", l_0, r_0)
    y_110 = torch.einsum("bcx, bcx -> bc", l_1, r_1)
    y_220 = torch.einsum("bcxy, bcxy -> bc", l_2, r_2)
    y_011 = torch.einsum("bc, bcx -> bcx", l_0, r_1)
    y_101 = torch.einsum("bcx, bc -> bcx", l_1, r_0)
    y_121 = torch.einsum("bcx, bcyx -> bcy", l_1, r_2)
    y_211 = torch.einsum("bcxy, bcy -> bcx", l_2, r_1)
    y_111 = torch.einsum("bcx, bcy, xyz -> bcz", l_1, r_1, lc)
    y_022 = torch.einsum("bc, bcxy -> bcxy", l_0, r_2)
    y_202 = torch.einsum("bcxy, bc -> bcxy", l_2, r_0)
    y_112 = torch.einsum("bcx, bcy -> bcxy", l_1, r_1)
    y_222 = torch.einsum("bcxy, bczy -> bcxz", l_2, r_2)
    y_212 = torch.einsum("bcxy, bcz, yzw -> bcxw", l_2, r_1, lc)
    return y_000, y_110, y_220, y_011, y_101, y_121, y_211, y_022, y_202, y_112, y_222, y_111, y_212


def cow0(l_0, l_1, r_0, r_1):
    """managan/codegen_tensor_products.py:279-282"""
    return torch.einsum("bc, bc -> bc", l_0, r_0), torch.einsum("bcx, bcx -> bc", l_1, r_1)


def cow1(l_0, l_1, r_0, r_1):
    """managan/codegen_tensor_products.py:284-288"""
    lc = levi_civita().to(l_0.dtype)
    return (torch.einsum("bc, bcx -> bcx", l_0, r_1), torch.einsum("bcx, bc -> bcx", l_1, r_0),
            torch.einsum("bcx, bcy, xyz -> bcz", l_1, r_1, lc))


def ant16(x_0, x_1, x_2, *pl):
    """managan/codegen_tensor_products.py:112-133: the dense-weight products; pl = (P, left) pairs in the order
    000,110,220, 011,101,121,211,111, 022,202,112,222,212 (Ant16.forward's argument order, :22-25)."""
    lc = levi_civita().to(x_0.dtype)
    (P_000, l_000, P_110, l_110, P_220, l_220, P_011, l_011, P_101, l_101, P_121, l_121, P_211, l_211, P_111, l_111,
     P_022, l_022, P_202, l_202, P_112, l_112, P_222, l_222, P_212, l_212) = pl
    y_0 = (torch.einsum("bl, br, olr -> bo", l_000, x_0, P_000) + torch.einsum("blx, brx, olr -> bo", l_110, x_1, P_110)
           + torch.einsum("blxy, brxy, olr -> bo", l_220, x_2, P_220))
    y_1 = (torch.einsum("bl, brx, olr -> box", l_011, x_1, P_011) + torch.einsum("blx, br, olr -> box", l_101, x_0, P_101)
           + torch.einsum("blx, bryx, olr -> boy", l_121, x_2, P_121) + torch.einsum("blxy, bry, olr -> box", l_211, x_1, P_211)
           + torch.einsum("blx, bry, olr, xyz -> boz", l_111, x_1, P_111, lc))
    y_2 = (torch.einsum("bl, brxy, olr -> boxy", l_022, x_2, P_022) + torch.einsum("blxy, br, olr -> boxy", l_202, x_0, P_202)
           + torch.einsum("blx, bry, olr -> boxy", l_112, x_1, P_112) + torch.einsum("blxy, brzy, olr -> boxz", l_222, x_2, P_222)
           + torch.einsum("blxy, brz, olr, yzw -> boxw", l_212, x_1, P_212, lc))
    return y_0, y_1, y_2


def tensor_prod_bare(inds_l, inds_r, inds_o, x_l, x_r):
    """managan/tensor_products.py:91-108: contract the trailing (inds_l + inds_r - inds_o) / 2 indices"""
    contracts = (inds_l + inds_r - inds_o) // 2
    letters = "ijklmn"[:inds_l + inds_r - contracts]
    c, keep_l, keep_r = letters[:contracts], letters[contracts:inds_l], letters[inds_l:]
    return torch.einsum(f"...{keep_l + c}, ...{keep_r + c} -> ...{keep_l + keep_r}", x_l, x_r)


class OTensorProds(nn.Module):
    """managan/tensor_products.py:111-123"""

    def __init__(self, inds_l, inds_r, inds_o, dim_l, dim_r, dim_o, rank):
        super().__init__()
        self.ranks = (inds_l, inds_r, inds_o)
        self.lin_l, self.lin_r, self.lin_o = OTensLinear(inds_l, dim_l, rank), OTensLinear(inds_r, dim_r, rank), OTensLinear(inds_o, rank, dim_o)

    def forward(self, x_l, x_r):
        return self.lin_o(tensor_prod_bare(*self.ranks, self.lin_l(x_l), self.lin_r(x_r)))


class OAVDFullTensorProds(nn.Module):
    """managan/tensor_products.py:250-265"""

    def __init__(self, dim_a, dim_v, dim_d, rank):
        super().__init__()
        dims = {0: dim_a, 1: dim_v, 2: dim_d}
        for code in ("000", "101", "110", "112", "202", "211", "220", "222"):
            l, r, o = (int(ch) for ch in code)
            setattr(self, "tp" + code, OTensorProds(l, r, o, dims[l], dims[r], dims[o], rank))

    def forward(self, x_a, x_v, x_d):
        y_a = self.tp000(x_a, x_a) + self.tp110(x_v, x_v) + self.tp220(x_d, x_d)
        y_v = self.tp101(x_v, x_a) + self.tp211(x_d, x_v)
        y_d = self.tp112(x_v, x_v) + self.tp202(x_d, x_a) + self.tp222(x_d, x_d)
        return y_a, y_v, y_d


# ---- radial encodings ---------------------------------------------------------------------------
def radial_encode_painn(r, n, rmax):
    """archs/meanflow_painn8.py:25-35"""
    hn = (n + 1) // 2
    coeffs = (torch.pi / rmax) * (1 + torch.arange(0, hn) // 2)
    dist = torch.linalg.vector_norm(r, dim=-1)[..., None]
    phase = coeffs * dist
    return torch.cat([torch.cos(phase), torch.sin(phase[..., :(n - hn)])], dim=-1)


def radial_encode_gaussian(r, n, rmax):
    """Gaussian basis with cosine cutoff asked for by the benchmark configs; not in the reference.
    centres m*rmax/(n-1), width rmax/(n-1), envelope 0.5(cos(pi d/rmax)+1) for d < rmax."""
    d = torch.linalg.vector_norm(r, dim=-1)[..., None]
    width = rmax / (n - 1) if n > 1 else rmax
    mu = torch.arange(n, dtype=r.dtype) * width
    env = torch.where(d < rmax, 0.5 * (torch.cos(math.pi * d / rmax) + 1.0), torch.zeros_like(d))
    return torch.exp(-0.5 * ((d - mu) / width) ** 2) * env


def radial_encode_edge(r, n, rmax):
    """archs/diffuser_atoms5.py:25-30"""
    npi = torch.pi * torch.arange(0, n)
    x_sq = (r ** 2).sum(-1) / rmax
    return torch.cos(npi * torch.sqrt(x_sq)[..., None]) * torch.relu(1. - x_sq)[..., None]


def radial_encode_cos(r, n, rmax):
    """managan/layers_common.py:122-126 (radial_encode there; rmax is unused)"""
    return torch.cos(torch.pi * torch.arange(0, n) * r[..., None])


def vec_linear(W, v):
    """managan/layers_common.py:81-89 (VecLinear.forward)"""
    return torch.einsum("oi, ...ik -> ...ok", W, v)


def jacobi_matrix(dim):
    """managan/jacobi_radenc.py:8-24: coefficients of shifted Jacobi(1,0) polynomials on [0,1]"""
    import sympy as sp
    from sympy import jacobi, Poly
    x = sp.symbols("x")
    A = torch.zeros(dim, 1 + dim)
    for i in range(dim):
        coeffs = Poly(jacobi(i, 1, 0, (2 * x - 1)), x, domain="R").all_coeffs()[::-1]
        for j in range(len(coeffs)):
            A[i, j] = float(coeffs[j])
    return A


_A8 = None


def radial_encode_8(r, rmax):
    """managan/jacobi_radenc.py:27-37"""
    global _A8
    if _A8 is None:
        _A8 = jacobi_matrix(8)
    z = (torch.linalg.vector_norm(r, dim=-1) / rmax)[..., None]
    pows = z ** torch.arange(_A8.shape[1])
    return F.linear(pows, _A8.to(r.dtype)) * torch.relu(1. - z)   # float64 inputs give the float64 oracle


def tens_sigmoid(inds, x):
    """managan/tensor_products.py:167-182"""
    dims = tuple(-(1 + n) for n in range(inds))
    xx = (x ** 2).sum(dims, keepdim=True)
    return x / torch.sqrt(1. + xx)


# ---- PaiNN layers (parameter names as in the reference so state dicts transfer) --------------------
class OTensLinear(nn.Module):
    def __init__(self, inds, dim_in, dim_out):
        super().__init__()
        self.W = nn.Parameter(torch.empty(dim_out, dim_in))
        self.inds = inds
        nn.init.normal_(self.W, std=dim_in ** -0.5)

    def forward(self, x):
        return tensor_linear(self.inds, self.W, x)


class OMLP(nn.Module):
    """archs/meanflow_painn8.py:38-51"""

    def __init__(self, dim_in, dim_out):
        super().__init__()
        self.layers = nn.Sequential(nn.Linear(dim_in, dim_out), nn.SiLU(), nn.Linear(dim_out, dim_out), nn.SiLU(),
                                    nn.Linear(dim_out, dim_out))

    def forward(self, x):
        return self.layers(x)


class OScalGroupNorm(nn.Module):
    """managan/layers_common.py:201-223"""

    def __init__(self, chan, groups, epsilon=1e-5):
        super().__init__()
        self.chan, self.groups, self.epsilon = chan, groups, epsilon
        self.gamma = nn.Parameter(torch.ones(chan))
        self.beta = nn.Parameter(torch.zeros(chan))

    def forward(self, x):
        batch, nodes, _ = x.shape
        x = x.reshape(batch, nodes, self.groups, -1)
        mean = x.mean([1, 3], keepdim=True)
        x_shift = x - mean
        var = (x_shift ** 2).mean([1, 3], keepdim=True)
        ans = x_shift / torch.sqrt(self.epsilon + var)
        return self.beta + self.gamma * ans.reshape(batch, nodes, self.chan)


class OUpdate(nn.Module):
    """archs/meanflow_painn8.py:53-75"""

    def __init__(self, n):
        super().__init__()
        self.n = n
        self.lin_l = OTensLinear(1, n, n)
        self.lin_r = OTensLinear(1, n, n)
        self.lin_v = OTensLinear(1, n, n)
        self.mlp = OMLP(2 * n, 3 * n)
        self.gn = OScalGroupNorm(n, 4, epsilon=1.)

    def forward(self, x_a, x_v):
        x_v_l = self.lin_l(x_v)
        x_v_r = self.lin_r(x_v)
        inner_prod = (x_v_l * x_v_r).sum(-1)
        y = self.mlp(torch.cat([x_a, torch.linalg.vector_norm(x_v_r, dim=-1)], dim=-1))
        x_v = self.lin_v(x_v)
        x_v = x_v * y[..., :self.n, None]
        inner_prod = self.gn(inner_prod * y[..., self.n:2 * self.n])
        x_a = inner_prod + y[..., 2 * self.n:]
        x_v = x_v / torch.sqrt(1. + (x_v ** 2).sum(-1, keepdim=True))
        return x_a, x_v


class OMessage(nn.Module):
    """archs/meanflow_painn8.py:77-100. radial: 'painn' (reference) or 'gaussian' (benchmark spec)."""

    def __init__(self, r0, n, n_rbf=None, radial="painn"):
        super().__init__()
        self.r0, self.n, self.epsilon, self.radial = r0, n, 0.1, radial
        self.n_rbf = n if n_rbf is None else n_rbf
        self.mlp_dist = OMLP(self.n_rbf, 4 * n)
        self.mlp_actv = OMLP(n, 4 * n)

    def forward(self, src, dst, x_a, x_v, r_ij):
        batch, atoms, n = x_a.shape
        Nt = batch * atoms
        enc = radial_encode_painn(r_ij, self.n_rbf, self.r0) if self.radial == "painn" else radial_encode_gaussian(r_ij, self.n_rbf, self.r0)
        dist_x_a = self.mlp_dist(enc)
        actv_x_a = self.mlp_actv(x_a.reshape(Nt, n)[dst.long()])
        prod_x_a = dist_x_a * actv_x_a
        direction = r_ij / torch.sqrt(self.epsilon + (r_ij ** 2).sum(-1, keepdim=True))
        x_v = x_v.reshape(Nt, n, 3)[dst.long()]
        cross = torch.linalg.cross(x_v, direction[:, None].expand_as(x_v))
        x_v = x_v * prod_x_a[..., :n, None]
        x_v = x_v + cross * prod_x_a[..., n:2 * n, None]
        x_v = x_v + direction[:, None] * prod_x_a[..., 2 * n:3 * n, None]
        x_v = edges_reduce_src(src, x_v, Nt).reshape(batch, atoms, n, 3)
        x_a = edges_reduce_src(src, prod_x_a[..., 3 * n:], Nt).reshape(batch, atoms, n)
        return x_a, x_v


class OBlock(nn.Module):
    """archs/meanflow_painn8.py:102-125 (pos_mutable=False)"""

    def __init__(self, r0, n, n_rbf=None, radial="painn"):
        super().__init__()
        self.r0 = r0
        self.message = OMessage(r0, n, n_rbf, radial)
        self.message_bond = OMessage(r0, n, n_rbf, radial)
        self.update = OUpdate(n)

    def forward(self, graph, graph_bond, x_a, x_v):
        """graph, graph_bond: (src, dst, r_ij)"""
        dx_a, dx_v = self.message_bond(graph_bond[0], graph_bond[1], x_a, x_v, graph_bond[2])
        x_a, x_v = x_a + dx_a, x_v + dx_v
        dx_a, dx_v = self.message(graph[0], graph[1], x_a, x_v, graph[2])
        x_a, x_v = x_a + dx_a, x_v + dx_v
        dx_a, dx_v = self.update(x_a, x_v)
        return x_a + dx_a, x_v + dx_v


class OCPaiNN(nn.Module):
    """archs/meanflow_painn8.py:128-143 with a type-embedding table for ResidueAtomEmbed"""

    def __init__(self, r0, n, blks, ntypes, n_rbf=None, radial="painn"):
        super().__init__()
        self.r0 = r0
        self.atom_embed = nn.Embedding(ntypes, n)
        self.blocks = nn.Sequential(*[OBlock(r0, n, n_rbf, radial) for _ in range(blks)])

    def forward(self, pos, graph_bond, x_a, x_v, box, types):
        x_a = x_a + self.atom_embed(types)[None]
        g = radius_graph(pos, self.r0, box)
        rij = g["rij"]
        if torch.is_grad_enabled() and pos.requires_grad:  # graph_setup's differentiable form (:167-172)
            flat = pos.reshape(-1, 3)
            rij = flat[g["dst"].long()] - flat[g["src"].long()]
            if box is not None:
                rij = boxwrap(torch.as_tensor(box, dtype=pos.dtype), rij)
        graph = (g["src"], g["dst"], rij)
        for blk in self.blocks:
            x_a, x_v = blk(graph, graph_bond, x_a, x_v)
        return x_a, x_v, g["E"]


class OTimeEmbedding(nn.Module):
    """archs/meanflow_painn8.py:145-165"""

    def __init__(self, freqs, outdim):
        super().__init__()
        self.freqs = freqs
        self.lin1 = nn.Linear(4 * freqs, outdim)

    def forward(self, st):
        s, t = st
        ang = torch.exp(-torch.arange(self.freqs) / (self.freqs - 1))
        phases = torch.cat([t[:, None] * ang[None, :], (t - s)[:, None] * ang[None, :]], dim=1)
        return self.lin1(torch.cat([torch.sin(phases), torch.cos(phases)], dim=1))


class OPosEmbed(nn.Module):
    """archs/meanflow_painn8.py:174-183"""

    def __init__(self, dim_v):
        super().__init__()
        self.lin_v = OTensLinear(1, 1, dim_v)

    def forward(self, pos_0, pos_1):
        return self.lin_v(0.1 * (pos_1[:, :, None] - pos_0[:, :, None]))


class OSE3ITO(nn.Module):
    """archs/meanflow_painn8.py:185-217; bond graph supplied as (src, dst) of a batch-1 template
    replicated over the batch as get_bond_graph does (managan/flavour_layers.py:256-272)."""

    def __init__(self, r0, n, natoms, ntypes=1, blks_0=2, blks_1=5, n_rbf=None, radial="painn"):
        super().__init__()
        self.r0 = r0
        self.atom_embeddings = nn.Parameter(torch.randn(natoms, n))
        self.t_embed = OTimeEmbedding(32, n)
        self.mlp_embed = OMLP(n, n)
        self.mlp_denoise = OMLP(n, n)
        self.pos_emb = OPosEmbed(n)
        self.cpainn_0 = OCPaiNN(r0, n, blks_0, ntypes, n_rbf, radial)
        self.cpainn_1 = OCPaiNN(r0, n, blks_1, ntypes, n_rbf, radial)
        self.v_readin = OTensLinear(1, 1, n)
        self.readout = OTensLinear(1, n, 1)
        self.edges_last = 0

    def forward(self, st, x0, x1, box, types, bond_src, bond_dst):
        s, t = st
        x1_t = x1
        r0b = x0.reshape(-1, 3)[bond_dst.long()] - x0.reshape(-1, 3)[bond_src.long()]
        r1b = x1.reshape(-1, 3)[bond_dst.long()] - x1.reshape(-1, 3)[bond_src.long()]
        x_a = self.atom_embeddings[None].expand(x0.shape[0], -1, -1)
        x_v = self.v_readin((x1 - x0)[..., None, :])
        x_a = self.mlp_embed(x_a)
        x_a, x_v, e0 = self.cpainn_0(x0, (bond_src, bond_dst, r0b), x_a, x_v, box, types)
        x_a = self.mlp_denoise(x_a + self.t_embed(st)[:, None])
        x_v = x_v + self.pos_emb(x0, x1)
        x_a, x_v, e1 = self.cpainn_1(x1, (bond_src, bond_dst, r1b), x_a, x_v, box, types)
        nb = bond_src.numel()
        self.edges_last = (e0 + nb) * len(self.cpainn_0.blocks) + (e1 + nb) * len(self.cpainn_1.blocks)
        v_pred = self.readout(x_v).squeeze(-2)
        return (1. - (t - s)[:, None, None]) * v_pred + x1_t - x1


def meanflow_generate(dn, x_0, noise, sigma_0, box, types, bond_src, bond_dst):
    """archs/meanflow_painn8.py:302-310 with the noise passed in"""
    batch = x_0.shape[0]
    z_1 = x_0 + sigma_0 * noise
    st = (torch.zeros(batch), torch.ones(batch))
    with torch.no_grad():
        v_pred = dn(st, x_0, z_1, box, types, bond_src, bond_dst)
    return z_1 - v_pred


def meanflow_loss(dn, x_prev, z_0, z_1, s, t, box, types, bond_src, bond_dst, loss_wt="ph"):
    """archs/meanflow_painn8.py:269-297 (_get_pos_and_vel, _get_jvp, _diffuser_step) with the random
    draws passed in and without the optimiser step"""
    tt = t[:, None, None]
    z_t, v = tt * z_1 + (1 - tt) * z_0, z_1 - z_0
    f = lambda z, tau: dn((s, tau), x_prev, z, box, types, bond_src, bond_dst)  # noqa: E731
    _, jvp = torch.autograd.functional.jvp(f, (z_t, t), (v, torch.ones_like(t)), create_graph=True)
    v_target = v - (t - s)[:, None, None] * jvp
    v_pred = f(z_t, t)
    d_sq = ((v_pred - v_target) ** 2).mean((1, 2))
    if loss_wt == "ph":
        d_sq = d_sq / (0.5 + d_sq.detach()) ** 0.7
    return d_sq.mean()


def proxattn(Q, K, V, X, Y, r0sq, box=None):
    """refimpl_proxattn of managan/triton_kernels/proxattn.py:9-27 (box=None) and of
    managan/triton_kernels/proxattn_periodic.py:9-28 (box = 3 lengths)"""
    Z = Q.shape[0]
    heads = r0sq.shape[0]
    assert Z % heads == 0
    r0 = r0sq[None].expand(Z // heads, -1).reshape(Z)[:, None, None]
    QK = torch.einsum("zmd, znd -> zmn", Q, K)
    R = X[:, :, None] - Y[:, None, :]
    if box is None:
        dist2 = (R ** 2).sum(-1)
    else:
        box = torch.as_tensor(box, dtype=Q.dtype)
        dist2 = ((1. - torch.cos(2 * torch.pi * R / box)) * box ** 2 / (2 * torch.pi * torch.pi)).sum(-1)
    return torch.einsum("zmn, znd -> zmd", r0 * QK / (r0 + dist2), V)


def chain_bonds(batch, nodes):
    i = torch.arange(nodes - 1)
    src = torch.cat([i, i + 1]); dst = torch.cat([i + 1, i])
    order = torch.argsort(src, stable=True)
    src, dst = src[order], dst[order]
    offs = nodes * torch.arange(batch)[:, None]
    return (src[None] + offs).reshape(-1), (dst[None] + offs).reshape(-1)


def avg_relative_diff(a, b):
    """managan/utils.py:45-52, the reference's comparison metric"""
    return (torch.abs(a - b) / torch.sqrt(0.0001 + 0.5 * (a ** 2 + b ** 2))).mean().item()


# ---- l<=2 ("Bee"-path) layers -------------------------------------------------------------------
V_ORDER = ("011", "101", "121", "211", "111")
D_ORDER = ("022", "202", "112", "222", "212")


def _add_y_maps(mod, dim_a, dim_v, dim_d, chan):
    """archs/diffuser_atoms15.py:29-42"""
    for name in ("000", "110", "220"):
        setattr(mod, "Y_" + name, OTensLinear(0, chan, dim_a))
    for name in V_ORDER:
        setattr(mod, "Y_" + name, OTensLinear(1, chan, dim_v))
    for name in D_ORDER:
        setattr(mod, "Y_" + name, OTensLinear(2, chan, dim_d))


def _apply_y_maps(mod, prods):
    """archs/diffuser_atoms15.py:52-57"""
    y_000, y_110, y_220, y_011, y_101, y_121, y_211, y_022, y_202, y_112, y_222, y_111, y_212 = prods
    y_0 = mod.Y_000(y_000) + mod.Y_110(y_110) + mod.Y_220(y_220)
    y_1 = mod.Y_011(y_011) + mod.Y_101(y_101) + mod.Y_121(y_121) + mod.Y_211(y_211) + mod.Y_111(y_111)
    y_2 = mod.Y_022(y_022) + mod.Y_202(y_202) + mod.Y_112(y_112) + mod.Y_222(y_222) + mod.Y_212(y_212)
    return y_0, y_1, y_2


class OBeeMLP(nn.Module):
    """archs/diffuser_atoms15.py:98-110"""

    def __init__(self, dim_a):
        super().__init__()
        self.lin_direct = nn.Linear(dim_a, dim_a, bias=False)
        self.layers = nn.Sequential(nn.Linear(dim_a, 2 * dim_a), nn.LeakyReLU(0.1), nn.Linear(2 * dim_a, 2 * dim_a),
                                    nn.LeakyReLU(0.1), nn.Linear(2 * dim_a, dim_a))

    def forward(self, x):
        return self.lin_direct(x) + self.layers(x)


class OTensGroupNorm(nn.Module):
    """managan/tensor_products.py:215-232"""

    def __init__(self, inds, chan, groups, epsilon=1e-5):
        super().__init__()
        self.inds, self.chan, self.groups, self.epsilon = inds, chan, groups, epsilon
        self.gamma = nn.Parameter(torch.ones(chan, *[1] * inds))

    def forward(self, x):
        batch, nodes = x.shape[0], x.shape[1]
        xg = x.reshape(batch, nodes, self.groups, -1, 3 ** self.inds)
        moment2 = (xg ** 2).sum(-1, keepdim=True).mean([1, 3], keepdim=True)
        ans = xg / torch.sqrt(self.epsilon + moment2)
        return self.gamma * ans.reshape(batch, nodes, self.chan, *[3] * self.inds)


class OMessages(nn.Module):
    """archs/diffuser_atoms15.py:227-253"""

    def __init__(self, r0, dim_a, dim_v, dim_d, chan):
        super().__init__()
        self.r0 = r0
        self.L0, self.L1, self.L2 = OTensLinear(0, dim_a, chan), OTensLinear(1, dim_v, chan), OTensLinear(2, dim_d, chan)
        _add_y_maps(self, dim_a, dim_v, dim_d, chan)
        self.lin_enc = nn.Linear(8, chan)
        self.mlp_a = OBeeMLP(dim_a)

    def forward(self, src, dst, r_ij, x_a, x_v, x_d):
        batch, nodes = x_a.shape[:2]
        Nt = batch * nodes
        rad = self.lin_enc(radial_encode_8(r_ij, self.r0))
        r = tens_sigmoid(1, r_ij * (7. / self.r0))
        phi_a = rad
        phi_v = rad[..., None] * r[..., None, :]
        phi_d = rad[..., None, None] * r[..., None, None, :] * r[..., None, :, None]
        j = dst.long()
        x_a_j = self.L0(x_a).reshape(Nt, -1)[j]
        x_v_j = self.L1(x_v).reshape(Nt, -1, 3)[j]
        x_d_j = self.L2(x_d).reshape(Nt, -1, 3, 3)[j]
        psi_a, psi_v, psi_d = _apply_y_maps(self, bee(x_a_j, x_v_j, x_d_j, phi_a, phi_v, phi_d))
        psi_a = psi_a + self.mlp_a(psi_a)
        B_a = edges_reduce_src(src, psi_a, Nt).reshape(batch, nodes, -1)
        B_v = edges_reduce_src(src, psi_v, Nt).reshape(batch, nodes, -1, 3)
        B_d = edges_reduce_src(src, psi_d, Nt).reshape(batch, nodes, -1, 3, 3)
        return 0.1 * B_a, 0.1 * B_v, 0.1 * B_d


class OSelfTensProds(nn.Module):
    """archs/diffuser_atoms15.py:59-95"""

    def __init__(self, dim_a, dim_v, dim_d, chan, groups=8):
        super().__init__()
        self.L0, self.R0 = OTensLinear(0, dim_a, chan), OTensLinear(0, dim_a, chan)
        self.L1, self.R1 = OTensLinear(1, dim_v, chan), OTensLinear(1, dim_v, chan)
        self.L2, self.R2 = OTensLinear(2, dim_d, chan), OTensLinear(2, dim_d, chan)
        _add_y_maps(self, dim_a, dim_v, dim_d, chan)
        self.gn_a, self.gn_v, self.gn_d = OTensGroupNorm(0, dim_a, groups), OTensGroupNorm(1, dim_v, groups), OTensGroupNorm(2, dim_d, groups)

    def forward(self, x_a, x_v, x_d):
        rest = x_a.shape[:-1]
        n = math.prod(rest)
        xa, xv, xd = x_a.reshape(n, -1), x_v.reshape(n, -1, 3), x_d.reshape(n, -1, 3, 3)
        prods = bee(self.L0(xa), self.L1(xv), self.L2(xd), self.R0(xa), self.R1(xv), self.R2(xd))
        y_a, y_v, y_d = _apply_y_maps(self, prods)
        return (self.gn_a(y_a.reshape(*rest, -1)), self.gn_v(y_v.reshape(*rest, -1, 3)), self.gn_d(y_d.reshape(*rest, -1, 3, 3)))


class OBeeBlock(nn.Module):
    def __init__(self, r0, dim_a, dim_v, dim_d, chan):
        super().__init__()
        self.messages = OMessages(r0, dim_a, dim_v, dim_d, chan)
        self.prods = OSelfTensProds(dim_a, dim_v, dim_d, chan)

    def forward(self, src, dst, r_ij, x_a, x_v, x_d):
        d = self.messages(src, dst, r_ij, x_a, x_v, x_d)
        x_a, x_v, x_d = x_a + d[0], x_v + d[1], x_d + d[2]
        d = self.prods(x_a, x_v, x_d)
        return x_a + d[0], x_v + d[1], x_d + d[2]


class OBeeDenoiser(nn.Module):
    """The l<=2 denoiser of benchmark configs 2 and 4 (see ld_b200.bee.BeeDenoiser): reference layers
    (archs/diffuser_atoms15.py Messages / SelfTensProds) between the read-in and read-out of
    archs/meanflow_painn8.py:185-217."""

    def __init__(self, r0, dim_a, dim_v, dim_d, chan, ntypes, depth):
        super().__init__()
        self.r0, self.dim_d = r0, dim_d
        self.type_embed = nn.Embedding(ntypes, dim_a)
        self.v_readin = OTensLinear(1, 1, dim_v)
        self.blocks = nn.ModuleList([OBeeBlock(r0, dim_a, dim_v, dim_d, chan) for _ in range(depth)])
        self.readout = OTensLinear(1, dim_v, 1)
        self.edges_last = 0

    def forward(self, x0, x1, box, types):
        batch, nodes, _ = x0.shape
        g = radius_graph(x1, self.r0, box)   # membership and r_ij in float32, as the graph builder defines them
        x_a = self.type_embed(types)[None].expand(batch, -1, -1)
        x_v = self.v_readin((x1 - x0)[..., None, :])
        x_d = torch.zeros(batch, nodes, self.dim_d, 3, 3, dtype=x0.dtype)
        rij = g["rij"].to(x0.dtype)
        for blk in self.blocks:
            x_a, x_v, x_d = blk(g["src"], g["dst"], rij, x_a, x_v, x_d)
        self.edges_last = g["E"] * len(self.blocks)
        return self.readout(x_v).squeeze(-2)

    def generate(self, x_0, noise, sigma_0, box, types):
        z_1 = x_0 + sigma_0 * noise
        with torch.no_grad():
            return z_1 - self.forward(x_0, z_1, box, types)
