"""PaiNN / meanflow denoiser on the fused kernels.

Mirrors archs/meanflow_painn8.py of the reference: radial_encode (:25-35), MLP (:38-51), Update
(:53-75), Message (:77-100), Block (:102-125), CPaiNN (:128-143), TimeEmbedding (:145-165),
graph_setup (:167-172), PosEmbed (:174-183), SE3ITO (:185-217) and Meanflow.generate (:302-310),
with the same parameter names and shapes. The protein-specific pieces the reference takes from
its metadata (ResidueAtomEmbed, get_bond_graph) are replaced by a per-node type-embedding table
and a caller-supplied bond Graph.

Without autograd (inference, the path the rollout metric times) Message runs as two kernels:
mlp_actv once per node, then the fused edge kernel. With autograd enabled it runs the
reference's op sequence on this library's autograd-aware gather / scatter / TensLinear."""
import math

import torch
import torch.nn as nn

from . import ops
from .graph_layers import Graph, edges_read, edges_read_dst, edges_reduce_src, boxwrap
from .tensor_products import TensLinear


def radial_encode(r, n, rmax):
    """r: (..., 3) -> (..., n): cosines then sines of (pi/rmax)(1 + m//2) |r|"""
    hn = (n + 1) // 2
    coeffs = (torch.pi / rmax) * (1 + torch.arange(0, hn, device=r.device) // 2)
    dist = torch.linalg.vector_norm(r, dim=-1)[..., None]
    phase = coeffs * dist
    return torch.cat([torch.cos(phase), torch.sin(phase[..., :(n - hn)])], dim=-1)


class MLP(nn.Module):
    def __init__(self, dim_in, dim_out):
        super().__init__()
        self.layers = nn.Sequential(
            nn.Linear(dim_in, dim_out), nn.SiLU(), nn.Linear(dim_out, dim_out), nn.SiLU(), nn.Linear(dim_out, dim_out))
        self._packed = None
        self._packed_key = None
        self.precision = "fp32"  # "bf16": the three layers run as tcgen05 GEMMs (2e-2 relative)

    def packed(self):
        lin = (self.layers[0], self.layers[2], self.layers[4])
        key = tuple((p.data_ptr(), p._version) for l in lin for p in (l.weight, l.bias))
        if self._packed_key != key:
            self._packed = ops.PackedMLP(lin)
            self._packed_key = key
        return self._packed

    def forward(self, x_a):
        if torch.is_grad_enabled() or not x_a.is_cuda:
            return self.layers(x_a)
        mlp = self.packed()
        if self.precision == "bf16" and all(d % 32 == 0 for d in mlp.dims[1:]):
            w = ops._packed_bf16(mlp)
            h = ops.linear_bf16_tc(x_a, w[0], mlp.dims[1], mlp.b[0], ops.ACT_SILU)
            h = ops.linear_bf16_tc(h, w[1], mlp.dims[2], mlp.b[1], ops.ACT_SILU)
            return ops.linear_bf16_tc(h, w[2], mlp.dims[3], mlp.b[2], ops.ACT_NONE)
        return ops.mlp3_rows(x_a, mlp, ops.ACT_SILU)


class ScalGroupNorm(nn.Module):
    """managan/layers_common.py:201-223: statistics over the nodes of a system and a channel group."""

    def __init__(self, chan, groups, epsilon=1e-5):
        super().__init__()
        assert chan % groups == 0
        self.chan, self.groups, self.epsilon = chan, groups, epsilon
        self.gamma = nn.Parameter(torch.ones(chan))
        self.beta = nn.Parameter(torch.zeros(chan))

    def forward(self, x, residual=None):
        """residual (shape of x): returns residual + norm(x) (one pass on the fused path)"""
        if not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.float32:
            return ops.group_norm(x, self.groups, self.epsilon, self.gamma, self.beta, center=True, residual=residual)
        batch, nodes, _ = x.shape
        xg = x.reshape(batch, nodes, self.groups, -1)
        mean = xg.mean([1, 3], keepdim=True)
        x_shift = xg - mean
        var = (x_shift ** 2).mean([1, 3], keepdim=True)
        ans = x_shift / torch.sqrt(self.epsilon + var)
        ans = self.beta + self.gamma * ans.reshape(batch, nodes, self.chan)
        return ans if residual is None else residual + ans


class Update(nn.Module):
    def __init__(self, n):
        super().__init__()
        self.n = n
        self.lin_l = TensLinear(1, n, n)
        self.lin_r = TensLinear(1, n, n)
        self.lin_v = TensLinear(1, n, n)
        self.mlp = MLP(2 * n, 3 * n)
        assert n % 4 == 0
        self.gn = ScalGroupNorm(n, 4, epsilon=1.)

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


def radial_encode_gaussian(r, n, rmax):
    """Gaussian basis with cosine cutoff (benchmark configs; not in the reference): centres
    m*rmax/(n-1), width rmax/(n-1), envelope 0.5(cos(pi d/rmax)+1) for d < rmax."""
    d = torch.linalg.vector_norm(r, dim=-1)[..., None]
    width = rmax / (n - 1) if n > 1 else rmax
    mu = torch.arange(n, dtype=r.dtype, device=r.device) * width
    env = torch.where(d < rmax, 0.5 * (torch.cos(math.pi * d / rmax) + 1.0), torch.zeros_like(d))
    return torch.exp(-0.5 * ((d - mu) / width) ** 2) * env


class Message(nn.Module):
    """radial="painn", n_rbf=None is the reference layer; radial="gaussian" with n_rbf basis
    functions is the variant the benchmark configs describe."""

    def __init__(self, r0, n, n_rbf=None, radial="painn"):
        super().__init__()
        self.r0 = r0
        self.n = n
        self.epsilon = 0.1
        self.radial = radial
        self.precision = "fp32"  # "bf16": per-edge MLP on the tensor cores (2e-2 relative)
        self.n_rbf = n if n_rbf is None else n_rbf
        self.mlp_dist = MLP(self.n_rbf, 4 * n)
        self.mlp_actv = MLP(n, 4 * n)

    def forward(self, graph, x_a, x_v, r_ij, residual=False, edge_counter=None):
        """x_a: (batch, atoms, n); x_v: (batch, atoms, n, 3); r_ij: (edges, 3).
        Returns the summed messages (dx_a, dx_v); with residual=True returns x + dx instead."""
        if torch.is_grad_enabled() or not x_a.is_cuda:
            return self._forward_unfused(graph, x_a, x_v, r_ij, residual)
        batch, atoms, n = x_a.shape
        Nt = batch * atoms
        xa = x_a.reshape(Nt, n).contiguous()
        xv = x_v.reshape(Nt, n, 3).contiguous()
        actv = self.mlp_actv(xa)
        fused = ops.painn_message_bf16_tc if self.precision == "bf16" else ops.painn_message_f32
        out_a, out_v = fused(
            graph.row_ptr, graph.dst32, r_ij.contiguous(), self.mlp_dist.packed(), actv, xv, rmax=self.r0,
            eps=self.epsilon, radial_kind=ops.RADIAL_PAINN if self.radial == "painn" else ops.RADIAL_GAUSSIAN, res_a=xa if residual else None,
            res_v=xv if residual else None, edge_counter=edge_counter)
        return out_a.reshape(batch, atoms, n), out_v.reshape(batch, atoms, n, 3)

    def _forward_unfused(self, graph, x_a, x_v, r_ij, residual):
        enc = radial_encode(r_ij, self.n_rbf, self.r0) if self.radial == "painn" else radial_encode_gaussian(r_ij, self.n_rbf, self.r0)
        dist_x_a = self.mlp_dist(enc)
        actv_x_a = self.mlp_actv(edges_read_dst(graph, x_a))
        prod_x_a = dist_x_a * actv_x_a
        direction = r_ij / torch.sqrt(self.epsilon + (r_ij ** 2).sum(-1, keepdim=True))
        x_v_e = edges_read_dst(graph, x_v)
        cross = torch.linalg.cross(x_v_e, direction[:, None].expand_as(x_v_e))
        m_v = x_v_e * prod_x_a[..., :self.n, None]
        m_v = m_v + cross * prod_x_a[..., self.n:2 * self.n, None]
        m_v = m_v + direction[:, None] * prod_x_a[..., 2 * self.n:3 * self.n, None]
        d_v = edges_reduce_src(graph, m_v)
        d_a = edges_reduce_src(graph, prod_x_a[..., 3 * self.n:])
        if residual:
            return x_a + d_a, x_v + d_v
        return d_a, d_v


def graph_setup(r0, box, pos, cache=None):
    """radius graph + wrapped displacements; box=None means open boundaries. cache: optional
    graph.RolloutGraphCache (fixed-capacity buffers, no wait for the edge count; inference only)."""
    graph = Graph.radius_graph(r0, box, pos, cache=cache)
    if torch.is_grad_enabled() and pos.requires_grad:
        # the reference's form (archs/meanflow_painn8.py:167-172): differentiable in the positions,
        # which the meanflow training step needs for its Jacobian-vector product
        pos_src, pos_dst = edges_read(graph, pos)
        delta = pos_dst - pos_src
        if box is None:
            return graph, delta
        return graph, boxwrap(torch.as_tensor(box, dtype=pos.dtype, device=pos.device), delta)
    return graph, graph.rij


class Block(nn.Module):
    def __init__(self, r0, n, pos_mutable=False, n_rbf=None, radial="painn"):
        super().__init__()
        self.pos_mutable = pos_mutable
        self.r0 = r0
        self.message = Message(r0, n, n_rbf, radial)
        self.message_bond = Message(r0, n, n_rbf, radial)
        self.update = Update(n)
        if self.pos_mutable:
            self.lin_push_pos = TensLinear(1, n, 1)
        self.graph_cache = None   # set by enable_rollout_graphs

    def forward(self, tup):
        pos, graph, r_ij, graph_bond, r_ij_bond, x_a, x_v, box = tup[:8]
        counter = tup[8] if len(tup) > 8 else None
        if graph is None:
            graph, r_ij = graph_setup(self.r0, box, pos, self.graph_cache)
        if graph_bond.src32.numel() > 0:  # a bond graph without edges contributes exactly zero
            x_a, x_v = self.message_bond(graph_bond, x_a, x_v, r_ij_bond, residual=True, edge_counter=counter)
        x_a, x_v = self.message(graph, x_a, x_v, r_ij, residual=True, edge_counter=counter)
        dx_a, dx_v = self.update(x_a, x_v)
        x_a, x_v = x_a + dx_a, x_v + dx_v
        if self.pos_mutable:
            pos = pos + self.lin_push_pos(x_v).squeeze(-2)
            graph, r_ij = None, None
        return (pos, graph, r_ij, graph_bond, r_ij_bond, x_a, x_v, box) + ((counter,) if len(tup) > 8 else ())


def enable_rollout_graphs(module, margin=1.25):
    """Give every layer of `module` that builds a radius graph a graph.RolloutGraphCache: inside torch.no_grad() its
    builds then reuse edge buffers of a fixed capacity (margin x the first build's edge count, grown when the count
    comes close) and do not read the edge count back, so a rollout loop never waits for the device."""
    from .graph import RolloutGraphCache
    for m in module.modules():
        if hasattr(m, "graph_cache"):
            m.graph_cache = RolloutGraphCache(margin)
    return module


def finish_rollout_graphs(module):
    """wait for the reports of the last builds (end of a rollout); raises if one overflowed its capacity"""
    for m in module.modules():
        if getattr(m, "graph_cache", None) is not None and m.graph_cache.builder is not None:
            m.graph_cache.finish()


class CPaiNN(nn.Module):
    def __init__(self, r0, n, blks, ntypes, mutate_pos=False, n_rbf=None, radial="painn"):
        super().__init__()
        self.atom_embed = nn.Embedding(ntypes, n)  # stands in for ResidueAtomEmbed(metadata)
        self.blocks = nn.Sequential(*[Block(r0, n, mutate_pos, n_rbf, radial) for _ in range(blks)])

    def forward(self, pos, graph_bond, r_ij_bond, x_a, x_v, box, types, counter=None):
        x_a = x_a + self.atom_embed(types)[None]
        out = self.blocks((pos, None, None, graph_bond, r_ij_bond, x_a, x_v, box, counter))
        return out[0], out[5], out[6]


class TimeEmbedding(nn.Module):
    def __init__(self, freqs, outdim):
        super().__init__()
        self.freqs = freqs
        self.lin1 = nn.Linear(4 * self.freqs, outdim)

    def raw_t_embed(self, st):
        s, t = st
        ang_freqs = torch.exp(-torch.arange(self.freqs, device=s.device) / (self.freqs - 1))
        phases = torch.cat([t[:, None] * ang_freqs[None, :], (t - s)[:, None] * ang_freqs[None, :]], dim=1)
        return torch.cat([torch.sin(phases), torch.cos(phases)], dim=1)

    def forward(self, st):
        return self.lin1(self.raw_t_embed(st))


class PosEmbed(nn.Module):
    def __init__(self, dim_v):
        super().__init__()
        self.lin_v = TensLinear(1, 1, dim_v)

    def forward(self, pos_0, pos_1):
        dpos_v = 0.1 * (pos_1[:, :, None] - pos_0[:, :, None])
        return self.lin_v(dpos_v)


def chain_bond_graph(batch, nodes, device):
    """Bonds i<->i+1 of a linear polymer, sorted by source, replicated over the batch."""
    i = torch.arange(nodes - 1, device=device)
    src = torch.cat([i, i + 1])
    dst = torch.cat([i + 1, i])
    order = torch.argsort(src, stable=True)
    src, dst = src[order], dst[order]
    offs = nodes * torch.arange(batch, device=device)[:, None]
    return Graph((src[None] + offs).reshape(-1), (dst[None] + offs).reshape(-1), None, batch, nodes)


def empty_bond_graph(batch, nodes, device):
    z = torch.zeros(0, dtype=torch.int64, device=device)
    return Graph(z, z, None, batch, nodes)


class SE3ITO(nn.Module):
    def __init__(self, r0, n, natoms, ntypes=1, blks_0=2, blks_1=5, n_rbf=None, radial="painn"):
        super().__init__()
        self.r0 = r0
        self.atom_embeddings = nn.Parameter(torch.randn(natoms, n))
        self.t_embed = TimeEmbedding(32, n)
        self.mlp_embed = MLP(n, n)
        self.mlp_denoise = MLP(n, n)
        self.pos_emb = PosEmbed(n)
        self.cpainn_0 = CPaiNN(r0, n, blks_0, ntypes, n_rbf=n_rbf, radial=radial)
        self.cpainn_1 = CPaiNN(r0, n, blks_1, ntypes, n_rbf=n_rbf, radial=radial)
        self.v_readin = TensLinear(1, 1, n)
        self.readout = TensLinear(1, n, 1)

    def get_v_pred(self, st, v_pred, x1_s_pred, x1_t):
        s, t = st
        return (1. - (t - s)[:, None, None]) * v_pred + x1_t - x1_s_pred

    def forward(self, st, x0, x1, box, types, graph_bond, counter=None):
        x0, x1 = x0.contiguous(), x1.contiguous()
        x1_t = x1
        flat0, flat1 = x0.reshape(-1, 3), x1.reshape(-1, 3)
        r_ij_bond_0 = flat0[graph_bond.dst] - flat0[graph_bond.src]
        r_ij_bond_1 = flat1[graph_bond.dst] - flat1[graph_bond.src]
        x_a = self.atom_embeddings[None].expand(x0.shape[0], -1, -1)
        x_v = self.v_readin((x1 - x0)[..., None, :])
        x_a = self.mlp_embed(x_a.contiguous())
        x0, x_a, x_v = self.cpainn_0(x0, graph_bond, r_ij_bond_0, x_a, x_v, box, types, counter)
        x_a = self.mlp_denoise(x_a + self.t_embed(st)[:, None])
        x_v = x_v + self.pos_emb(x0, x1)
        x1, x_a, x_v = self.cpainn_1(x1, graph_bond, r_ij_bond_1, x_a, x_v, box, types, counter)
        return self.get_v_pred(st, self.readout(x_v).squeeze(-2), x1, x1_t)


def set_precision(module, precision):
    """"fp32" (default, 1e-5 parity) or "bf16" (tensor-core per-edge MLP, 2e-2) for every Message below `module`."""
    assert precision in ("fp32", "bf16")
    for m in module.modules():
        if isinstance(m, (Message, MLP)):
            m.precision = precision
    return module


class Meanflow:
    """The reference's Meanflow wrapper: generate/predict (:302-318) and the training objective (:269-297)."""

    def __init__(self, dn, box, sigma_0, types, graph_bond):
        self.dn, self.box, self.sigma_0, self.types, self.graph_bond = dn, box, sigma_0, types, graph_bond

    @torch.no_grad()
    def generate(self, x_0, noise=None, counter=None):
        lead = x_0.shape[:-2]
        atoms = x_0.shape[-2]
        batch = math.prod(lead)
        x_0 = x_0.reshape(batch, atoms, 3)
        if noise is None:
            noise = torch.randn_like(x_0)
        z_1 = x_0 + self.sigma_0 * noise.reshape(batch, atoms, 3)
        st = (torch.zeros(batch, device=x_0.device), torch.ones(batch, device=x_0.device))
        v_pred = self.dn(st, x_0, z_1, self.box, self.types, self.graph_bond, counter)
        if x_0.is_cuda:
            ops.check_tc_status(x_0.device, block=False)   # a kernel that gave up on a wait is reported, not passed on
        return (z_1 - v_pred).reshape(*lead, atoms, 3)

    def predict(self, state, counter=None):
        """state: a ModelState (the reference's calling convention, :316-318) or a position tensor"""
        x = state if isinstance(state, torch.Tensor) else state.x
        return self.generate(x, counter=counter)

    def set_eval(self, bool_eval):
        self.dn.train(not bool_eval)

    def diffuser_loss(self, x_prev, z_0, z_1, s, t, loss_wt="ph"):
        """The meanflow training objective of the reference's _diffuser_step
        (archs/meanflow_painn8.py:269-297) with the random draws (z_1, s, t) passed in and the
        optimiser left to the caller: v_target = v - (t - s) * d/dt dn along (v, 1), taken as a
        Jacobian-vector product with create_graph=True, so the loss gradient is a double backward
        through every kernel-backed autograd function of this library."""
        tt = t[:, None, None]
        z_t, v = tt * z_1 + (1 - tt) * z_0, z_1 - z_0
        f = lambda z, tau: self.dn((s, tau), x_prev, z, self.box, self.types, self.graph_bond)  # noqa: E731
        _, jvp = torch.autograd.functional.jvp(f, (z_t, t), (v, torch.ones_like(t)), create_graph=True)
        v_target = v - (t - s)[:, None, None] * jvp
        v_pred = f(z_t, t)
        d_sq = ((v_pred - v_target) ** 2).mean((1, 2))
        if loss_wt == "ph":
            d_sq = d_sq / (0.5 + d_sq.detach()) ** 0.7
        return d_sq.mean()
