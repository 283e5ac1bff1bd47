"""Host-side mirror of the proximity-attention modules of managan/attention_layers.py (the older WGAN architectures):
ProbePoints2 (reference lines 41-73), ProximityFlashAttention (:275-338) and ProximityFlashAttentionPeriodic (:341-404),
with the reference's parameter names and shapes, so its state dicts load unchanged. The all-pairs operator underneath is
this library's `proxattn` / `proxattn_periodic` (csrc/proxattn.cu, csrc/proxattn_tc.cu) in place of the reference's
Triton kernels; `precision="tf32"` selects the tensor-core forward (no gradient)."""
import torch
import torch.nn as nn

from .proxattn import proxattn, proxattn_periodic


class VecRootS(nn.Module):
    """activation that is S-shaped along any direction: v (1 + |v|^2)^(-1/4) (managan/layers_common.py:91-98)"""

    def forward(self, v):
        return v * (1. + (v * v).sum(-1, keepdim=True)) ** (-0.25)


class ProbePoints2(nn.Module):
    """One probe point per head and node: a softmax mixture of the given base points plus a mix of the node's vectors
    -> (batch, heads, nodes, 3)."""

    def __init__(self, n_base_pts, heads, adim, vdim):
        super().__init__()
        self.n_base_pts, self.H = n_base_pts, heads
        self.lin_mix = nn.Linear(adim, n_base_pts * heads, bias=False)   # kept for state-dict parity; unused, as in the reference
        self.W_mix = nn.Parameter(torch.empty(heads, n_base_pts, adim))
        self.W_vec = nn.Parameter(torch.empty(heads, vdim))

    def self_init(self):
        nn.init.normal_(self.W_vec, std=self.W_vec.shape[1] ** -0.5)
        nn.init.normal_(self.W_mix, std=self.W_mix.shape[2] ** -0.5)

    def forward(self, ax, vx, positions):
        base = torch.stack(positions, dim=2)                                      # (batch, nodes, base points, 3)
        assert base.shape[2] == self.n_base_pts
        mix = torch.softmax(torch.einsum("hpj,bnj->bhnp", self.W_mix, ax), dim=3)
        return torch.einsum("bnpv,bhnp->bhnv", base, mix) + torch.einsum("hj,bnjv->bhnv", self.W_vec, vx)


class _ProximityFlashAttentionBase(nn.Module):
    def __init__(self, r0_list, adim, vdim, chan, vec_actv_class=VecRootS):
        super().__init__()
        self.H, self.chan = len(r0_list), chan
        self.register_buffer("r0sq", torch.tensor(r0_list) ** 2, persistent=False)
        for name, width in (("W_aq", adim), ("W_vq", vdim), ("W_ak", adim), ("W_vk", vdim), ("W_av", adim), ("W_vv", vdim)):
            setattr(self, name, nn.Parameter(torch.empty(self.H, chan, width)))
        self.W_ao = nn.Parameter(torch.empty(self.H, adim, chan))
        self.W_vo = nn.Parameter(torch.empty(self.H, vdim, chan))
        self.vec_actv = vec_actv_class()
        self.precision = "fp32"

    def self_init(self):
        for name in ("W_aq", "W_vq", "W_ak", "W_vk", "W_av", "W_vv"):
            p = getattr(self, name)
            nn.init.normal_(p, std=p.shape[1] ** -0.5)

    @staticmethod
    def stack_av(a, v):
        """(..., chan), (..., chan, 3) -> (..., 4 chan): per channel the scalar followed by its vector"""
        return torch.cat([a[..., None], v], dim=-1).flatten(-2)

    @staticmethod
    def split_av(t):
        chan = t.shape[-1] // 4
        return t[..., :chan], t[..., chan:].reshape(*t.shape[:-1], chan, 3)

    def _qkv(self, ax, vx):
        batch, nodes = ax.shape[0], ax.shape[1]
        def proj(Wa, Wv):
            return self.stack_av(torch.einsum("hij,bnj->bhni", Wa, ax), torch.einsum("hij,bnjv->bhniv", Wv, vx)) \
                .reshape(batch * self.H, nodes, 4 * self.chan).contiguous()
        # the activation runs along the stacked dimension of size 4 chan, as in the reference
        return self.vec_actv(proj(self.W_aq, self.W_vq)), self.vec_actv(proj(self.W_ak, self.W_vk)), proj(self.W_av, self.W_vv)

    def _out(self, O, batch, nodes):
        O = O / nodes ** 0.5
        ay, vy = self.split_av(O)
        return (torch.einsum("hji,bhni->bnj", self.W_ao, ay.reshape(batch, self.H, nodes, self.chan)),
                torch.einsum("hji,bhniv->bnjv", self.W_vo, vy.reshape(batch, self.H, nodes, self.chan, 3)))


class ProximityFlashAttention(_ProximityFlashAttentionBase):
    """ax (batch, nodes, adim), vx (batch, nodes, vdim, 3), pos_k / pos_q (batch, heads, nodes, 3) -> ay, vy."""

    def forward(self, ax, vx, pos_k, pos_q):
        batch, nodes = ax.shape[0], ax.shape[1]
        Q, K, V = self._qkv(ax, vx)
        O = proxattn(Q, K, V, pos_q.reshape(batch * self.H, nodes, 3).contiguous(), pos_k.reshape(batch * self.H, nodes, 3).contiguous(),
                     self.r0sq, precision=self.precision)
        return self._out(O, batch, nodes)


class ProximityFlashAttentionPeriodic(_ProximityFlashAttentionBase):
    """the same in a periodic box (Lx, Ly, Lz)"""

    def forward(self, ax, vx, pos_k, pos_q, box):
        batch, nodes = ax.shape[0], ax.shape[1]
        Q, K, V = self._qkv(ax, vx)
        O = proxattn_periodic(Q, K, V, pos_q.reshape(batch * self.H, nodes, 3).contiguous(),
                              pos_k.reshape(batch * self.H, nodes, 3).contiguous(), self.r0sq, box, precision=self.precision)
        return self._out(O, batch, nodes)
