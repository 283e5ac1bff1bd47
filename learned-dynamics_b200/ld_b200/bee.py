"""l<=2 ("Bee"-path) message layer on the fused kernels.

Mirrors Messages of archs/diffuser_atoms15.py:227-253 (and its helpers MLP :98-110,
add_tens_prod_submodules :29-42, apply_tens_prod_submodules :52-57, radial_encode_8 of
managan/jacobi_radenc.py:8-37) with the reference's parameter names. Without autograd the layer
runs as: three node-level channel mixings (L0, L1, L2), one pass over the edges for the rank-1/2
products summed per node, one pass for the scalar channel (per-edge Y maps + mlp_a), and two
node-level channel mixings for the hoisted Y maps. With autograd it runs the reference's op
sequence on this library's Bee / TensLinear / gather / segment-sum functions."""
from math import comb

import torch
import torch.nn as nn

from . import ops
from ._lib import lib, check, ptr, stream_ptr, KERNEL_TIMER
from .codegen_tensor_products import Bee
from .graph_layers import edges_read_dst, edges_reduce_src
from .tensor_products import TensLinear, tens_sigmoid

V_ORDER = ("011", "101", "121", "211", "111")
D_ORDER = ("022", "202", "112", "222", "212")


def jacobi_matrix(dim=8):
    """Coefficients (ascending powers of x) of the shifted Jacobi(1,0) polynomials on [0,1]:
    P_n(x) = sum_s C(n+1, n-s) C(n, s) (x-1)^s x^(n-s); exact integers, as the reference's sympy expansion."""
    A = torch.zeros(dim, dim + 1)
    for n in range(dim):
        coeffs = [0] * (n + 1)
        for s in range(n + 1):
            w = comb(n + 1, n - s) * comb(n, s)
            for t in range(s + 1):
                coeffs[n - s + t] += w * comb(s, t) * (-1) ** (s - t)
        for j, c in enumerate(coeffs):
            A[n, j] = float(c)
    return A


def radial_encode_8(r, rmax):
    """r: (..., 3) -> (..., 8). The power sum is evaluated in float64 (as the fused kernels do): the coefficients reach
    2.7e4 with alternating signs, and in float32 the cancellation costs four digits."""
    A = jacobi_matrix(8).to(device=r.device, dtype=torch.float64)
    z = (torch.linalg.vector_norm(r, dim=-1) / rmax)[..., None]
    pows = z.double() ** torch.arange(A.shape[1], device=r.device)
    return (torch.nn.functional.linear(pows, A) * torch.relu(1. - z).double()).to(r.dtype)


class MLP(nn.Module):
    def __init__(self, dim_a):
        super().__init__()
        self.lin_direct = nn.Linear(dim_a, dim_a, bias=False)
        self.layers = nn.Sequential(
            nn.Linear(dim_a, 2 * dim_a), nn.LeakyReLU(0.1), nn.Linear(2 * dim_a, 2 * dim_a), nn.LeakyReLU(0.1),
            nn.Linear(2 * dim_a, dim_a))

    def forward(self, x):
        return self.lin_direct(x) + self.layers(x)


_ROWS_CACHE = {}


def _gather_rows_buffer(Nt, chan, device):
    """[Nt][2][chan][8] BF16 buffer for the neighbour rows of the fused edge kernel, zero-initialised once: three of
    the sixteen values per (node, channel) are never written and must stay finite (they meet zeros in the MMA).
    One buffer per (size, device) serves all layers: they use it one after the other on the same stream."""
    key = (Nt, chan, torch.device(device).index, torch.cuda.current_stream(device).cuda_stream)
    buf = _ROWS_CACHE.get(key)
    if buf is None:
        if len(_ROWS_CACHE) > 8:
            _ROWS_CACHE.clear()
        buf = torch.zeros(Nt, 2, chan, 8, dtype=torch.bfloat16, device=device)
        _ROWS_CACHE[key] = buf
    return buf


class Messages(nn.Module):
    def __init__(self, r0, dim_a, dim_v, dim_d, chan):
        super().__init__()
        self.r0, self.dim_a, self.dim_v, self.dim_d, self.chan = r0, dim_a, dim_v, dim_d, chan
        self.L0 = TensLinear(0, dim_a, chan)
        self.L1 = TensLinear(1, dim_v, chan)
        self.L2 = TensLinear(2, dim_d, chan)
        for name in ("000", "110", "220"):
            setattr(self, "Y_" + name, TensLinear(0, chan, dim_a))
        for name in V_ORDER:
            setattr(self, "Y_" + name, TensLinear(1, chan, dim_v))
        for name in D_ORDER:
            setattr(self, "Y_" + name, TensLinear(2, chan, dim_d))
        self.lin_enc = nn.Linear(8, chan)
        self.mlp_a = MLP(dim_a)
        self._packed = None
        self._packed_key = None
        self.precision = "fp32"  # "bf16": scalar channel on the tensor cores (2e-2 relative)
        # bf16, chan = dim_a = 128: True runs the layer as ONE edge kernel (rows gathered once, per-node sums accumulated
        # by the tensor cores). Correct and deterministic, but measured slower than the two-kernel path on B200 (its
        # per-edge synchronisation leaves the warps latency-bound), so it is opt-in.
        self.fused_kernel = False
        # bf16, chan = 128: True forms the rank-1 / rank-2 product sums on the tensor cores (one MMA per edge with the
        # scaled row as a tensor-memory operand, sums accumulated in tensor memory) instead of FP32 FMAs. Correct and
        # deterministic, four times fewer instructions per edge, but measured slower on B200 (about 24 ms against 17 ms
        # per 19.4 M edges): its warps wait on one another once per four edges, the FMA kernel's never do. Opt-in.
        self.vd_tensor_core = False
        # bf16, chan = 128: L0, L1, L2 as one launch that writes whole neighbour rows
        self.rows_one_launch = True

    def load_state_dict(self, state, *a, **k):
        # the reference wraps mlp_a in torch.compile, which prefixes its keys
        state = {key.replace("mlp_a._orig_mod.", "mlp_a."): v for key, v in state.items()}
        return super().load_state_dict(state, *a, **k)

    def _pack(self):
        key = (self.precision,) + tuple((p.data_ptr(), p._version) for p in self.parameters())
        if self._packed_key != key:
            dev = self.lin_enc.weight.device
            f = lambda t: t.detach().float().contiguous()
            lay = self.mlp_a.layers
            self._packed = {
                "jac": jacobi_matrix(8).to(dev).contiguous(),
                "enc_w": f(self.lin_enc.weight), "enc_b": f(self.lin_enc.bias),
                "Yt": f(torch.cat([self.Y_000.W, self.Y_110.W, self.Y_220.W], dim=1).t()),
                "Yv": f(torch.cat([getattr(self, "Y_" + n).W for n in V_ORDER], dim=1)),
                "Yd": f(torch.cat([getattr(self, "Y_" + n).W for n in D_ORDER], dim=1)),
                "W1t": f(lay[0].weight.t()), "b1": f(lay[0].bias), "W2t": f(lay[2].weight.t()), "b2": f(lay[2].bias),
                "W3t": f(lay[4].weight.t()), "b3": f(lay[4].bias), "Wdt": f(self.mlp_a.lin_direct.weight.t()),
            }
            if self.precision == "bf16":
                eye = torch.eye(self.dim_a, device=dev)
                p = self._packed
                p["Yp"] = ops.pack_weights_bf16(p["Yt"].t().contiguous())
                p["W1p"] = ops.pack_weights_bf16(f(lay[0].weight))
                p["W2p"] = ops.pack_weights_bf16(f(lay[2].weight))
                p["W3p"] = ops.pack_weights_bf16(torch.cat([f(lay[4].weight), f(self.mlp_a.lin_direct.weight) + eye], dim=1).contiguous())
                p["Yvp"], p["Ydp"] = ops.pack_weights_bf16(p["Yv"]), ops.pack_weights_bf16(p["Yd"])
            self._packed_key = key
        return self._packed

    def _forward_fused_tc(self, graph, r_ij, x_a, x_v, x_d):
        """chan = 128, dim_a = 128 on the tensor cores: three channel mixings that write the neighbour rows in the
        gather layout, ONE edge kernel (rows gathered once by bulk copies, products by tcgen05, per-edge MLP), and the
        two hoisted Y maps per node."""
        batch, nodes = x_a.shape[0], x_a.shape[1]
        Nt, C, dev = batch * nodes, self.chan, x_a.device
        w = self._pack()
        pk = lambda m: m._packed_for(ops)
        rows = _gather_rows_buffer(Nt, C, dev)
        ops.linear_bf16_tc(x_a.reshape(Nt, -1), pk(self.L0), C, inds=0, out=rows, out_layout=(16 * C, 8, 0))
        ops.linear_bf16_tc(x_v.reshape(Nt, -1, 3), pk(self.L1), C, inds=1, out=rows, out_layout=(16 * C, 8, 1))
        ops.linear_bf16_tc(x_d.reshape(Nt, -1, 3, 3), pk(self.L2), C, inds=2, out=rows, out_layout=(16 * C, 8, 4),
                           out_split=(4, 8 * C - 8))
        S_v = torch.empty(Nt, 3, 5 * C, dtype=torch.bfloat16, device=dev)
        S_d = torch.empty(Nt, 9, 5 * C, dtype=torch.bfloat16, device=dev)
        B_a = torch.empty(Nt, self.dim_a, dtype=torch.float32, device=dev)
        with KERNEL_TIMER.region("bee_messages_fused_tc"):
            check(lib().ld_bee_messages_fused_bf16_tc(ptr(graph.row_ptr), ptr(graph.dst32), ptr(r_ij.contiguous()), Nt, C, self.dim_a,
                                                      float(self.r0), ptr(rows), ptr(w["enc_w"]), ptr(w["enc_b"]), ptr(w["jac"]),
                                                      ptr(w["Yp"]), ptr(w["W1p"]), ptr(w["b1"]), ptr(w["W2p"]), ptr(w["b2"]),
                                                      ptr(w["W3p"]), ptr(w["b3"]), 0.1, ptr(B_a), ptr(S_v), ptr(S_d),
                                                      ptr(ops.tc_status(dev)), stream_ptr(dev)))
        B_v = ops.linear_bf16_tc_cm(S_v, w["Yvp"], self.dim_v, 1)
        B_d = ops.linear_bf16_tc_cm(S_d, w["Ydp"], self.dim_d, 2)
        return (B_a.reshape(batch, nodes, -1), B_v.reshape(batch, nodes, -1, 3), B_d.reshape(batch, nodes, -1, 3, 3))

    def cm_ready(self):
        """the tensor-core path that takes component-major activations applies (widths in whole tensor-core tiles)"""
        return (self.precision == "bf16" and self.chan % 32 == 0 and self.chan <= 512 and self.dim_a in (64, 128)
                and self.dim_v % 32 == 0 and self.dim_d % 32 == 0 and self.dim_v % 4 == 0 and self.dim_d % 4 == 0)

    def forward_cm(self, graph, r_ij, x_a, x_v, x_d):
        """forward for component-major activations, x_v [B, N, 3, dim_v], x_d [B, N, 9, dim_d] (results in the same
        form): every channel mixing then works on plain rows (16-byte loads, coalesced stores)."""
        batch, nodes = x_a.shape[0], x_a.shape[1]
        Nt, C, dev = batch * nodes, self.chan, x_a.device
        w = self._pack()
        pk = lambda m: m._packed_for(ops)
        lp = torch.empty(Nt, C, 16, dtype=torch.bfloat16, device=dev)
        ops.linear_bf16_tc(x_a.reshape(Nt, -1), pk(self.L0), C, inds=0, out=lp, out_layout=(16 * C, 16, 0))
        ops.linear_bf16_tc(x_v.reshape(Nt, 3, -1), pk(self.L1), C, inds=1, out=lp, out_layout=(16 * C, 16, 1), in_cm=True)
        ops.linear_bf16_tc(x_d.reshape(Nt, 9, -1), pk(self.L2), C, inds=2, out=lp, out_layout=(16 * C, 16, 4), in_cm=True)
        rij = r_ij.contiguous()
        S_v = torch.empty(Nt, 3, 5 * C, dtype=torch.bfloat16, device=dev)
        S_d = torch.empty(Nt, 9, 5 * C, dtype=torch.bfloat16, device=dev)
        B_a = torch.empty(Nt, self.dim_a, dtype=torch.float32, device=dev)
        st = stream_ptr(dev)
        with KERNEL_TIMER.region("bee_messages_vd"):
            check(lib().ld_bee_messages_vd_f32(ptr(graph.row_ptr), ptr(graph.dst32), ptr(rij), Nt, C, float(self.r0), ptr(lp),
                                               ptr(lp), ptr(lp), ptr(w["enc_w"]), ptr(w["enc_b"]), ptr(w["jac"]), 0.1,
                                               ptr(S_v), ptr(S_d), 2, 1, st))
        with KERNEL_TIMER.region("bee_messages_scalar_tc"):
            check(lib().ld_bee_messages_scalar_bf16_tc(ptr(graph.row_ptr), ptr(graph.dst32), ptr(rij), Nt, C, self.dim_a,
                                                       float(self.r0), ptr(lp), ptr(lp), ptr(lp), ptr(w["enc_w"]),
                                                       ptr(w["enc_b"]), ptr(w["jac"]), ptr(w["Yp"]), ptr(w["W1p"]), ptr(w["b1"]),
                                                       ptr(w["W2p"]), ptr(w["b2"]), ptr(w["W3p"]), ptr(w["b3"]), 0.1, ptr(B_a),
                                                       2, ptr(ops.tc_status(dev)), st))
        B_v = ops.linear_bf16_tc_rows16(S_v, w["Yvp"], self.dim_v)
        B_d = ops.linear_bf16_tc_rows16(S_d, w["Ydp"], self.dim_d)
        return (B_a.reshape(batch, nodes, -1), B_v.reshape(batch, nodes, 3, -1), B_d.reshape(batch, nodes, 9, -1))

    def forward(self, graph, r_ij, x_a, x_v, x_d, add_input=False):
        """add_input: returns the inputs plus the messages (the residual form the layers use), added inside the kernels'
        epilogues on the tensor-core path"""
        out, added = self._forward(graph, r_ij, x_a, x_v, x_d, add_input)
        if add_input and not added:
            out = (x_a + out[0], x_v + out[1], x_d + out[2])
        return out

    def _forward(self, graph, r_ij, x_a, x_v, x_d, add_input):
        """returns (messages, whether the inputs were already added to them)"""
        if torch.is_grad_enabled() or not x_a.is_cuda:
            return self._forward_unfused(graph, r_ij, x_a, x_v, x_d), False
        batch, nodes = x_a.shape[0], x_a.shape[1]
        Nt, C, dev = batch * nodes, self.chan, x_a.device
        if (self.precision == "bf16" and self.fused_kernel and C == 128 and self.dim_a == 128 and self.dim_v % 32 == 0
                and self.dim_d % 32 == 0):
            return self._forward_fused_tc(graph, r_ij, x_a, x_v, x_d), False
        w = self._pack()
        feat16 = self.precision == "bf16" and C % 32 == 0 and C <= 512
        if feat16:
            # left operands straight to BF16, interleaved per channel as [node][chan][16] = (l0, l1[3], l2[9], pad):
            # the edge kernels fetch all thirteen values of a (neighbour, channel) with one 32-byte load
            pk = lambda m: m._packed_for(ops)
            lp = torch.empty(Nt, C, 16, dtype=torch.bfloat16, device=dev)
            da, dv, dd = x_a.shape[-1], x_v.shape[-2], x_d.shape[-3]
            if (self.rows_one_launch and C == 128 and da % 16 == 0 and dv % 16 == 0 and dd % 16 == 0 and da + 3 * dv + 9 * dd <= 640
                    and all(t.dtype == torch.float32 for t in (x_a, x_v, x_d))):
                # one launch that writes whole 32-byte rows (three launches write 2, 6 and 18 bytes of each)
                with KERNEL_TIMER.region("linear_bf16_tc"):
                    check(lib().ld_bee_left_rows_bf16_tc(ptr(x_a.contiguous()), ptr(x_v.contiguous()), ptr(x_d.contiguous()), Nt, da, dv,
                                                         dd, C, ptr(pk(self.L0)), ptr(pk(self.L1)), ptr(pk(self.L2)), ptr(lp),
                                                         ptr(ops.tc_status(dev)), stream_ptr(dev)))
            else:
                ops.linear_bf16_tc(x_a.reshape(Nt, -1), pk(self.L0), C, inds=0, out=lp, out_layout=(16 * C, 16, 0))
                ops.linear_bf16_tc(x_v.reshape(Nt, -1, 3), pk(self.L1), C, inds=1, out=lp, out_layout=(16 * C, 16, 1))
                ops.linear_bf16_tc(x_d.reshape(Nt, -1, 3, 3), pk(self.L2), C, inds=2, out=lp, out_layout=(16 * C, 16, 4))
            l0 = l1 = l2 = lp
        else:
            l0 = self.L0(x_a.reshape(Nt, -1))
            l1 = self.L1(x_v.reshape(Nt, -1, 3))
            l2 = self.L2(x_d.reshape(Nt, -1, 3, 3))
        rij = r_ij.contiguous()
        # the per-node product sums feed tensor-core channel mixings on the bf16 path, which round them to BF16 anyway
        sums16 = self.precision == "bf16" and self.dim_v % 32 == 0 and self.dim_d % 32 == 0
        sdt = torch.bfloat16 if sums16 else torch.float32
        # (BF16 sums are component-major, [Nt][3 | 9][5C]: a (node, component) row is the GEMM's contiguous K)
        S_v = torch.empty((Nt, 3, 5 * C) if sums16 else (Nt, 5 * C, 3), dtype=sdt, device=dev)
        S_d = torch.empty((Nt, 9, 5 * C) if sums16 else (Nt, 5 * C, 3, 3), dtype=sdt, device=dev)
        B_a = torch.empty(Nt, self.dim_a, dtype=torch.float32, device=dev)
        st = stream_ptr(dev)
        if feat16 and sums16 and C == 128 and self.vd_tensor_core:
            with KERNEL_TIMER.region("bee_messages_vd_tc"):
                check(lib().ld_bee_messages_vd_bf16_tc(ptr(graph.row_ptr), ptr(graph.dst32), ptr(rij), Nt, C, float(self.r0), ptr(lp),
                                                       ptr(w["enc_w"]), ptr(w["enc_b"]), ptr(w["jac"]), 0.1, ptr(S_v), ptr(S_d),
                                                       ptr(ops.tc_status(dev)), st))
        else:
            with KERNEL_TIMER.region("bee_messages_vd"):
                check(lib().ld_bee_messages_vd_f32(ptr(graph.row_ptr), ptr(graph.dst32), ptr(rij), Nt, C, float(self.r0), ptr(l0),
                                                   ptr(l1), ptr(l2), ptr(w["enc_w"]), ptr(w["enc_b"]), ptr(w["jac"]), 0.1,
                                                   ptr(S_v), ptr(S_d), 2 if feat16 else 0, 1 if sums16 else 0, st))
        # the residual form: the rank-1 and rank-2 adds happen in the epilogues of the two Y maps (the scalar edge kernel
        # writes a node's row on its critical path, where a load of the residual cost more than the separate add)
        fuse_add = (add_input and self.precision == "bf16" and sums16 and all(t.dtype == torch.float32 for t in (x_a, x_v, x_d)))
        if self.precision == "bf16":
            with KERNEL_TIMER.region("bee_messages_scalar_tc"):
                check(lib().ld_bee_messages_scalar_bf16_tc(ptr(graph.row_ptr), ptr(graph.dst32), ptr(rij), Nt, C, self.dim_a,
                                                           float(self.r0), ptr(l0), ptr(l1), ptr(l2), ptr(w["enc_w"]),
                                                           ptr(w["enc_b"]), ptr(w["jac"]), ptr(w["Yp"]), ptr(w["W1p"]), ptr(w["b1"]),
                                                           ptr(w["W2p"]), ptr(w["b2"]), ptr(w["W3p"]), ptr(w["b3"]), 0.1, ptr(B_a),
                                                           2 if feat16 else 0, ptr(ops.tc_status(dev)), st))
            if fuse_add:
                B_a += x_a.reshape(Nt, -1)
        else:
            with KERNEL_TIMER.region("bee_messages_scalar"):
                check(lib().ld_bee_messages_scalar_f32(ptr(graph.row_ptr), ptr(graph.dst32), ptr(rij), Nt, C, self.dim_a,
                                                       float(self.r0), ptr(l0), ptr(l1), ptr(l2), ptr(w["enc_w"]),
                                                       ptr(w["enc_b"]), ptr(w["jac"]), ptr(w["Yt"]), ptr(w["W1t"]), ptr(w["b1"]),
                                                       ptr(w["W2t"]), ptr(w["b2"]), ptr(w["W3t"]), ptr(w["b3"]), ptr(w["Wdt"]),
                                                       0.1, ptr(B_a), st))
        if sums16:
            B_v = ops.linear_bf16_tc_cm(S_v, w["Yvp"], self.dim_v, 1, residual=x_v.reshape(Nt, -1, 3) if fuse_add else None)
            B_d = ops.linear_bf16_tc_cm(S_d, w["Ydp"], self.dim_d, 2, residual=x_d.reshape(Nt, -1, 3, 3) if fuse_add else None)
        else:
            B_v = ops.tensor_linear(1, w["Yv"], S_v)
            B_d = ops.tensor_linear(2, w["Yd"], S_d)
        return (B_a.reshape(batch, nodes, -1), B_v.reshape(batch, nodes, -1, 3), B_d.reshape(batch, nodes, -1, 3, 3)), fuse_add

    def _forward_unfused(self, graph, r_ij, x_a, x_v, x_d):
        rad_enc_ij = self.lin_enc(radial_encode_8(r_ij, self.r0))
        r = tens_sigmoid(1, r_ij * (7. / self.r0))
        phi_a = rad_enc_ij
        phi_v = rad_enc_ij[..., None] * r[..., None, :]
        phi_d = rad_enc_ij[..., None, None] * r[..., None, None, :] * r[..., None, :, None]
        x_a_j = edges_read_dst(graph, self.L0(x_a))
        x_v_j = edges_read_dst(graph, self.L1(x_v))
        x_d_j = edges_read_dst(graph, self.L2(x_d))
        (y_000, y_110, y_220, y_011, y_101, y_121, y_211, y_022, y_202, y_112, y_222, y_111, y_212) = Bee.apply(
            x_a_j, x_v_j, x_d_j, phi_a.contiguous(), phi_v.contiguous(), phi_d.contiguous())
        psi_a = self.Y_000(y_000) + self.Y_110(y_110) + self.Y_220(y_220)
        psi_v = self.Y_011(y_011) + self.Y_101(y_101) + self.Y_121(y_121) + self.Y_211(y_211) + self.Y_111(y_111)
        psi_d = self.Y_022(y_022) + self.Y_202(y_202) + self.Y_112(y_112) + self.Y_222(y_222) + self.Y_212(y_212)
        psi_a = psi_a + self.mlp_a(psi_a)
        B_a = edges_reduce_src(graph, psi_a)
        B_v = edges_reduce_src(graph, psi_v)
        B_d = edges_reduce_src(graph, psi_d)
        return 0.1 * B_a, 0.1 * B_v, 0.1 * B_d


def set_precision(module, precision):
    """"fp32" or "bf16" (scalar channel of every Messages layer on the tensor cores, 2e-2 relative)."""
    assert precision in ("fp32", "bf16")
    for m in module.modules():
        if isinstance(m, Messages):
            m.precision = precision
    # the node-level channel mixings inside the l<=2 layers follow (read-in / read-out stay FP32)
    for m in module.modules():
        if isinstance(m, (Messages, SelfTensProds)):
            for sub in m.modules():
                if isinstance(sub, TensLinear):
                    sub.precision = precision
    return module


class SelfTensProds(nn.Module):
    """Node-local tensor products (archs/diffuser_atoms15.py:59-95): left/right channel mixings,
    the 13 Bee products, the Y maps and a group norm per rank."""

    def __init__(self, dim_a, dim_v, dim_d, chan, groups=8):
        super().__init__()
        from .tensor_products import TensGroupNorm
        self.L0, self.R0 = TensLinear(0, dim_a, chan), TensLinear(0, dim_a, chan)
        self.L1, self.R1 = TensLinear(1, dim_v, chan), TensLinear(1, dim_v, chan)
        self.L2, self.R2 = TensLinear(2, dim_d, chan), TensLinear(2, dim_d, chan)
        for name in ("000", "110", "220"):
            setattr(self, "Y_" + name, TensLinear(0, chan, dim_a))
        for name in V_ORDER:
            setattr(self, "Y_" + name, TensLinear(1, chan, dim_v))
        for name in D_ORDER:
            setattr(self, "Y_" + name, TensLinear(2, chan, dim_d))
        self.gn_a = TensGroupNorm(0, dim_a, groups)
        self.gn_v = TensGroupNorm(1, dim_v, groups)
        self.gn_d = TensGroupNorm(2, dim_d, groups)
        self.chan = chan
        self._cat, self._cat_key = None, None
        # bf16, chan = 128: the six channel mixings in front of the products and the products as one launch
        self.front_one_launch = True

    def _cat_weights(self):
        """left|right weights stacked per rank and the Y maps concatenated along their inputs (cached)"""
        key = tuple((p.data_ptr(), p._version) for p in self.parameters()) + (self.L0.precision,)
        if self._cat_key != key:
            f = lambda t: t.detach().float().contiguous()
            c = {"LR0": f(torch.cat([self.L0.W, self.R0.W], dim=0)), "LR1": f(torch.cat([self.L1.W, self.R1.W], dim=0)),
                 "LR2": f(torch.cat([self.L2.W, self.R2.W], dim=0)),
                 "Ya": f(torch.cat([self.Y_000.W, self.Y_110.W, self.Y_220.W], dim=1)),
                 "Yv": f(torch.cat([getattr(self, "Y_" + n).W for n in V_ORDER], dim=1)),
                 "Yd": f(torch.cat([getattr(self, "Y_" + n).W for n in D_ORDER], dim=1))}
            if self.L0.precision == "bf16":
                for k in list(c):
                    c[k + "p"] = ops.pack_weights_bf16(c[k])
            self._cat, self._cat_key = c, key
        return self._cat

    def _mix(self, c, name, inds, x):
        W = c[name]
        if name + "p" in c and W.shape[0] % 32 == 0 and W.shape[0] <= 512:
            return ops.linear_bf16_tc(x, c[name + "p"], W.shape[0], None, ops.ACT_NONE, inds=inds)
        return ops.tensor_linear_fwd(inds, W, x.contiguous())

    def cm_ready(self):
        c = self._cat_weights() if self.L0.precision == "bf16" else {}
        return (self.L0.precision == "bf16" and self.chan % 32 == 0 and 2 * self.chan <= 512
                and all(n + "p" in c and c[n].shape[0] % 32 == 0 and c[n].shape[1] % 4 == 0 for n in ("LR0", "LR1", "LR2", "Ya", "Yv", "Yd")))

    def forward_cm(self, x_a, x_v, x_d):
        """forward for component-major activations x_v [B, N, 3, dim_v], x_d [B, N, 9, dim_d] (results in the same form):
        all six channel mixings run on plain rows."""
        batch, nodes = x_a.shape[0], x_a.shape[1]
        n = batch * nodes
        c = self._cat_weights()
        lin = lambda name, x: ops.linear_bf16_tc(x, c[name + "p"], c[name].shape[0], None, ops.ACT_NONE, inds=0)
        lr0 = lin("LR0", x_a.reshape(n, -1))
        lr1 = lin("LR1", x_v.reshape(n * 3, -1)).reshape(n, 3, -1)
        lr2 = lin("LR2", x_d.reshape(n * 9, -1)).reshape(n, 9, -1)
        P_a, P_v, P_d = ops.bee_self_products_cm(lr0, lr1, lr2)
        y_a = lin("Ya", P_a)
        y_v = ops.linear_bf16_tc_rows16(P_v, c["Yvp"], c["Yv"].shape[0])
        y_d = ops.linear_bf16_tc_rows16(P_d, c["Ydp"], c["Yd"].shape[0])
        return (self.gn_a(y_a.reshape(batch, nodes, -1)),
                ops.group_norm_cm(y_v.reshape(batch, nodes, 3, -1), self.gn_v.groups, self.gn_v.epsilon, self.gn_v.gamma),
                ops.group_norm_cm(y_d.reshape(batch, nodes, 9, -1), self.gn_d.groups, self.gn_d.epsilon, self.gn_d.gamma))

    def forward(self, x_a, x_v, x_d, add_input=False):
        """add_input: returns the inputs plus the normalised products (the residual form the layers use), added inside the
        group norms' second pass on the fused path"""
        rest = x_a.shape[:-1]
        n = 1
        for d in rest:
            n *= d
        xa, xv, xd = x_a.reshape(n, -1), x_v.reshape(n, -1, 3), x_d.reshape(n, -1, 3, 3)
        if not torch.is_grad_enabled() and x_a.is_cuda and self.chan % 32 == 0:
            # three channel mixings in (left|right stacked), one product kernel, three channel mixings out
            c = self._cat_weights()
            tc_out = all(n + "p" in c and c[n].shape[0] % 32 == 0 for n in ("Yv", "Yd"))  # BF16 products for tcgen05 Y maps
            da, dv, dd = xa.shape[1], xv.shape[1], xd.shape[1]
            if (tc_out and self.front_one_launch and "LR0p" in c and self.chan == 128 and da % 16 == 0 and dv % 16 == 0
                    and dd % 16 == 0 and da + 3 * dv + 9 * dd <= 640 and all(t.dtype == torch.float32 for t in (xa, xv, xd))):
                # the six channel mixings and the products in one launch: the mixed features never leave the SM
                dev, C = xa.device, self.chan
                P_a = torch.empty(n, 3 * C, dtype=torch.float32, device=dev)
                P_v = torch.empty(n, 3, 5 * C, dtype=torch.bfloat16, device=dev)
                P_d = torch.empty(n, 9, 5 * C, dtype=torch.bfloat16, device=dev)
                with KERNEL_TIMER.region("bee_self_products"):
                    check(lib().ld_bee_self_front_bf16_tc(ptr(xa.contiguous()), ptr(xv.contiguous()), ptr(xd.contiguous()), n, da, dv, dd,
                                                          C, ptr(c["LR0p"]), ptr(c["LR1p"]), ptr(c["LR2p"]), ptr(P_a), ptr(P_v), ptr(P_d),
                                                          ptr(ops.tc_status(dev)), stream_ptr(dev)))
            else:
                P_a, P_v, P_d = ops.bee_self_products(self._mix(c, "LR0", 0, xa), self._mix(c, "LR1", 1, xv), self._mix(c, "LR2", 2, xd),
                                                      out_bf16=tc_out)
            y_a = self._mix(c, "Ya", 0, P_a)
            if tc_out:
                y_v = ops.linear_bf16_tc_cm(P_v, c["Yvp"], c["Yv"].shape[0], 1)
                y_d = ops.linear_bf16_tc_cm(P_d, c["Ydp"], c["Yd"].shape[0], 2)
            else:
                y_v, y_d = self._mix(c, "Yv", 1, P_v), self._mix(c, "Yd", 2, P_d)
            if add_input and len(rest) == 2:
                return (self.gn_a(y_a.reshape(*rest, -1), residual=x_a), self.gn_v(y_v.reshape(*rest, -1, 3), residual=x_v),
                        self.gn_d(y_d.reshape(*rest, -1, 3, 3), residual=x_d))
            out = (self.gn_a(y_a.reshape(*rest, -1)), self.gn_v(y_v.reshape(*rest, -1, 3)), self.gn_d(y_d.reshape(*rest, -1, 3, 3)))
            return (x_a + out[0], x_v + out[1], x_d + out[2]) if add_input else out
        y = Bee.apply(self.L0(xa), self.L1(xv), self.L2(xd), self.R0(xa), self.R1(xv), self.R2(xd))
        (y_000, y_110, y_220, y_011, y_101, y_121, y_211, y_022, y_202, y_112, y_222, y_111, y_212) = y
        y_a = self.Y_000(y_000) + self.Y_110(y_110) + self.Y_220(y_220)
        y_v = self.Y_011(y_011) + self.Y_101(y_101) + self.Y_121(y_121) + self.Y_211(y_211) + self.Y_111(y_111)
        y_d = self.Y_022(y_022) + self.Y_202(y_202) + self.Y_112(y_112) + self.Y_222(y_222) + self.Y_212(y_212)
        out = (self.gn_a(y_a.reshape(*rest, -1)), self.gn_v(y_v.reshape(*rest, -1, 3)), self.gn_d(y_d.reshape(*rest, -1, 3, 3)))
        return (x_a + out[0], x_v + out[1], x_d + out[2]) if add_input else out


class BeeBlock(nn.Module):
    """One l<=2 layer: neighbour messages then node-local products, both residual."""

    def __init__(self, r0, dim_a, dim_v, dim_d, chan):
        super().__init__()
        self.messages = Messages(r0, dim_a, dim_v, dim_d, chan)
        self.prods = SelfTensProds(dim_a, dim_v, dim_d, chan)

    def forward(self, graph, r_ij, x_a, x_v, x_d):
        x_a, x_v, x_d = self.messages(graph, r_ij, x_a, x_v, x_d, add_input=True)
        return self.prods(x_a, x_v, x_d, add_input=True)

    def cm_ready(self):
        return self.messages.cm_ready() and not self.messages.fused_kernel and self.prods.cm_ready()

    def forward_cm(self, graph, r_ij, x_a, x_v, x_d):
        """the same layer on component-major activations (x_v [B, N, 3, dim_v], x_d [B, N, 9, dim_d])"""
        d_a, d_v, d_d = self.messages.forward_cm(graph, r_ij, x_a, x_v, x_d)
        x_a, x_v, x_d = x_a + d_a, x_v + d_v, x_d + d_d
        d_a, d_v, d_d = self.prods.forward_cm(x_a, x_v, x_d)
        return x_a + d_a, x_v + d_v, x_d + d_d


class BeeDenoiser(nn.Module):
    """Meanflow-style denoiser with scalar, vector and rank-2 channels: the model the benchmark
    configs 2 and 4 describe (type embedding -> `depth` l<=2 layers on the radius graph of the
    noised positions -> vector read-out), built from the reference's Messages / SelfTensProds
    layers (archs/diffuser_atoms15.py) and the read-in / read-out of archs/meanflow_painn8.py:185-217."""

    def __init__(self, r0, dim_a, dim_v, dim_d, chan, ntypes, depth):
        super().__init__()
        self.r0, self.dim_d = r0, dim_d
        self.type_embed = nn.Embedding(ntypes, dim_a)
        self.v_readin = TensLinear(1, 1, dim_v)
        self.blocks = nn.ModuleList([BeeBlock(r0, dim_a, dim_v, dim_d, chan) for _ in range(depth)])
        self.readout = TensLinear(1, dim_v, 1)
        self.graph_cache = None   # set by painn.enable_rollout_graphs: fixed-capacity graph buffers for rollouts
        # True: between the layers the vector / rank-2 features are kept as [B, N, 3 | 9, chan] (every channel mixing reads
        # and writes plain rows). Same results; measured 2 % slower than the [.., chan, 3^l] form with the present
        # tensor-core linear (its epilogue for plain rows goes through shared memory), so it is off by default.
        self.component_major = False

    def forward(self, x0, x1, box, types, counter=None):
        from .graph_layers import Graph
        batch, nodes, _ = x0.shape
        graph = Graph.radius_graph(self.r0, box, x1.contiguous(), cache=self.graph_cache)
        x_a = self.type_embed(types)[None].expand(batch, -1, -1).contiguous()
        x_v = self.v_readin((x1 - x0)[..., None, :].contiguous())
        if self.component_major and not torch.is_grad_enabled() and x0.is_cuda and all(blk.cm_ready() for blk in self.blocks):
            # between the layers the vector / rank-2 features stay component-major ([B, N, 3 | 9, chan]): every channel
            # mixing then reads and writes plain rows; converted only here and at the read-out
            x_v = x_v.transpose(-1, -2).contiguous()
            x_d = torch.zeros(batch, nodes, 9, self.dim_d, device=x0.device)
            for blk in self.blocks:
                x_a, x_v, x_d = blk.forward_cm(graph, graph.rij, x_a, x_v, x_d)
            if counter is not None:
                graph.count_edges(counter, len(self.blocks))
            return torch.matmul(x_v, self.readout.W.t()).squeeze(-1)
        x_d = torch.zeros(batch, nodes, self.dim_d, 3, 3, device=x0.device)
        for blk in self.blocks:
            x_a, x_v, x_d = blk(graph, graph.rij, x_a, x_v, x_d)
        if counter is not None:
            graph.count_edges(counter, len(self.blocks))
        return self.readout(x_v).squeeze(-2)

    @torch.no_grad()
    def generate(self, x_0, noise, sigma_0, box, types, counter=None):
        z_1 = x_0 + sigma_0 * noise
        out = z_1 - self.forward(x_0, z_1, box, types, counter)
        ops.check_tc_status(x_0.device, block=False)   # a kernel that gave up on a wait is reported, not passed on
        return out
