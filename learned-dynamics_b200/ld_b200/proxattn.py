"""Host-side mirror of the reference's dense proximity-attention operators
(managan/triton_kernels/proxattn.py:239-311 `proxattn`, managan/triton_kernels/proxattn_periodic.py
`proxattn`): same argument order, shapes and restrictions (dim in {16, 32, 64, 128}, every tensor
contiguous and on the GPU, Z a multiple of the number of heads), with gradients for Q, K, V, X and
Y and none for r0sq (and none for the box).

    proxattn(Q, K, V, X, Y, r0sq)               -> out (Z, N, dim)
    proxattn_periodic(Q, K, V, X, Y, r0sq, box) -> out (Z, N, dim), box = (Lx, Ly, Lz)

precision="fp32" (default): the FP32 kernels ld_proxattn_fwd / ld_proxattn_bwd, 2e-5 against the einsum
definition. precision="tf32": the forward runs on the tensor cores (ld_proxattn_fwd_tf32_tc, the precision of
the reference's Triton kernel, about 1e-3); the backward stays FP32."""
import torch

from ._lib import lib, check, ptr, stream_ptr, require_cuda_f32, KERNEL_TIMER
from .ops import tc_status


def _check(Q, K, V, X, Y, r0sq):
    for name, t in (("Q", Q), ("K", K), ("V", V), ("X", X), ("Y", Y), ("r0sq", r0sq)):
        require_cuda_f32(t, name)
        if not t.is_contiguous():
            raise RuntimeError(f"proxattn: {name} must be contiguous")
    if Q.dim() != 3:
        raise RuntimeError("proxattn: Q must be (Z, N, dim)")
    Z, N, dim = Q.shape
    if tuple(K.shape) != (Z, N, dim) or tuple(V.shape) != (Z, N, dim):
        raise RuntimeError("proxattn: K and V must have Q's shape")
    if tuple(X.shape) != (Z, N, 3) or tuple(Y.shape) != (Z, N, 3):
        raise RuntimeError("proxattn: X and Y must be (Z, N, 3)")
    if dim not in (16, 32, 64, 128):
        raise RuntimeError("proxattn: dim must be one of 16, 32, 64, 128")
    if r0sq.dim() != 1 or Z % r0sq.shape[0] != 0:
        raise RuntimeError("proxattn: Z must be a multiple of the number of heads")
    return Z, N, dim, r0sq.shape[0]


def _box_args(box):
    if box is None:
        return 0, 0.0, 0.0, 0.0
    bx, by, bz = (float(b) for b in box)
    return 1, bx, by, bz


class _ProxAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, X, Y, r0sq, box, precision):
        Z, N, dim, heads = _check(Q, K, V, X, Y, r0sq)
        if precision not in ("fp32", "tf32"):
            raise RuntimeError("proxattn: precision must be 'fp32' or 'tf32'")
        out = torch.empty_like(Q)
        with KERNEL_TIMER.region("proxattn_fwd"):
            if precision == "tf32":
                check(lib().ld_proxattn_fwd_tf32_tc(ptr(Q), ptr(K), ptr(V), ptr(X), ptr(Y), ptr(r0sq), heads, Z, N, dim,
                                                    *_box_args(box), ptr(out), ptr(tc_status(Q.device)), stream_ptr(Q.device)))
            else:
                check(lib().ld_proxattn_fwd(ptr(Q), ptr(K), ptr(V), ptr(X), ptr(Y), ptr(r0sq), heads, Z, N, dim,
                                            *_box_args(box), ptr(out), stream_ptr(Q.device)))
        ctx.save_for_backward(Q, K, V, X, Y, r0sq)
        ctx.box = box
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_out):
        Q, K, V, X, Y, r0sq = ctx.saved_tensors
        Z, N, dim = Q.shape
        d_out = d_out.contiguous()
        dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
        dX, dY = torch.empty_like(X), torch.empty_like(Y)
        with KERNEL_TIMER.region("proxattn_bwd"):
            check(lib().ld_proxattn_bwd(ptr(Q), ptr(K), ptr(V), ptr(X), ptr(Y), ptr(r0sq), r0sq.shape[0], Z, N, dim,
                                        *_box_args(ctx.box), ptr(d_out), ptr(dQ), ptr(dK), ptr(dV), ptr(dX), ptr(dY),
                                        stream_ptr(Q.device)))
        return dQ, dK, dV, dX, dY, None, None, None


def proxattn(Q, K, V, X, Y, r0sq, precision="fp32"):
    return _ProxAttn.apply(Q, K, V, X, Y, r0sq, None, precision)


def proxattn_periodic(Q, K, V, X, Y, r0sq, box, precision="fp32"):
    if isinstance(box, torch.Tensor):
        box = tuple(box.tolist())
    return _ProxAttn.apply(Q, K, V, X, Y, r0sq, tuple(box), precision)
