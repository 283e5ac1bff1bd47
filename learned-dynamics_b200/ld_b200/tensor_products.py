"""Host-side mirror of the hot-path pieces of managan/tensor_products.py: TensLinear (:26-37), the
TensorProdBare / TensorProds / AVDFullTensorProds product modules (:91-123, :250-265),
tens_sigmoid (:167-182) and TensGroupNorm (:215-232). Parameter names and shapes match the
reference (W is [dim_out, dim_in]) so its state dicts load unchanged."""
import torch
import torch.nn as nn

from . import ops
from .ops import tensor_linear


class TensLinear(nn.Module):
    """Linear layer for rank-`inds` Cartesian tensor activations (..., chan, (3,)^inds)."""

    def __init__(self, inds, dim_in, dim_out):
        super().__init__()
        self.W = nn.Parameter(torch.empty(dim_out, dim_in))
        self.inds = inds
        self.precision = "fp32"  # "bf16": tcgen05 GEMM without autograd (2e-2 relative)
        self._packed, self._packed_key = None, None
        self.self_init()

    def self_init(self):
        _, fan_in = self.W.shape
        nn.init.normal_(self.W, std=fan_in ** -0.5)

    def _packed_for(self, ops_module):
        key = (self.W.data_ptr(), self.W._version)
        if self._packed_key != key:
            self._packed, self._packed_key = ops_module.pack_weights_bf16(self.W.detach().float()), key
        return self._packed

    def forward(self, x):
        if self.precision == "bf16" and not torch.is_grad_enabled() and x.is_cuda and self.W.shape[0] % 32 == 0 \
                and self.W.shape[0] <= 512:
            return ops.linear_bf16_tc(x, self._packed_for(ops), self.W.shape[0], None, ops.ACT_NONE, inds=self.inds)
        return tensor_linear(self.inds, self.W, x.contiguous())


def tens_sigmoid(inds, x):
    """x / sqrt(1 + |x|^2) with the norm over the trailing `inds` axes."""
    dims = tuple(-(1 + n) for n in range(inds))
    xx = (x ** 2).sum(dims, keepdim=True) if inds > 0 else x ** 2
    return x / torch.sqrt(1.0 + xx)


class TensGroupNorm(nn.Module):
    def __init__(self, inds, chan, groups, epsilon=1e-5):
        super().__init__()
        assert chan % groups == 0
        self.inds, self.chan, self.groups, self.epsilon = inds, chan, groups, epsilon
        self.gamma = nn.Parameter(torch.ones(chan, *[1] * inds))

    def forward(self, x, residual=None):
        """residual (shape of x): returns residual + norm(x) (one pass on the fused path)"""
        if not torch.is_grad_enabled() and x.is_cuda and x.dim() == 3 + self.inds and x.dtype == torch.float32:
            return ops.group_norm(x, self.groups, self.epsilon, self.gamma, None, center=False, residual=residual)
        batch, nodes = x.shape[0], x.shape[1]
        xg = x.reshape(batch, nodes, self.groups, -1, 3 ** self.inds)
        moment2 = (xg ** 2).sum(-1, keepdim=True).mean([1, 3], keepdim=True)
        ans = xg / torch.sqrt(self.epsilon + moment2)
        ans = self.gamma * ans.reshape(batch, nodes, self.chan, *[3] * self.inds)
        return ans if residual is None else residual + ans


class _BareProdFn(torch.autograd.Function):
    """Channel-wise product with trailing-index contraction; the two adjoints are the same kernel in its
    other modes."""

    @staticmethod
    def forward(ctx, ranks, x_l, x_r):
        from . import ant16
        x_l, x_r = x_l.contiguous(), x_r.contiguous()
        ctx.ranks = ranks
        ctx.save_for_backward(x_l, x_r)
        return ant16.tensor_prod_bare(0, *ranks, x_l, x_r)

    @staticmethod
    def backward(ctx, dy):
        from . import ant16
        x_l, x_r = ctx.saved_tensors
        dy = dy.contiguous()
        dl = ant16.tensor_prod_bare(1, *ctx.ranks, dy, x_r) if ctx.needs_input_grad[1] else None
        dr = ant16.tensor_prod_bare(2, *ctx.ranks, dy, x_l) if ctx.needs_input_grad[2] else None
        return None, dl, dr


class TensorProdBare(nn.Module):
    """managan/tensor_products.py:91-108: x_l[..., keep_l + c] * x_r[..., keep_r + c] -> [..., keep_l + keep_r]
    with c = (inds_l + inds_r - inds_o) / 2 trailing indices contracted; no linear maps around it."""

    def __init__(self, inds_l, inds_r, inds_o):
        super().__init__()
        twice = inds_l + inds_r - inds_o
        assert twice % 2 == 0, "parity mismatch"
        contracts = twice // 2
        assert 0 <= contracts <= min(inds_l, inds_r), \
            f"{contracts} contractions is out of range for {inds_l}, {inds_r} index tensors"
        self.ranks = (inds_l, inds_r, inds_o)

    def forward(self, x_l, x_r):
        shape_l, shape_r = x_l.shape[:x_l.dim() - self.ranks[0]], x_r.shape[:x_r.dim() - self.ranks[1]]
        if shape_l != shape_r:  # einsum broadcasting of the leading dims
            lead = torch.broadcast_shapes(shape_l, shape_r)
            x_l = x_l.expand(*lead, *x_l.shape[x_l.dim() - self.ranks[0]:])
            x_r = x_r.expand(*lead, *x_r.shape[x_r.dim() - self.ranks[1]:])
        return _BareProdFn.apply(self.ranks, x_l, x_r)


class TensorProds(nn.Module):
    """managan/tensor_products.py:111-123: lin_l, lin_r -> product -> lin_o."""

    def __init__(self, inds_l, inds_r, inds_o, dim_l, dim_r, dim_o, rank):
        super().__init__()
        self.prod = TensorProdBare(inds_l, inds_r, inds_o)
        self.lin_l = TensLinear(inds_l, dim_l, rank)
        self.lin_r = TensLinear(inds_r, dim_r, rank)
        self.lin_o = TensLinear(inds_o, rank, dim_o)

    def forward(self, x_l, x_r):
        return self.lin_o(self.prod(self.lin_l(x_l), self.lin_r(x_r)))


class AVDFullTensorProds(nn.Module):
    """managan/tensor_products.py:250-265: the eight products among scalar / vector / rank-2 activations."""

    def __init__(self, dim_a, dim_v, dim_d, rank):
        super().__init__()
        self.tp000 = TensorProds(0, 0, 0, dim_a, dim_a, dim_a, rank)
        self.tp101 = TensorProds(1, 0, 1, dim_v, dim_a, dim_v, rank)
        self.tp110 = TensorProds(1, 1, 0, dim_v, dim_v, dim_a, rank)
        self.tp112 = TensorProds(1, 1, 2, dim_v, dim_v, dim_d, rank)
        self.tp202 = TensorProds(2, 0, 2, dim_d, dim_a, dim_d, rank)
        self.tp211 = TensorProds(2, 1, 1, dim_d, dim_v, dim_v, rank)
        self.tp220 = TensorProds(2, 2, 0, dim_d, dim_d, dim_a, rank)
        self.tp222 = TensorProds(2, 2, 2, dim_d, dim_d, dim_d, rank)

    def forward(self, x_a, x_v, x_d):
        y_a = self.tp000(x_a, x_a) + self.tp110(x_v, x_v) + self.tp220(x_d, x_d)
        y_v = self.tp101(x_v, x_a) + self.tp211(x_d, x_v)
        y_d = self.tp112(x_v, x_v) + self.tp202(x_d, x_a) + self.tp222(x_d, x_d)
        return y_a, y_v, y_d
