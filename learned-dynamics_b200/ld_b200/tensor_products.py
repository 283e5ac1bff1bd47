"""Host-side mirror of the hot-path pieces of managan/tensor_products.py: TensLinear (:26-37),
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

    def forward(self, x):
        batch, nodes = x.shape[0], x.shape[1]
        xg = x.reshape(batch, nodes, self.groups, -1, 3 ** self.inds)
        moment2 = (xg ** 2).sum(-1, keepdim=True).mean([1, 3], keepdim=True)
        ans = xg / torch.sqrt(self.epsilon + moment2)
        return self.gamma * ans.reshape(batch, nodes, self.chan, *[3] * self.inds)
