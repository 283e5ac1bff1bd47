"""Host-side mirror of the pieces of managan/layers_common.py that sit on the message-passing path:
VecLinear (:81-89), radial_encode (:122-126), ScalGroupNorm (:201-223), plus radial_encode_edge of
archs/diffuser_atoms5.py:25-30. Parameter names follow the reference so its state dicts load."""
import torch
import torch.nn as nn

from . import ops
from .painn import ScalGroupNorm  # noqa: F401  (the reference defines it in layers_common)
from .tensor_products import TensLinear


class VecLinear(TensLinear):
    """einsum("oi, ...ik -> ...ok", W, v): the rank-1 channel mixing under the name older archs use. Same parameter
    (`W` [dim_out, dim_in]) and the same kernels as TensLinear(1, dim_in, dim_out)."""

    def __init__(self, dim_in, dim_out):
        super().__init__(1, dim_in, dim_out)

    def self_init(self):
        nn.init.normal_(self.W, std=self.W.shape[1] ** -0.5)


def _encode(kind, r, n, rmax, vector=True):
    if not r.is_cuda or torch.is_grad_enabled() and r.requires_grad:
        return None
    rr = r.contiguous().float()
    rows = rr.numel() // (3 if vector else 1)
    out = torch.empty(tuple(rr.shape[:-1] if vector else rr.shape) + (n,), dtype=torch.float32, device=r.device)
    return ops.radial_encode(kind, rr, rows, n, rmax, out)


def radial_encode(r, n, rmax):
    """r: (...) -> (..., n): cos(pi * m * r), m = 0..n-1 (rmax is unused, as in the reference)"""
    out = _encode(ops.RADIAL_COS, r, n, rmax, vector=False)
    if out is not None:
        return out
    m = torch.arange(0, n, device=r.device)
    return torch.cos(torch.pi * m * r[..., None])


def radial_encode_edge(r, n, rmax):
    """r: (..., 3) -> (..., n): cos(m * pi * sqrt(|r|^2 / rmax)) * relu(1 - |r|^2 / rmax)"""
    out = _encode(ops.RADIAL_EDGE, r, n, rmax)
    if out is not None:
        return out
    npi = torch.pi * torch.arange(0, n, device=r.device)
    x_sq = (r ** 2).sum(-1) / rmax
    return torch.cos(npi * torch.sqrt(x_sq)[..., None]) * torch.relu(1. - x_sq)[..., None]
