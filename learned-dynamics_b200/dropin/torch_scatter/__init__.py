"""Drop-in for the one torch_scatter entry point the reference uses: segment_coo(src, index,
dim_size=...) with sorted `index` and sum reduction (call site managan/graph_layers.py:54-59)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from ld_b200 import graph as _graph  # noqa: E402
from ld_b200.graph_layers import _GatherFn  # noqa: E402


class _SegmentCoo(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, index, dim_size):
        row_ptr = _graph.row_ptr_from_src(index, dim_size)
        ctx.save_for_backward(index)
        return _graph.segment_sum(x, row_ptr, dim_size)

    @staticmethod
    def backward(ctx, grad):
        index, = ctx.saved_tensors  # gather through an autograd function: differentiable again
        return _GatherFn.apply(grad.contiguous(), index.to(torch.int32), index.to(torch.int64)), None, None


def segment_coo(src, index, out=None, dim_size=None, reduce="sum"):
    if reduce != "sum" or out is not None:
        raise NotImplementedError("segment_coo drop-in: only reduce='sum' without `out`")
    if dim_size is None:
        dim_size = int(index.max().item()) + 1 if index.numel() else 0
    return _SegmentCoo.apply(src, index, dim_size)
