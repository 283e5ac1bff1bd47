"""Host-side mirror of managan/graph_layers.py (reference lines 9-77): Graph, radius_graph,
edges_read, edges_read_dst, edges_reduce_src, boxwrap, expand_graph - same names and argument
meaning - on the CUDA kernels of this library. int32 indices and the CSR offsets are kept beside
the int64 views the reference exposes, so fused kernels can use them without conversion."""
import torch

from . import graph as _g


class Graph:
    """Batch of graphs with the same node count; edges flat, src non-decreasing (reference :9-24)."""

    def __init__(self, src, dst, edge_indices, batch, nodes, row_ptr=None, rij=None, num_edges=None):
        self.src32 = src if src.dtype == torch.int32 and src.is_contiguous() else src.to(torch.int32).contiguous()
        self.dst32 = dst if dst.dtype == torch.int32 and dst.is_contiguous() else dst.to(torch.int32).contiguous()
        self._src64 = src if src.dtype == torch.int64 else None
        self._dst64 = dst if dst.dtype == torch.int64 else None
        self.edge_indices = edge_indices
        self.batch = batch
        self.nodes = nodes
        self._row_ptr = row_ptr
        self.rij = rij  # wrapped displacement per edge when built by radius_graph
        # fixed-capacity graphs (rollouts): the buffers are longer than the edge list and the count lives on the device
        self.num_edges_dev = num_edges

    def _trim(self, t):
        return t if self.num_edges_dev is None else t[: int(self.num_edges_dev.item())]

    @property
    def src(self):
        """int64 view, as the reference exposes (managan/graph_layers.py:19-20); made on first use"""
        if self._src64 is None:
            self._src64 = self._trim(self.src32).to(torch.int64)
        return self._src64

    @property
    def dst(self):
        if self._dst64 is None:
            self._dst64 = self._trim(self.dst32).to(torch.int64)
        return self._dst64

    def count_edges(self, counter, times=1):
        """counter (device int64[1]) += times * number of edges, without a host read"""
        if self.num_edges_dev is not None:
            counter += self.num_edges_dev.to(torch.int64) * times
        else:
            counter += self.src32.numel() * times

    @property
    def row_ptr(self):
        if self._row_ptr is None:
            self._row_ptr = _g.row_ptr_from_src(self.src32, self.batch * self.nodes)
        return self._row_ptr

    @staticmethod
    def radius_graph(r0, box, pos, celllist_max=32, neighbours_max=64, mode=_g.MODE_EXACT, cache=None):
        """Nodes within r0 are connected. box: (bx,by,bz) periodic, or None for open boundaries
        (the reference has periodic only). celllist_max / neighbours_max are accepted and unused:
        the CSR build has no capacities to overflow. cache: a graph.RolloutGraphCache; the build then reuses its
        buffers at a fixed capacity and does not wait for the device (inference loops only: src / dst are then longer
        than the edge list, row_ptr delimits it)."""
        batch, nodes, three = pos.shape
        assert three == 3
        if cache is not None and not torch.is_grad_enabled():
            g = cache.build(r0, box, pos.contiguous(), mode)
            ans = Graph(g["src"], g["dst"], g["edge_counts"], batch, nodes, row_ptr=g["row_ptr"], rij=g["rij"],
                        num_edges=g["num_edges"])
            ans.box = box
            return ans
        builder = _g.RadiusGraphBuilder(batch, nodes, r0, box, mode=mode, device=pos.device)
        g = builder.build(pos.contiguous(), want_rij=True)
        _g.check_status_flags(builder.status)  # NaN positions raise, as the reference's assert does
        ans = Graph(g["src"], g["dst"], g["edge_counts"], batch, nodes, row_ptr=g["row_ptr"], rij=g["rij"])
        ans.box = box
        return ans


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_flat, idx32, idx64):
        ctx.save_for_backward(idx64)
        ctx.n = x_flat.shape[0]
        return _g.gather_rows(x_flat, idx32)

    @staticmethod
    def backward(ctx, grad):
        idx64, = ctx.saved_tensors
        out = torch.zeros((ctx.n,) + tuple(grad.shape[1:]), dtype=grad.dtype, device=grad.device)
        out.index_add_(0, idx64, grad)
        return out, None, None


class _SegmentSumFn(torch.autograd.Function):
    """The gradient of the per-node sum is the gather by source node, taken through _GatherFn so that
    it can be differentiated again."""

    @staticmethod
    def forward(ctx, x_edge, row_ptr, src32, src64, n):
        ctx.save_for_backward(src32, src64)
        return _g.segment_sum(x_edge, row_ptr, n)

    @staticmethod
    def backward(ctx, grad):
        src32, src64 = ctx.saved_tensors
        return _GatherFn.apply(grad.contiguous(), src32, src64), None, None, None, None


def edges_read(graph, x_node):
    """x_node: (batch, nodes, ...) -> (x_src, x_dst), each (edges, ...)"""
    assert x_node.shape[0] == graph.batch and x_node.shape[1] == graph.nodes
    flat = x_node.reshape(graph.batch * graph.nodes, *x_node.shape[2:]).contiguous()
    return _GatherFn.apply(flat, graph.src32, graph.src), _GatherFn.apply(flat, graph.dst32, graph.dst)


def edges_read_dst(graph, x_node):
    assert x_node.shape[0] == graph.batch and x_node.shape[1] == graph.nodes
    flat = x_node.reshape(graph.batch * graph.nodes, *x_node.shape[2:]).contiguous()
    return _GatherFn.apply(flat, graph.dst32, graph.dst)


def edges_reduce_src(graph, x_edge):
    """sum edge data onto source nodes: (edges, ...) -> (batch, nodes, ...)"""
    n = graph.batch * graph.nodes
    ans = _SegmentSumFn.apply(x_edge.contiguous(), graph.row_ptr, graph.src32, graph.src, n)
    return ans.reshape(graph.batch, graph.nodes, *ans.shape[1:])


def boxwrap(box, delta_pos):
    """shortest periodic image of a displacement (reference :62-66)"""
    return (delta_pos + 0.5 * box) % box - 0.5 * box


def expand_graph(graph, new_batch):
    assert graph.batch == 1, "Graph to be expanded should have batch size 1"
    offs = graph.nodes * torch.arange(new_batch, device=graph.src.device)[:, None]
    src = (graph.src[None].expand(new_batch, -1) + offs).flatten()
    dst = (graph.dst[None].expand(new_batch, -1) + offs).flatten()
    return Graph(src, dst, None, new_batch, graph.nodes)
