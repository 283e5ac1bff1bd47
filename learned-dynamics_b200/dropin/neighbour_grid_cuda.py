"""Drop-in for the reference's `neighbour_grid_cuda` extension module
(extensions/neighbour_grid/neighbour_grid.cpp:198-203): same function names, positional
signatures, dtypes and error texts, backed by libld_hotpath.so.

Put this directory and its parent on PYTHONPATH in place of the reference's built extension.
MODE selects the cell grid: 0 (default) finds every pair within the cutoff; 1 reproduces the
reference's ceil(box/cutoff) grid including the pairs it misses."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ld_b200 import graph as _graph  # noqa: E402
from ld_b200._lib import lib as _lib, check as _check, ptr as _ptr, stream_ptr as _stream_ptr, LD_FLAG_CAPACITY  # noqa: E402

MODE = int(os.environ.get("LD_NEIGHBOUR_MODE", "0"))


def _check_input(x, name="x"):
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _check_listmax(listmax):
    if listmax not in (32, 64, 128, 256):
        raise RuntimeError("expected listmax to be one of 32, 64, 128, 256. other values not supported!")


def _build(cutoff, box, x, want_rij=False):
    _check_input(x)
    if x.dim() != 3 or x.shape[2] != 3:
        raise RuntimeError("x must have shape (batch, nodes, 3)")
    batch, nodes, _ = x.shape
    b = _graph.RadiusGraphBuilder(batch, nodes, cutoff, box, mode=MODE, device=x.device)
    return b, b.build(x.float(), want_rij=want_rij)


def get_edges(listmax, neighboursmax, cutoff, box_x, box_y, box_z, x):
    """-> (src int32 [E], dst int32 [E], edgeCounts int32 [batch], cumulative).
    listmax / neighboursmax are accepted for compatibility; the CSR build has no per-cell or
    per-node capacity, so the reference's overflow errors cannot occur."""
    _check_listmax(listmax)
    _, g = _build(cutoff, (box_x, box_y, box_z), x)
    return g["src"], g["dst"], g["edge_counts"]


def get_neighbours(listmax, neighboursmax, cutoff, box_x, box_y, box_z, x):
    """-> (neighbourLists int32 [batch, nodes, neighboursmax], neighbourCounts int32 [batch, nodes]).
    Entries past a node's count are unspecified in the reference; here they are 0."""
    _check_listmax(listmax)
    b, g = _build(cutoff, (box_x, box_y, box_z), x)
    batch, nodes, _ = x.shape
    lists = torch.empty(batch, nodes, neighboursmax, dtype=torch.int32, device=x.device)
    counts = torch.empty(batch, nodes, dtype=torch.int32, device=x.device)
    b.status.zero_()
    _check(_lib().ld_neighbour_lists_from_csr(_ptr(g["row_ptr"]), _ptr(g["dst"]), batch, nodes, int(neighboursmax), _ptr(lists),
                                             _ptr(counts), _ptr(b.status), _stream_ptr(x.device)))
    if int(b.status.item()) & LD_FLAG_CAPACITY:
        raise RuntimeError("Neighbour list overflow occurred. Try increasing neighboursmax.")
    return lists, counts


def _check_padded(neighbourCounts, neighbours, x, xdim):
    for t, n in ((neighbourCounts, "neighbourCounts"), (neighbours, "neighbours"), (x, "x")):
        _check_input(t, n)
    if neighbourCounts.dim() != 2:
        raise RuntimeError("neighbourCounts must have shape (batch, nodes)")
    if neighbours.dim() != 3:
        raise RuntimeError("neighbours must have shape (batch, nodes, neighboursmax)")
    if x.dim() != xdim:
        raise RuntimeError("x must have shape (batch, nodes, chan)" if xdim == 3 else
                           "x must have shape (batch, nodes, neighboursmax, chan)")
    batch, nodes = neighbourCounts.shape
    if not (batch == neighbours.shape[0] == x.shape[0]):
        raise RuntimeError("batch dimension of all tensors must match")
    if not (nodes == neighbours.shape[1] == x.shape[1]):
        raise RuntimeError("node dimension of all tensors must match")
    if neighbourCounts.dtype != torch.int32 or neighbours.dtype != torch.int32 or x.dtype != torch.float32:
        raise RuntimeError("expected int32 neighbourCounts and neighbours, float32 x")
    return batch, nodes, neighbours.shape[2]


def edges_read(neighbourCounts, neighbours, x):
    """Legacy dense padded gather -> [batch, nodes, neighboursmax, chan], zero past the count
    (neighbour_grid.cpp:105-134)."""
    batch, nodes, nmax = _check_padded(neighbourCounts, neighbours, x, 3)
    chan = x.shape[2]
    out = torch.empty(batch, nodes, nmax, chan, dtype=torch.float32, device=x.device)
    _check(_lib().ld_edges_read_padded(_ptr(neighbours), _ptr(neighbourCounts), _ptr(x), batch, nodes, nmax, chan, _ptr(out),
                                      _stream_ptr(x.device)))
    return out


def edges_reduce(neighbourCounts, neighbours, x):
    """Legacy dense padded sum over the neighbour axis -> [batch, nodes, chan] (neighbour_grid.cpp:136-168)."""
    batch, nodes, nmax = _check_padded(neighbourCounts, neighbours, x, 4)
    if nmax != x.shape[2]:
        raise RuntimeError("neighboursmax dimension must match between neighbours and x")
    chan = x.shape[3]
    out = torch.empty(batch, nodes, chan, dtype=torch.float32, device=x.device)
    _check(_lib().ld_edges_reduce_padded(_ptr(neighbourCounts), _ptr(x), batch, nodes, nmax, chan, _ptr(out),
                                        _stream_ptr(x.device)))
    return out
