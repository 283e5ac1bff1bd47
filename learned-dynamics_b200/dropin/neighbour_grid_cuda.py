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
    _, g = _build(cutoff, (box_x, box_y, box_z), x)
    batch, nodes, _ = x.shape
    row_ptr = g["row_ptr"].long()
    counts = (row_ptr[1:] - row_ptr[:-1]).to(torch.int32)
    if counts.numel() > 0 and int(counts.max().item()) > neighboursmax:
        raise RuntimeError("Neighbour list overflow occurred. Try increasing neighboursmax.")
    lists = torch.zeros(batch * nodes, neighboursmax, dtype=torch.int32, device=x.device)
    if g["E"] > 0:
        src = g["src"].long()
        slot = torch.arange(g["E"], device=x.device) - row_ptr[src]
        lists[src, slot] = (g["dst"].long() - (src // nodes) * nodes).to(torch.int32)
    return lists.reshape(batch, nodes, neighboursmax), counts.reshape(batch, nodes)


def edges_read(neighbourCounts, neighbours, x):
    """Legacy dense padded gather [batch, nodes, neighboursmax, chan] (zero past the count)."""
    for t, n in ((neighbourCounts, "neighbourCounts"), (neighbours, "neighbours"), (x, "x")):
        _check_input(t, n)
    if neighbourCounts.dim() != 2 or neighbours.dim() != 3 or x.dim() != 3:
        raise RuntimeError("expected neighbourCounts (batch, nodes), neighbours (batch, nodes, neighboursmax), x (batch, nodes, chan)")
    batch, nodes, nmax = neighbours.shape
    idx = neighbours.long() + (torch.arange(batch, device=x.device) * nodes)[:, None, None]
    out = x.reshape(batch * nodes, -1)[idx.reshape(-1)].reshape(batch, nodes, nmax, -1)
    mask = torch.arange(nmax, device=x.device)[None, None, :] < neighbourCounts[:, :, None]
    return out * mask[..., None]


def edges_reduce(neighbourCounts, neighbours, x):
    """Legacy dense padded sum over the neighbour axis -> [batch, nodes, chan]."""
    for t, n in ((neighbourCounts, "neighbourCounts"), (neighbours, "neighbours"), (x, "x")):
        _check_input(t, n)
    if x.dim() != 4:
        raise RuntimeError("x must have shape (batch, nodes, neighboursmax, chan)")
    nmax = x.shape[2]
    mask = torch.arange(nmax, device=x.device)[None, None, :] < neighbourCounts[:, :, None]
    return (x * mask[..., None]).sum(2)
