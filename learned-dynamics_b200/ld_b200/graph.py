"""Radius graph and edge<->node movement on top of the C ABI.

Host-side mirror of extensions/neighbour_grid (get_edges, neighbour_grid.cpp:170-195) and of the
graph helpers in managan/graph_layers.py:9-77 of the reference."""
import ctypes

import torch

from . import _lib
from ._lib import lib, check, ptr, stream_ptr, require_cuda_f32, KERNEL_TIMER

MODE_EXACT, MODE_REFERENCE = 0, 1


def _box_arg(box):
    if box is None:
        return 0, None, None
    arr = (ctypes.c_float * 3)(float(box[0]), float(box[1]), float(box[2]))
    return 1, arr, ctypes.cast(arr, ctypes.c_void_p)


class RadiusGraphBuilder:
    """Owns the workspace for repeated graph builds of one (batch, nodes, box, cutoff) shape."""

    def __init__(self, batch, nodes, cutoff, box=None, mode=MODE_EXACT, open_cells_cap=0, device="cuda"):
        self.batch, self.nodes, self.cutoff, self.mode = int(batch), int(nodes), float(cutoff), int(mode)
        self.box = None if box is None else tuple(float(b) for b in box)
        self.open_cells_cap = int(open_cells_cap)
        self.device = torch.device(device)
        self.periodic, self._box_arr, self._box_ptr = _box_arg(self.box)
        nbytes = ctypes.c_size_t(0)
        check(lib().ld_radius_graph_workspace_size(self.batch, self.nodes, self.periodic, self.cutoff, self._box_ptr,
                                                   self.mode, self.open_cells_cap, ctypes.byref(nbytes)))
        self.workspace = torch.empty(max(nbytes.value, 16), dtype=torch.uint8, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        Nt = self.batch * self.nodes
        self.row_ptr = torch.empty(Nt + 1, dtype=torch.int32, device=self.device)
        self.edge_counts = torch.empty(max(self.batch, 1), dtype=torch.int32, device=self.device)[: self.batch]

    def count(self, pos):
        require_cuda_f32(pos, "pos")
        if tuple(pos.shape) != (self.batch, self.nodes, 3):
            raise RuntimeError("x must have shape (batch, nodes, 3)")
        with KERNEL_TIMER.region("radius_graph_count", launches=13):
            check(lib().ld_radius_graph_count(ptr(pos), self.batch, self.nodes, self.periodic, self.cutoff, self._box_ptr,
                                              self.mode, self.open_cells_cap, ptr(self.workspace), self.workspace.numel(),
                                              ptr(self.row_ptr), ptr(self.edge_counts), ptr(self.status),
                                              stream_ptr(self.device)))

    def fill(self, pos, capacity, src, dst, shift=None, rij=None):
        with KERNEL_TIMER.region("radius_graph_fill"):
            check(lib().ld_radius_graph_fill(ptr(pos), self.batch, self.nodes, self.periodic, self.cutoff, self._box_ptr,
                                             self.mode, self.open_cells_cap, ptr(self.workspace), self.workspace.numel(),
                                             ptr(self.row_ptr), int(capacity), ptr(src), ptr(dst), ptr(shift), ptr(rij),
                                             ptr(self.status), stream_ptr(self.device)))

    def build(self, pos, want_shift=False, want_rij=True):
        """count -> read E (one 4-byte device->host copy) -> fill. Returns a dict of tensors."""
        self.status.zero_()
        self.count(pos)
        E = int(self.row_ptr[-1].item())
        dev = self.device
        src = torch.empty(E, dtype=torch.int32, device=dev)
        dst = torch.empty(E, dtype=torch.int32, device=dev)
        shift = torch.empty(E, dtype=torch.int32, device=dev) if want_shift else None
        rij = torch.empty(E, 3, dtype=torch.float32, device=dev) if want_rij else None
        self.fill(pos, E, src, dst, shift, rij)
        return {"src": src, "dst": dst, "shift": shift, "rij": rij, "row_ptr": self.row_ptr.clone(),
                "edge_counts": self.edge_counts.clone(), "E": E}

    def build_fixed(self, pos, capacity, src, dst, shift=None, rij=None):
        """No host synchronisation: edges beyond `capacity` raise LD_FLAG_CAPACITY in self.status."""
        self.count(pos)
        self.fill(pos, capacity, src, dst, shift, rij)


class RolloutGraphCache:
    """Edge buffers of a fixed capacity reused over the steps of a rollout, so that no step waits for the device to
    learn its edge count (the reference's get_edges reads it back with .item() on every build,
    neighbour_grid.cpp:180-194). The first build is the ordinary one and fixes the capacity at `margin` times its edge
    count. Later builds run count + fill back to back at that capacity; the kernels downstream take their ranges from
    row_ptr, so the unused tail of the buffers is never read. After every build the edge count and the status word
    are copied to pinned host memory without waiting; a later build looks at the copies that have arrived, grows the
    buffers when the count comes within 10 % of the capacity, and raises if a build did overflow (the steps since
    then are invalid and must be redone: use a larger margin)."""

    def __init__(self, margin=1.25):
        self.margin = float(margin)
        self.builder = None
        self.capacity = 0
        self.buffers = None
        self._host = None
        self._event = None

    def _allocate(self, capacity, device):
        self.capacity = int(capacity)
        self.buffers = (torch.empty(self.capacity, dtype=torch.int32, device=device),
                        torch.empty(self.capacity, dtype=torch.int32, device=device),
                        torch.empty(self.capacity, 3, dtype=torch.float32, device=device))

    def _poll(self, block=False):
        if self._event is None or not (block or self._event.query()):
            return
        if block:
            self._event.synchronize()
        edges, flags = int(self._host[0]), int(self._host[1])
        self._event = None
        if flags != 0:
            self.builder.status.zero_()
            if flags & _lib.LD_FLAG_CAPACITY:
                need = int(edges * self.margin) + 1024
                self._allocate(need, self.builder.device)
                raise _lib.HotpathError(_lib.LD_ERR_CAPACITY, f"a fixed-capacity graph build overflowed ({edges} edges); the buffers "
                                        f"were grown to {need}, the steps since that build must be redone")
            check_status_flags(torch.tensor([flags]))
        if edges * 1.1 > self.capacity:
            self._allocate(int(edges * self.margin) + 1024, self.builder.device)

    def build(self, r0, box, pos, mode=MODE_EXACT):
        batch, nodes, _ = pos.shape
        key = (batch, nodes, float(r0), None if box is None else tuple(float(b) for b in box), mode, pos.device)
        if self.builder is None or self._key != key:
            self.builder = RadiusGraphBuilder(batch, nodes, r0, box, mode=mode, device=pos.device)
            self._key = key
            g = self.builder.build(pos, want_rij=True)            # ordinary build: learns the edge count
            check_status_flags(self.builder.status)
            self._allocate(int(g["E"] * self.margin) + 1024, pos.device)
            self._host = torch.zeros(2, dtype=torch.int32).pin_memory()
            self._event = None
        else:
            self._poll()
        b = self.builder
        src, dst, rij = self.buffers
        b.build_fixed(pos, self.capacity, src, dst, None, rij)
        # edge count and status of this build, on their way to the host while the step goes on
        self._host[0:1].copy_(b.row_ptr[-1:], non_blocking=True)
        self._host[1:2].copy_(b.status, non_blocking=True)
        self._event = torch.cuda.Event()
        self._event.record(torch.cuda.current_stream(pos.device))
        return {"src": src, "dst": dst, "rij": rij, "row_ptr": b.row_ptr, "edge_counts": b.edge_counts,
                "num_edges": b.row_ptr[-1:]}

    def finish(self):
        """wait for the last build's report (end of a rollout): raises if it overflowed"""
        self._poll(block=True)


def unpack_shift(shift):
    """int32 packed lattice shift -> [E,3] int32"""
    s = shift.to(torch.int32)
    parts = [((s >> (8 * a)) & 0xFF) for a in range(3)]
    return torch.stack([torch.where(p >= 128, p - 256, p) for p in parts], dim=1)


def check_status_flags(status):
    flags = int(status.item())
    if flags & _lib.LD_FLAG_NONFINITE:
        raise RuntimeError("some positions are NaN!")
    if flags & _lib.LD_FLAG_CAPACITY:
        raise RuntimeError("Neighbour list overflow occurred. Try increasing the edge capacity.")
    if flags & _lib.LD_FLAG_OVERFLOW:
        raise RuntimeError("radius graph: more than 2^31-1 edges, or a lattice shift beyond 127 box lengths")
    if flags & _lib.LD_FLAG_TIMEOUT:
        raise RuntimeError("device-side wait ran out")


def row_ptr_from_src(src, num_nodes):
    """CSR offsets [num_nodes+1] from a sorted source-node array (int32 or int64)."""
    src = src.contiguous()
    row_ptr = torch.empty(num_nodes + 1, dtype=torch.int32, device=src.device)
    nbytes = 8 if src.dtype == torch.int64 else 4
    if src.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("index must be int32 or int64")
    check(lib().ld_row_ptr_from_sorted(ptr(src), nbytes, src.numel(), num_nodes, ptr(row_ptr), stream_ptr(src.device)))
    return row_ptr


def segment_sum(x_edge, row_ptr, num_nodes):
    x_edge = x_edge.contiguous()
    require_cuda_f32(x_edge, "x_edge")
    rest = tuple(x_edge.shape[1:])
    F = 1
    for d in rest:
        F *= d
    out = torch.empty((num_nodes,) + rest, dtype=torch.float32, device=x_edge.device)
    if F == 0:
        return out
    with KERNEL_TIMER.region("segment_sum"):
        check(lib().ld_segment_sum(ptr(x_edge), ptr(row_ptr), num_nodes, F, ptr(out), stream_ptr(x_edge.device)))
    return out


def gather_rows(x_node, idx):
    x_node = x_node.contiguous()
    require_cuda_f32(x_node, "x_node")
    idx = idx.contiguous()
    rest = tuple(x_node.shape[1:])
    F = 1
    for d in rest:
        F *= d
    E = idx.numel()
    out = torch.empty((E,) + rest, dtype=torch.float32, device=x_node.device)
    nbytes = 8 if idx.dtype == torch.int64 else 4
    with KERNEL_TIMER.region("gather_rows"):
        check(lib().ld_gather_rows(ptr(x_node), ptr(idx), nbytes, E, F, ptr(out), stream_ptr(x_node.device)))
    return out
