"""The allocation-free graph build (scratch inside the library) against the ordinary two-call build
with a caller workspace, through the C ABI. Lives in its own file that sorts last so that a run
stopping at the first failure has already executed every other test; it also passes alone in a
fresh process (the first call on the device performs the address look-up)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_build(pos, cutoff, box):
    from ld_b200 import graph as G
    B, N, _ = pos.shape
    b = G.RadiusGraphBuilder(B, N, cutoff, box)
    return b.build(pos, want_shift=True, want_rij=True)


def _noalloc_build(pos, cutoff, box, capacity):
    """Only pre-existing tensors are passed in; the call itself must not allocate."""
    from ld_b200 import _lib
    L = _lib.lib()
    B, N, _ = pos.shape
    dev = pos.device
    row_ptr = torch.empty(B * N + 1, dtype=torch.int32, device=dev)
    counts = torch.empty(B, dtype=torch.int32, device=dev)
    src = torch.full((capacity,), -1, dtype=torch.int32, device=dev)
    dst = torch.full((capacity,), -1, dtype=torch.int32, device=dev)
    shift = torch.zeros(capacity, dtype=torch.int32, device=dev)
    rij = torch.zeros(capacity, 3, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    periodic = 0 if box is None else 1
    box_arr = (ctypes.c_float * 3)(*(box if box is not None else (0.0, 0.0, 0.0)))

    def call():
        return L.ld_radius_graph_build_noalloc(pos.data_ptr(), B, N, periodic, cutoff, ctypes.cast(box_arr, ctypes.c_void_p), 0, 0,
                                               row_ptr.data_ptr(), counts.data_ptr(), capacity, src.data_ptr(), dst.data_ptr(),
                                               shift.data_ptr(), rij.data_ptr(), status.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)

    # The first call on a device resolves the scratch array's address and makes the driver load the kernels, which may
    # take device memory once; the guarantee is about every call after that. torch's own counters cannot see a raw
    # cudaMalloc inside the library, so the driver's free-memory figure is compared (no torch allocation in between).
    call()
    torch.cuda.synchronize()
    status.zero_()
    free_before = torch.cuda.mem_get_info()[0]
    rc = call()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free build changed the device's free memory"
    return rc, row_ptr, counts, src, dst, shift, rij, status


def test_noalloc_build_matches_workspace_build_twice():
    gen = torch.Generator().manual_seed(31)
    cases = [((torch.rand(4, 3000, 3, generator=gen) * 12.0).cuda(), 2.0, (12.0, 12.0, 12.0)),
             (torch.cumsum(torch.randn(16, 256, 3, generator=gen) / 3 ** 0.5, dim=1).cuda(), 5.0, None)]
    # two calls in a row on the shared scratch: a periodic case, then an open-boundary case of another shape
    for pos, cutoff, box in cases:
        want = _reference_build(pos, cutoff, box)
        E = want["E"]
        rc, row_ptr, counts, src, dst, shift, rij, status = _noalloc_build(pos, cutoff, box, E + 64)
        assert rc == 0 and int(status.item()) == 0
        assert torch.equal(row_ptr, want["row_ptr"]) and torch.equal(counts, want["edge_counts"])
        # integer outputs bit-exact, displacements bit-identical (same kernels, same order)
        assert torch.equal(src[:E], want["src"]) and torch.equal(dst[:E], want["dst"])
        assert torch.equal(shift[:E], want["shift"]) and torch.equal(rij[:E], want["rij"])
        assert (src[E:] == -1).all()


def test_noalloc_build_refuses_oversized_problem_and_small_capacity():
    from ld_b200 import _lib
    pos = torch.rand(8, 40000, 3, device="cuda") * 60.0   # 320k nodes: beyond the built-in scratch
    rc, *_ = _noalloc_build(pos, 2.0, (60.0, 60.0, 60.0), 16)
    assert rc == _lib.LD_ERR_WORKSPACE
    assert b"8 MiB" in _lib.lib().ld_last_error()
    pos = torch.rand(1, 500, 3, device="cuda") * 5.0
    rc, row_ptr, counts, src, dst, shift, rij, status = _noalloc_build(pos, 1.5, (5.0, 5.0, 5.0), 10)
    assert rc == 0 and int(status.item()) & _lib.LD_FLAG_CAPACITY
    assert int(row_ptr[-1]) > 10
    # capacity 0: nothing can be written, but the edges that do not fit are still reported
    rc, row_ptr, counts, src, dst, shift, rij, status = _noalloc_build(pos, 1.5, (5.0, 5.0, 5.0), 0)
    assert rc == 0 and int(status.item()) & _lib.LD_FLAG_CAPACITY
