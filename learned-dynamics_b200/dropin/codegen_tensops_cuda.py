"""Drop-in for the Bee and Cow entry points of the reference's `codegen_tensops_cuda` module
(extensions/codegen_tensops/codegen_tensops.cpp:1519-2011): same names, argument order and
output order. The Ant16 family is not provided yet and raises on use."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ld_b200 import ops as _ops  # noqa: E402


def set_kern_attributes():
    """The reference raises a shared-memory limit here; these kernels need no opt-in."""
    return None


def bee_fwd_cuda(l_0, l_1, l_2, r_0, r_1, r_2):
    return _ops.bee_fwd(l_0, l_1, l_2, r_0, r_1, r_2)


def bee_bwl_cuda(r_0, r_1, r_2, *dy):
    return _ops.bee_bw(True, r_0, r_1, r_2, dy)


def bee_bwr_cuda(l_0, l_1, l_2, *dy):
    return _ops.bee_bw(False, l_0, l_1, l_2, dy)


def cow_o0_fwd_cuda(l_0, l_1, r_0, r_1):
    return _ops.cow_o0_fwd(l_0, l_1, r_0, r_1)


def cow_o0_bwl_cuda(r_0, r_1, dy_000, dy_110):
    return _ops.cow_o0_bw(r_0, r_1, dy_000, dy_110)


def cow_o0_bwr_cuda(l_0, l_1, dy_000, dy_110):
    return _ops.cow_o0_bw(l_0, l_1, dy_000, dy_110)


def cow_o1_fwd_cuda(l_0, l_1, r_0, r_1):
    return _ops.cow_o1_fwd(l_0, l_1, r_0, r_1)


def cow_o1_bwl_cuda(r_0, r_1, dy_011, dy_101, dy_111):
    return _ops.cow_o1_bw(True, r_0, r_1, dy_011, dy_101, dy_111)


def cow_o1_bwr_cuda(l_0, l_1, dy_011, dy_101, dy_111):
    return _ops.cow_o1_bw(False, l_0, l_1, dy_011, dy_101, dy_111)


def _ant16_missing(name):
    def f(*a, **k):
        raise NotImplementedError(f"{name}: the Ant16 dense-P contraction kernels are not built in this library")
    f.__name__ = name
    return f


for _o in ("o0", "o1", "o2", "oc"):
    for _suffix in ("", "_backward", "_backleft", "_wtsback"):
        _n = f"ant16_{_o}{_suffix}_cuda"
        globals()[_n] = _ant16_missing(_n)
