"""Drop-in for the reference's `codegen_tensops_cuda` module
(extensions/codegen_tensops/codegen_tensops.cpp:610-2011): the Bee, Cow and Ant16 entry points with
the same names, argument order and output order (every function returns a list of tensors)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ld_b200 import ops as _ops  # noqa: E402
from ld_b200 import ant16 as _ant16  # noqa: E402


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


def _ant16_entry(name, fn):
    def f(*args):
        return fn(*args)
    f.__name__ = name
    f.__doc__ = fn.__doc__
    return f


for _o in ("o0", "o1", "o2", "oc"):
    for _suffix in ("", "_backward", "_backleft", "_wtsback"):
        _n = f"ant16_{_o}{_suffix}_cuda"
        globals()[_n] = _ant16_entry(_n, getattr(_ant16, f"ant16_{_o}{_suffix}"))
