"""Dense-weight l<=2 tensor products (the reference's Ant16 family) on the C ABI.

y_o[b, o, .] = sum_{l, r} P[o, l, r] * (left[b, l, .] (x) x_r[b, r, .]) for the thirteen products of
managan/codegen_tensor_products.py:112-133. Same entry points, argument order and output order as
codegen_tensops_cuda.ant16_{o0,o1,o2,oc}{,_backward,_backleft,_wtsback}_cuda
(extensions/codegen_tensops/codegen_tensops.cpp:610-1517).

Each direction is a channel-mixing GEMM with P viewed as [(o l), r] (the library's tensor_linear kernels)
plus one small coupling contraction (ld_ant16_*); rows are processed in chunks so the intermediate
U[b, (o l), 3^rank_r] stays bounded."""
import torch

from ._lib import lib, check, ptr, stream_ptr, require_cuda_f32, KERNEL_TIMER
from . import ops

# name -> (product id in the fixed order, rank of left, rank of the right operand x, rank of the output)
PRODUCTS = {"000": (0, 0, 0, 0), "110": (1, 1, 1, 0), "220": (2, 2, 2, 0), "011": (3, 0, 1, 1), "101": (4, 1, 0, 1),
            "121": (5, 1, 2, 1), "211": (6, 2, 1, 1), "022": (7, 0, 2, 2), "202": (8, 2, 0, 2), "112": (9, 1, 1, 2),
            "222": (10, 2, 2, 2), "111": (11, 1, 1, 1), "212": (12, 2, 1, 2)}
GROUPS = {"o0": ("000", "110", "220"), "o1": ("011", "101", "121", "211"), "o2": ("022", "202", "112", "222"),
          "oc": ("111", "212")}
SCRATCH_BYTES = 256 << 20  # bound on the intermediate U per chunk


def _sfx(rank):
    return (3,) * rank


def _check(name, t, batch, chan, rank):
    require_cuda_f32(t, name)
    want = (batch, chan) + _sfx(rank)
    if tuple(t.shape) != want:
        raise RuntimeError(f"{name}: expected shape {want}, got {tuple(t.shape)}")


def _check_P(name, P, dim_o=None, dim_l=None, dim_r=None):
    require_cuda_f32(P, name)
    if P.dim() != 3:
        raise RuntimeError(f"{name} has wrong number of axes")
    for axis, want in enumerate((dim_o, dim_l, dim_r)):
        if want is not None and P.shape[axis] != want:
            raise RuntimeError(f"{name}: expected axis {axis} to have size {want}")


def _chunks(rows, dim_o, dim_l, rank_r):
    per_row = dim_o * dim_l * 3 ** rank_r * 4
    step = max(1, SCRATCH_BYTES // per_row)
    for lo in range(0, rows, step):
        yield lo, min(rows, lo + step)


def _U(P, x, rank_r):
    """U[b, (o l), J] = sum_r P[o, l, r] x[b, r, J]"""
    dim_o, dim_l, dim_r = P.shape
    return ops.tensor_linear_fwd(rank_r, P.reshape(dim_o * dim_l, dim_r), x)


def product_fwd(name, x, P, left, y, accumulate):
    pid, rl, rr, ro = PRODUCTS[name]
    dim_o, dim_l, dim_r = P.shape
    rows = x.shape[0]
    st = stream_ptr(x.device)
    for lo, hi in _chunks(rows, dim_o, dim_l, rr):
        U = _U(P, x[lo:hi], rr)
        with KERNEL_TIMER.region("ant16_contract_left"):
            check(lib().ld_ant16_contract_left(pid, ptr(left[lo:hi]), ptr(U), hi - lo, dim_o, dim_l, ptr(y[lo:hi]),
                                               1 if accumulate else 0, st))


def product_backward(name, dy, P, left, dx, accumulate):
    """dx (+)= d/dx of the product, given the output gradient dy"""
    pid, rl, rr, ro = PRODUCTS[name]
    dim_o, dim_l, dim_r = P.shape
    rows = dy.shape[0]
    st = stream_ptr(dy.device)
    Pt = P.reshape(dim_o * dim_l, dim_r).t()  # strided view: tensor_linear takes the strides
    for lo, hi in _chunks(rows, dim_o, dim_l, rr):
        dU = torch.empty((hi - lo, dim_o * dim_l) + _sfx(rr), dtype=torch.float32, device=dy.device)
        with KERNEL_TIMER.region("ant16_expand"):
            check(lib().ld_ant16_expand(pid, ptr(left[lo:hi]), ptr(dy[lo:hi]), hi - lo, dim_o, dim_l, ptr(dU), st))
        part = ops.tensor_linear_fwd(rr, Pt, dU)
        if accumulate:
            dx[lo:hi] += part
        else:
            dx[lo:hi] = part


def product_backleft(name, x, dy, P):
    pid, rl, rr, ro = PRODUCTS[name]
    dim_o, dim_l, dim_r = P.shape
    rows = x.shape[0]
    st = stream_ptr(x.device)
    dleft = torch.empty((rows, dim_l) + _sfx(rl), dtype=torch.float32, device=x.device)
    for lo, hi in _chunks(rows, dim_o, dim_l, rr):
        U = _U(P, x[lo:hi], rr)
        with KERNEL_TIMER.region("ant16_contract_out"):
            check(lib().ld_ant16_contract_out(pid, ptr(U), ptr(dy[lo:hi]), hi - lo, dim_o, dim_l, ptr(dleft[lo:hi]), st))
    return dleft


def product_wtsback(name, x, dy, left):
    pid, rl, rr, ro = PRODUCTS[name]
    rows, dim_r = x.shape[0], x.shape[1]
    dim_o, dim_l = dy.shape[1], left.shape[1]
    st = stream_ptr(x.device)
    dP = torch.zeros(dim_o * dim_l, dim_r, dtype=torch.float32, device=x.device)
    for lo, hi in _chunks(rows, dim_o, dim_l, rr):
        dU = torch.empty((hi - lo, dim_o * dim_l) + _sfx(rr), dtype=torch.float32, device=x.device)
        with KERNEL_TIMER.region("ant16_expand"):
            check(lib().ld_ant16_expand(pid, ptr(left[lo:hi]), ptr(dy[lo:hi]), hi - lo, dim_o, dim_l, ptr(dU), st))
        dP += ops.tensor_linear_dw(rr, dU, x[lo:hi].contiguous(), dim_o * dim_l, dim_r)
    return dP.reshape(dim_o, dim_l, dim_r)


# ---- the sixteen entry points ------------------------------------------------------------------------

def _pairs(flat):
    """(P_a, left_a, P_b, left_b, ...) -> [(P_a, left_a), ...]"""
    return [(flat[i], flat[i + 1]) for i in range(0, len(flat), 2)]


def _xs_dict(x_0, x_1, x_2):
    return {0: x_0, 1: x_1, 2: x_2}


def _validate_fwd(group, xs, pl):
    batch = next(t for t in xs.values() if t is not None).shape[0]
    for r, t in xs.items():
        if t is not None:
            _check(f"x_{r}", t, batch, t.shape[1] if t.dim() > 1 else -1, r)
    dim_l = pl[0][0].shape[1] if pl[0][0].dim() == 3 else None
    for name, (P, left) in zip(GROUPS[group], pl):
        _, rl, rr, ro = PRODUCTS[name]
        _check_P(f"P_{name}", P, None, dim_l, xs[rr].shape[1])
        _check(f"left_{name}", left, batch, dim_l, rl)
    return batch


def _forward_group(group, xs, flat):
    pl = _pairs(flat)
    batch = _validate_fwd(group, xs, pl)
    outs = {}
    for name, (P, left) in zip(GROUPS[group], pl):
        _, rl, rr, ro = PRODUCTS[name]
        dim_o = P.shape[0]
        if ro in outs:
            if outs[ro].shape[1] != dim_o:
                raise RuntimeError(f"P_{name}: expected axis 0 to have size {outs[ro].shape[1]}")
            acc = True
        else:
            outs[ro] = torch.empty((batch, dim_o) + _sfx(ro), dtype=torch.float32, device=left.device)
            acc = False
        if batch > 0:
            product_fwd(name, xs[rr].contiguous(), P.contiguous(), left.contiguous(), outs[ro], acc)
    return [outs[k] for k in sorted(outs)]


def _backward_group(group, dys, flat, ranks_out):
    """dys: {rank_o: dy}; returns dx for every rank in ranks_out (zeros where no product of the group reads it)"""
    pl = _pairs(flat)
    batch = next(iter(dys.values())).shape[0]
    dims = {}
    for name, (P, left) in zip(GROUPS[group], pl):
        _, rl, rr, ro = PRODUCTS[name]
        _check_P(f"P_{name}", P, dys[ro].shape[1], None, None)
        _check(f"left_{name}", left, batch, P.shape[1], rl)
        dims.setdefault(rr, P.shape[2])
    dx, started = {}, set()
    for r in ranks_out:
        chan = dims.get(r, dys[r].shape[1] if r in dys else 0)
        dx[r] = torch.zeros((batch, chan) + _sfx(r), dtype=torch.float32, device=next(iter(dys.values())).device)
    if batch > 0:
        for name, (P, left) in zip(GROUPS[group], pl):
            _, rl, rr, ro = PRODUCTS[name]
            product_backward(name, dys[ro].contiguous(), P.contiguous(), left.contiguous(), dx[rr], rr in started)
            started.add(rr)
    return [dx[r] for r in ranks_out]


def _backleft_group(group, xs, dys, Ps):
    out = []
    for name, P in zip(GROUPS[group], Ps):
        _, rl, rr, ro = PRODUCTS[name]
        _check_P(f"P_{name}", P, dys[ro].shape[1], None, xs[rr].shape[1])
        out.append(product_backleft(name, xs[rr].contiguous(), dys[ro].contiguous(), P.contiguous()))
    return out


def _wtsback_group(group, xs, dys, lefts):
    out = []
    for name, left in zip(GROUPS[group], lefts):
        _, rl, rr, ro = PRODUCTS[name]
        _check(f"left_{name}", left, xs[rr].shape[0], left.shape[1], rl)
        out.append(product_wtsback(name, xs[rr].contiguous(), dys[ro].contiguous(), left.contiguous()))
    return out


def ant16_o0(x_0, x_1, x_2, *pl):
    return _forward_group("o0", _xs_dict(x_0, x_1, x_2), pl)


def ant16_o0_backward(dy_0, *pl):
    return _backward_group("o0", {0: dy_0}, pl, (0, 1, 2))


def ant16_o0_backleft(x_0, x_1, x_2, dy_0, *Ps):
    return _backleft_group("o0", _xs_dict(x_0, x_1, x_2), {0: dy_0}, Ps)


def ant16_o0_wtsback(x_0, x_1, x_2, dy_0, *lefts):
    return _wtsback_group("o0", _xs_dict(x_0, x_1, x_2), {0: dy_0}, lefts)


def ant16_o1(x_0, x_1, x_2, *pl):
    return _forward_group("o1", _xs_dict(x_0, x_1, x_2), pl)


def ant16_o1_backward(dy_1, *pl):
    return _backward_group("o1", {1: dy_1}, pl, (0, 1, 2))


def ant16_o1_backleft(x_0, x_1, x_2, dy_1, *Ps):
    return _backleft_group("o1", _xs_dict(x_0, x_1, x_2), {1: dy_1}, Ps)


def ant16_o1_wtsback(x_0, x_1, x_2, dy_1, *lefts):
    return _wtsback_group("o1", _xs_dict(x_0, x_1, x_2), {1: dy_1}, lefts)


def ant16_o2(x_0, x_1, x_2, *pl):
    return _forward_group("o2", _xs_dict(x_0, x_1, x_2), pl)


def ant16_o2_backward(dy_2, *pl):
    return _backward_group("o2", {2: dy_2}, pl, (0, 1, 2))


def ant16_o2_backleft(x_0, x_1, x_2, dy_2, *Ps):
    return _backleft_group("o2", _xs_dict(x_0, x_1, x_2), {2: dy_2}, Ps)


def ant16_o2_wtsback(x_0, x_1, x_2, dy_2, *lefts):
    return _wtsback_group("o2", _xs_dict(x_0, x_1, x_2), {2: dy_2}, lefts)


def ant16_oc(x_1, x_2, *pl):
    """the two chiral products (Levi-Civita couplings): returns y_1c, y_2c"""
    return _forward_group("oc", {0: None, 1: x_1, 2: x_2}, pl)


def ant16_oc_backward(dy_1, dy_2, *pl):
    """returns dx_1, dx_2; no chiral product reads x_2, so dx_2 is zero (the reference writes zeros too)"""
    return _backward_group("oc", {1: dy_1, 2: dy_2}, pl, (1, 2))


def ant16_oc_backleft(x_1, x_2, dy_1, dy_2, *Ps):
    return _backleft_group("oc", {0: None, 1: x_1, 2: x_2}, {1: dy_1, 2: dy_2}, Ps)


def ant16_oc_wtsback(x_1, x_2, dy_1, dy_2, *lefts):
    return _wtsback_group("oc", {0: None, 1: x_1, 2: x_2}, {1: dy_1, 2: dy_2}, lefts)


def tensor_prod_bare(mode, inds_l, inds_r, inds_o, a, b):
    """Channel-wise product with trailing-index contraction (einsum of managan/tensor_products.py:91-108).
    mode 0: (x_l, x_r) -> y; mode 1: (dy, x_r) -> dx_l; mode 2: (dy, x_l) -> dx_r."""
    require_cuda_f32(a, "a")
    require_cuda_f32(b, "b")
    ranks = {0: (inds_l, inds_r, inds_o), 1: (inds_o, inds_r, inds_l), 2: (inds_o, inds_l, inds_r)}[mode]
    lead = a.shape[:a.dim() - ranks[0]]
    if tuple(b.shape[:b.dim() - ranks[1]]) != tuple(lead):
        raise RuntimeError("tensor product operands differ in their leading (batch, channel) shape")
    for t, r in ((a, ranks[0]), (b, ranks[1])):
        if tuple(t.shape[t.dim() - r:]) != _sfx(r):
            raise RuntimeError("expected trailing tensor index dims of size 3")
    n = 1
    for d in lead:
        n *= d
    out = torch.empty(tuple(lead) + _sfx(ranks[2]), dtype=torch.float32, device=a.device)
    with KERNEL_TIMER.region("tensor_prod_bare"):
        check(lib().ld_tensor_prod_bare(mode, inds_l, inds_r, inds_o, ptr(a), ptr(b), n, ptr(out), stream_ptr(a.device)))
    return out
