"""Channel mixing, l<=2 tensor products, dense MLP rows and the fused PaiNN message, on the C ABI."""
import ctypes

import torch

from ._lib import lib, check, ptr, stream_ptr, require_cuda_f32, KERNEL_TIMER

ACT_NONE, ACT_SILU, ACT_LEAKY01 = 0, 1, 2
KERNEL_TIMER = KERNEL_TIMER  # re-exported for bench.py
RADIAL_PAINN, RADIAL_GAUSSIAN, RADIAL_EDGE, RADIAL_COS, RADIAL_JACOBI8 = 0, 1, 2, 3, 4

BEE_SUFFIX = ("", "", "", (3,), (3,), (3,), (3,), (3, 3), (3, 3), (3, 3), (3, 3), (3,), (3, 3))


def tensor_linear_fwd(inds, W, x):
    """y[..., o, s] = sum_i W[o, i] x[..., i, s]; W may be strided, x contiguous float32 CUDA."""
    if not W.is_cuda:
        raise RuntimeError("W must be a CUDA tensor")
    require_cuda_f32(x, "x")
    if W.dim() != 2:
        raise RuntimeError("expected W to be a matrix (2 dims)")
    if inds not in (0, 1, 2):
        raise RuntimeError("tensor_linear currently only supports a number of indices up to 2.")
    dim_out, dim_in = W.shape
    shape = list(x.shape)
    bd = len(shape) - (1 + inds)
    if bd < 0:
        raise RuntimeError("x has too few dims")
    if shape[bd] != dim_in:
        raise RuntimeError("channel dim size mismatch for x")
    for i in range(bd + 1, bd + 1 + inds):
        if shape[i] != 3:
            raise RuntimeError("expected tensor index dim to be 3d for input x")
    rows = 1
    for d in shape[:bd]:
        rows *= d
    shape[bd] = dim_out
    y = torch.empty(shape, dtype=torch.float32, device=x.device)
    if rows == 0:
        return y
    with KERNEL_TIMER.region("tensor_linear"):
        check(lib().ld_tensor_linear(inds, ptr(W), W.stride(0), W.stride(1), ptr(x), ptr(y), rows, dim_in, dim_out,
                                     stream_ptr(x.device)))
    return y


def tensor_linear_dw(inds, dy, x, dim_out, dim_in):
    rows = x.numel() // max(dim_in * 3 ** inds, 1)
    dW = torch.empty(dim_out, dim_in, dtype=torch.float32, device=x.device)
    nbytes = ctypes.c_size_t(0)
    check(lib().ld_tensor_linear_dw_workspace(inds, rows, dim_in, dim_out, ctypes.byref(nbytes)))
    ws = torch.empty(max(nbytes.value, 4), dtype=torch.uint8, device=x.device)
    check(lib().ld_tensor_linear_dw(inds, ptr(dy), ptr(x), ptr(dW), rows, dim_in, dim_out, ptr(ws), nbytes.value,
                                    stream_ptr(x.device)))
    return dW


class TensorLinearFn(torch.autograd.Function):
    """Same split as the reference's C++ autograd function (extensions/tensor_ops/tensor_ops.cpp:31-170):
    dx is the forward kernel on W transposed (swapped strides), dW is its own kernel. Unlike the
    reference, the backward is itself built from autograd functions, so gradients of any order exist
    (the double backward of torch.autograd.functional.jvp(create_graph=True), as the meanflow
    training step uses at archs/meanflow_painn8.py:274-282)."""

    @staticmethod
    def forward(ctx, inds, W, x):
        ctx.inds = inds
        ctx.save_for_backward(W, x)
        return tensor_linear_fwd(inds, W, x)

    @staticmethod
    def backward(ctx, dy):
        W, x = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dW = None
        if ctx.needs_input_grad[2]:
            dx = TensorLinearFn.apply(ctx.inds, W.t(), dy)
        if ctx.needs_input_grad[1]:
            dW = TensorLinearDwFn.apply(ctx.inds, dy, x)
        return None, dW, dx


class TensorLinearDwFn(torch.autograd.Function):
    """dW[o,i] = sum over rows and tensor components of dy[.,o,s] x[.,i,s]; its own gradients are two
    tensor_linear calls: d(dy) = G x, d(x) = G^T dy for an incoming G of W's shape."""

    @staticmethod
    def forward(ctx, inds, dy, x):
        ctx.inds = inds
        ctx.save_for_backward(dy, x)
        bd = x.dim() - (1 + inds)
        return tensor_linear_dw(inds, dy, x, dy.shape[bd], x.shape[bd])

    @staticmethod
    def backward(ctx, G):
        dy, x = ctx.saved_tensors
        G = G.contiguous()
        g_dy = g_x = None
        if ctx.needs_input_grad[1]:
            g_dy = TensorLinearFn.apply(ctx.inds, G, x)
        if ctx.needs_input_grad[2]:
            g_x = TensorLinearFn.apply(ctx.inds, G.t(), dy)
        return None, g_dy, g_x


def tensor_linear(inds, W, x):
    return TensorLinearFn.apply(inds, W, x)


def radial_encode(kind, r, rows, n, rmax, out, coeff=None):
    """out[rows, n] = radial encoding `kind` (RADIAL_*) of r[rows, 3] (r[rows] for RADIAL_COS)"""
    require_cuda_f32(r, "r")
    with KERNEL_TIMER.region("radial_encode"):
        check(lib().ld_radial_encode(kind, ptr(r), rows, n, float(rmax), ptr(coeff), ptr(out), stream_ptr(r.device)))
    return out


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


def _check_operands(names, tensors, ranks):
    batch, chan = None, None
    for name, t, r in zip(names, tensors, ranks):
        require_cuda_f32(t, name)
        if t.dim() != 2 + r:
            raise RuntimeError(f"{name} has wrong number of axes")
        if batch is None:
            batch, chan = t.shape[0], t.shape[1]
        if t.shape[0] != batch:
            raise RuntimeError(f"{name}: expected axis 0 to have size batch")
        if t.shape[1] != chan:
            raise RuntimeError(f"{name}: expected axis 1 to have size chan")
        for a in range(r):
            if t.shape[2 + a] != 3:
                raise RuntimeError(f"{name}: expected axis {2 + a} to have size 3")
    return batch, chan


def bee_fwd(l_0, l_1, l_2, r_0, r_1, r_2):
    batch, chan = _check_operands(("l_0", "l_1", "l_2", "r_0", "r_1", "r_2"), (l_0, l_1, l_2, r_0, r_1, r_2), (0, 1, 2, 0, 1, 2))
    outs = [torch.empty((batch, chan) + tuple(s), dtype=torch.float32, device=l_0.device) for s in BEE_SUFFIX]
    if batch > 0:
        arr = _ptr_array(outs)
        check(lib().ld_bee_fwd(ptr(l_0), ptr(l_1), ptr(l_2), ptr(r_0), ptr(r_1), ptr(r_2), batch, chan, arr, stream_ptr(l_0.device)))
    return outs


def bee_self_products_cm(lr_0, lr_1, lr_2):
    """bee_self_products for component-major operands lr_1 [rows, 3, 2*chan], lr_2 [rows, 9, 2*chan]; P_v / P_d BF16
    component-major."""
    for name, t in (("lr_0", lr_0), ("lr_1", lr_1), ("lr_2", lr_2)):
        require_cuda_f32(t, name)
    rows, chan = lr_0.shape[0], lr_0.shape[1] // 2
    if lr_0.shape != (rows, 2 * chan) or lr_1.shape != (rows, 3, 2 * chan) or lr_2.shape != (rows, 9, 2 * chan):
        raise RuntimeError("bee_self_products_cm: expected [rows, 2*chan], [rows, 3, 2*chan], [rows, 9, 2*chan]")
    dev = lr_0.device
    P_a = torch.empty(rows, 3 * chan, dtype=torch.float32, device=dev)
    P_v = torch.empty(rows, 3, 5 * chan, dtype=torch.bfloat16, device=dev)
    P_d = torch.empty(rows, 9, 5 * chan, dtype=torch.bfloat16, device=dev)
    with KERNEL_TIMER.region("bee_self_products"):
        check(lib().ld_bee_self_products_cm(ptr(lr_0), ptr(lr_1), ptr(lr_2), rows, chan, ptr(P_a), ptr(P_v), ptr(P_d), stream_ptr(dev)))
    return P_a, P_v, P_d


def bee_self_products(lr_0, lr_1, lr_2, out_bf16=False):
    """13 Bee products of left = lr[:, :chan], right = lr[:, chan:], concatenated per rank:
    P_a [rows, 3*chan], P_v [rows, 5*chan, 3], P_d [rows, 5*chan, 3, 3] (the inputs of concatenated Y maps).
    out_bf16: P_v [rows, 3, 5*chan] and P_d [rows, 9, 5*chan] as BF16, component-major (for linear_bf16_tc_cm, which
    rounds its operands to BF16 anyway)."""
    for name, t in (("lr_0", lr_0), ("lr_1", lr_1), ("lr_2", lr_2)):
        require_cuda_f32(t, name)
    rows, chan = lr_0.shape[0], lr_0.shape[1] // 2
    if lr_0.shape != (rows, 2 * chan) or lr_1.shape != (rows, 2 * chan, 3) or lr_2.shape != (rows, 2 * chan, 3, 3):
        raise RuntimeError("bee_self_products: expected [rows, 2*chan], [rows, 2*chan, 3], [rows, 2*chan, 3, 3]")
    dev = lr_0.device
    P_a = torch.empty(rows, 3 * chan, dtype=torch.float32, device=dev)
    odt = torch.bfloat16 if out_bf16 else torch.float32
    P_v = torch.empty((rows, 3, 5 * chan) if out_bf16 else (rows, 5 * chan, 3), dtype=odt, device=dev)
    P_d = torch.empty((rows, 9, 5 * chan) if out_bf16 else (rows, 5 * chan, 3, 3), dtype=odt, device=dev)
    with KERNEL_TIMER.region("bee_self_products"):
        check(lib().ld_bee_self_products(ptr(lr_0), ptr(lr_1), ptr(lr_2), rows, chan, ptr(P_a), ptr(P_v), ptr(P_d),
                                         1 if out_bf16 else 0, stream_ptr(dev)))
    return P_a, P_v, P_d


def bee_bw(left, o_0, o_1, o_2, grads):
    names = ("r_0", "r_1", "r_2") if left else ("l_0", "l_1", "l_2")
    batch, chan = _check_operands(names, (o_0, o_1, o_2), (0, 1, 2))
    grads = [g.contiguous() for g in grads]
    dev = o_0.device
    d0 = torch.empty(batch, chan, dtype=torch.float32, device=dev)
    d1 = torch.empty(batch, chan, 3, dtype=torch.float32, device=dev)
    d2 = torch.empty(batch, chan, 3, 3, dtype=torch.float32, device=dev)
    if batch > 0:
        arr = _ptr_array(grads)
        check(lib().ld_bee_bw(1 if left else 0, ptr(o_0), ptr(o_1), ptr(o_2), arr, batch, chan, ptr(d0), ptr(d1), ptr(d2), stream_ptr(dev)))
    return [d0, d1, d2]


def cow_o0_fwd(l_0, l_1, r_0, r_1):
    batch, chan = _check_operands(("l_0", "l_1", "r_0", "r_1"), (l_0, l_1, r_0, r_1), (0, 1, 0, 1))
    dev = l_0.device
    y000 = torch.empty(batch, chan, dtype=torch.float32, device=dev)
    y110 = torch.empty(batch, chan, dtype=torch.float32, device=dev)
    if batch > 0:
        check(lib().ld_cow_o0_fwd(ptr(l_0), ptr(l_1), ptr(r_0), ptr(r_1), batch, chan, ptr(y000), ptr(y110), stream_ptr(dev)))
    return [y000, y110]


def cow_o0_bw(o_0, o_1, g000, g110):
    batch, chan = _check_operands(("o_0", "o_1"), (o_0, o_1), (0, 1))
    dev = o_0.device
    g000, g110 = g000.contiguous(), g110.contiguous()
    d0 = torch.empty(batch, chan, dtype=torch.float32, device=dev)
    d1 = torch.empty(batch, chan, 3, dtype=torch.float32, device=dev)
    if batch > 0:
        check(lib().ld_cow_o0_bw(ptr(o_0), ptr(o_1), ptr(g000), ptr(g110), batch, chan, ptr(d0), ptr(d1), stream_ptr(dev)))
    return [d0, d1]


def cow_o1_fwd(l_0, l_1, r_0, r_1):
    batch, chan = _check_operands(("l_0", "l_1", "r_0", "r_1"), (l_0, l_1, r_0, r_1), (0, 1, 0, 1))
    dev = l_0.device
    outs = [torch.empty(batch, chan, 3, dtype=torch.float32, device=dev) for _ in range(3)]
    if batch > 0:
        check(lib().ld_cow_o1_fwd(ptr(l_0), ptr(l_1), ptr(r_0), ptr(r_1), batch, chan, ptr(outs[0]), ptr(outs[1]), ptr(outs[2]), stream_ptr(dev)))
    return outs


def cow_o1_bw(left, o_0, o_1, g011, g101, g111):
    batch, chan = _check_operands(("o_0", "o_1"), (o_0, o_1), (0, 1))
    dev = o_0.device
    g011, g101, g111 = g011.contiguous(), g101.contiguous(), g111.contiguous()
    d0 = torch.empty(batch, chan, dtype=torch.float32, device=dev)
    d1 = torch.empty(batch, chan, 3, dtype=torch.float32, device=dev)
    if batch > 0:
        check(lib().ld_cow_o1_bw(1 if left else 0, ptr(o_0), ptr(o_1), ptr(g011), ptr(g101), ptr(g111), batch, chan, ptr(d0), ptr(d1), stream_ptr(dev)))
    return [d0, d1]


class PackedMLP:
    """Weights of a 3-layer MLP in the kernels' layouts: FP32 [in][out] per layer for the SIMT
    kernels and (built on first use) BF16 operand panels for the tensor-core kernels."""

    def __init__(self, linears, direct=None):
        l1, l2, l3 = linears
        self._linears = (l1, l2, l3)
        self._bf16 = None
        self.Wt = [l.weight.detach().t().contiguous().float() for l in (l1, l2, l3)]
        self.b = [None if l.bias is None else l.bias.detach().contiguous().float() for l in (l1, l2, l3)]
        self.dims = (l1.weight.shape[1], l1.weight.shape[0], l2.weight.shape[0], l3.weight.shape[0])
        self.Wdt = None if direct is None else direct.weight.detach().t().contiguous().float()


def _packed_bf16(mlp):
    if mlp._bf16 is None:
        mlp._bf16 = [pack_weights_bf16(l.weight.detach().float()) for l in mlp._linears]
    return mlp._bf16


def mlp3_rows(x, mlp, act=ACT_SILU):
    """Three dense layers (activation after the first two) on the rows of x[..., k0]."""
    x = x.contiguous()
    require_cuda_f32(x, "x")
    k0, n1, n2, n3 = mlp.dims
    if x.shape[-1] != k0:
        raise RuntimeError("mlp3_rows: input width mismatch")
    rows = x.numel() // k0
    out = torch.empty(tuple(x.shape[:-1]) + (n3,), dtype=torch.float32, device=x.device)
    with KERNEL_TIMER.region("mlp3_rows"):
        check(lib().ld_mlp3_rows(ptr(x), rows, k0, ptr(mlp.Wt[0]), ptr(mlp.b[0]), n1, ptr(mlp.Wt[1]), ptr(mlp.b[1]), n2,
                                 ptr(mlp.Wt[2]), ptr(mlp.b[2]), n3, act, ptr(mlp.Wdt), ptr(out), stream_ptr(x.device)))
    return out


def painn_message_f32(row_ptr, dst, rij, mlp_dist, actv, x_v, rmax, eps=0.1, radial_kind=RADIAL_PAINN, res_a=None,
                      res_v=None, edge_counter=None):
    """Fused PaiNN message; returns (out_a [Nt,n], out_v [Nt,n,3]). actv = mlp_actv(x_a) as [Nt,4n]."""
    require_cuda_f32(actv, "actv")
    require_cuda_f32(x_v, "x_v")
    require_cuda_f32(rij, "rij")
    Nt, n = x_v.shape[0], x_v.shape[1]
    n_rbf, n1, n2, n3 = mlp_dist.dims
    if not (n1 == n2 == n3 == 4 * n) or actv.shape != (Nt, 4 * n):
        raise RuntimeError("painn_message: widths must be n_rbf -> 4n -> 4n -> 4n and actv [Nt,4n]")
    if dst.dtype != torch.int32 or row_ptr.dtype != torch.int32:
        raise RuntimeError("painn_message: row_ptr and dst must be int32")
    out_a = torch.empty(Nt, n, dtype=torch.float32, device=x_v.device)
    out_v = torch.empty(Nt, n, 3, dtype=torch.float32, device=x_v.device)
    with KERNEL_TIMER.region("painn_message"):
        check(lib().ld_painn_message_f32(ptr(row_ptr), ptr(dst), ptr(rij), Nt, n, n_rbf, radial_kind, float(rmax), float(eps),
                                         ptr(mlp_dist.Wt[0]), ptr(mlp_dist.b[0]), ptr(mlp_dist.Wt[1]), ptr(mlp_dist.b[1]),
                                         ptr(mlp_dist.Wt[2]), ptr(mlp_dist.b[2]), ptr(actv), ptr(x_v), ptr(res_a), ptr(res_v),
                                         ptr(out_a), ptr(out_v), ptr(edge_counter), stream_ptr(x_v.device)))
    return out_a, out_v


_TC_STATUS = {}


def tc_status(device):
    """Device status word shared by the tensor-core kernels of one device (LD_FLAG_* bits)."""
    key = torch.device(device).index or 0
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


_TC_WATCH = {}


def check_tc_status(device, block=True):
    """Raise HotpathError(LD_ERR_TIMEOUT) if a tensor-core kernel on `device` gave up on a bounded wait (its outputs are
    then incomplete), and clear the status word. block=True reads the word now (synchronises the device).
    block=False is for rollout loops: it looks at the copy of the word requested by the previous call, if that copy
    has arrived, and requests a new one on the current stream without waiting for it; a timeout is then reported one or
    two steps late, but no step waits for the device. ModelPredictor.predict and the generate() loops call it this way
    every step and with block=True once at the end."""
    from ._lib import HotpathError, LD_ERR_TIMEOUT
    dev = torch.device(device)
    key = dev.index or 0
    word = tc_status(dev)

    def report(value):
        if value != 0:
            word.zero_()
            _TC_WATCH.pop(key, None)
            raise HotpathError(LD_ERR_TIMEOUT, f"a tensor-core kernel gave up on a bounded wait (status flags {value:#x}); "
                                               "the outputs of the affected step are incomplete")

    pending = _TC_WATCH.get(key)
    if block:
        _TC_WATCH.pop(key, None)
        report(int(word.item()))
        return
    if pending is not None:
        host, ev = pending
        if not ev.query():
            return
        report(int(host[0]))
    else:
        host = torch.zeros(1, dtype=torch.int32).pin_memory()
    host.copy_(word, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(dev))
    _TC_WATCH[key] = (host, ev)


def pack_weights_bf16(W):
    """[N, K] float32 (any strides) -> BF16 operand panels for the tensor-core kernels."""
    N, K = W.shape
    n = lib().ld_packed_weight_elems(N, K)
    out = torch.empty(n, dtype=torch.bfloat16, device=W.device)
    check(lib().ld_pack_weights_bf16(ptr(W), W.stride(0), W.stride(1), N, K, ptr(out), stream_ptr(W.device)))
    return out


def linear_bf16_tc(x, W_packed, N, bias=None, act=ACT_NONE, inds=0, out_bf16=False, out=None, out_layout=None, out_split=None,
                   in_cm=False):
    """y[..., o, s] = act(sum_i W[o,i] x[..., i, s] + b[o]) on tcgen05 (BF16 operands, FP32 accumulate).
    out_bf16: round the result to BF16. out / out_layout=(ld_row, ld_col, off): write BF16 element (r, o, s)
    to out.flatten()[r*ld_row + o*ld_col + s + off] instead of a new tensor; out_split=(s_split, s_jump) moves the
    components s >= s_split another s_jump elements on. in_cm (with out): x is component-major, [..., 3**inds, K]."""
    x = x.contiguous()
    require_cuda_f32(x, "x")
    S = 3 ** inds
    shape = list(x.shape)
    if in_cm:
        if out is None or x.dim() < 2 or (inds > 0 and shape[-2] != S):
            raise RuntimeError("linear_bf16_tc: component-major input is [..., 3**inds, K] and needs an output buffer")
        shape = shape[:-2] + [shape[-1]] + [3] * inds if inds > 0 else shape
    bd = len(shape) - (1 + inds)
    K = shape[bd]
    rows = 1
    for d in shape[:bd]:
        rows *= d
    shape[bd] = N
    st, status = stream_ptr(x.device), ptr(tc_status(x.device))
    with KERNEL_TIMER.region("linear_bf16_tc"):
        if out is not None and (out_split is not None or in_cm):
            ld_row, ld_col, off = out_layout
            sp = out_split if out_split is not None else (1 << 30, 0)
            check(lib().ld_linear_bf16_tc_out16_split(ptr(x), rows, K, S, ptr(W_packed), ptr(bias), N, act, ptr(out), ld_row,
                                                      ld_col, off, sp[0], sp[1], 1 if in_cm else 0, status, st))
            return out
        if out is not None:
            ld_row, ld_col, off = out_layout
            check(lib().ld_linear_bf16_tc_out16(ptr(x), rows, K, S, ptr(W_packed), ptr(bias), N, act, ptr(out), ld_row, ld_col,
                                                off, status, st))
            return out
        if out_bf16:
            y = torch.empty(shape, dtype=torch.bfloat16, device=x.device)
            check(lib().ld_linear_bf16_tc_out16(ptr(x), rows, K, S, ptr(W_packed), ptr(bias), N, act, ptr(y), N * S, S, 0,
                                                status, st))
            return y
        y = torch.empty(shape, dtype=torch.float32, device=x.device)
        check(lib().ld_linear_bf16_tc(ptr(x), rows, K, S, ptr(W_packed), ptr(bias), N, act, ptr(y), status, st))
    return y


def linear_bf16_tc_rows16(x16, W_packed, N, bias=None, act=ACT_NONE):
    """y [..., N] FP32 = act(x16 [..., K] W^T + b) for BF16 rows (K contiguous, a multiple of 8). With component-major
    activations [rows, 3**inds, K] the result is component-major as well, [rows, 3**inds, N]: plain rows in and out."""
    if not x16.is_cuda or x16.dtype != torch.bfloat16 or not x16.is_contiguous():
        raise RuntimeError("linear_bf16_tc_rows16: expected a contiguous CUDA BF16 tensor")
    K = x16.shape[-1]
    rows = x16.numel() // K
    y = torch.empty(tuple(x16.shape[:-1]) + (N,), dtype=torch.float32, device=x16.device)
    with KERNEL_TIMER.region("linear_bf16_tc"):
        check(lib().ld_linear_bf16_tc_in16(ptr(x16), rows, K, 1, ptr(W_packed), ptr(bias), N, act, ptr(y),
                                           ptr(tc_status(x16.device)), stream_ptr(x16.device)))
    return y


def linear_bf16_tc_cm(x16, W_packed, N, inds, bias=None, act=ACT_NONE, residual=None):
    """linear_bf16_tc for activations stored as BF16 in component-major form, x16 [rows, 3**inds, K] (K contiguous,
    a multiple of 8): returns y [rows, N, (3,)*inds] FP32. Same result as the FP32 [rows, K, (3,)*inds] form of the
    same values (the MMA operands are BF16 either way). residual (FP32, shape of y): returns residual + y, added in the
    kernel's epilogue where the streaming kernel serves the shape, by a separate add otherwise."""
    if not x16.is_cuda or x16.dtype != torch.bfloat16 or not x16.is_contiguous() or x16.dim() != 3 or x16.shape[1] != 3 ** inds:
        raise RuntimeError("linear_bf16_tc_cm: expected a contiguous CUDA BF16 tensor [rows, 3**inds, K]")
    rows, S, K = x16.shape
    y = torch.empty((rows, N) + (3,) * inds, dtype=torch.float32, device=x16.device)
    if residual is not None:
        residual = residual.reshape(y.shape).contiguous()
        if residual.dtype == torch.float32 and K % 128 == 0 and N <= 128 and K * N * 2 <= 94 * 1024:
            with KERNEL_TIMER.region("linear_bf16_tc"):
                check(lib().ld_linear_bf16_tc_in16_res(ptr(x16), ptr(residual), rows, K, S, ptr(W_packed), ptr(bias), N, act, ptr(y),
                                                       ptr(tc_status(x16.device)), stream_ptr(x16.device)))
            return y
    with KERNEL_TIMER.region("linear_bf16_tc"):
        check(lib().ld_linear_bf16_tc_in16(ptr(x16), rows, K, S, ptr(W_packed), ptr(bias), N, act, ptr(y),
                                           ptr(tc_status(x16.device)), stream_ptr(x16.device)))
    return y if residual is None else residual + y


def painn_message_bf16_tc(row_ptr, dst, rij, mlp_dist, actv, x_v, rmax, eps=0.1, radial_kind=RADIAL_PAINN, res_a=None,
                          res_v=None, edge_counter=None):
    """Tensor-core variant of painn_message_f32 (BF16 operands in the per-edge MLP, 2e-2 relative)."""
    require_cuda_f32(actv, "actv")
    require_cuda_f32(x_v, "x_v")
    require_cuda_f32(rij, "rij")
    Nt, n = x_v.shape[0], x_v.shape[1]
    n_rbf, n1, n2, n3 = mlp_dist.dims
    if not (n1 == n2 == n3 == 4 * n) or actv.shape != (Nt, 4 * n):
        raise RuntimeError("painn_message: widths must be n_rbf -> 4n -> 4n -> 4n and actv [Nt,4n]")
    if dst.dtype != torch.int32 or row_ptr.dtype != torch.int32:
        raise RuntimeError("painn_message: row_ptr and dst must be int32")
    w = _packed_bf16(mlp_dist)
    out_a = torch.empty(Nt, n, dtype=torch.float32, device=x_v.device)
    out_v = torch.empty(Nt, n, 3, dtype=torch.float32, device=x_v.device)
    st = stream_ptr(x_v.device)
    # neighbour features as 128-byte BF16 records per 8 channels: the edge kernel gathers 2 KB instead of 3.5 KB per edge
    g16 = torch.empty(Nt, n // 8, 64, dtype=torch.bfloat16, device=x_v.device)
    with KERNEL_TIMER.region("painn_pack_gather"):
        check(lib().ld_painn_pack_gather(ptr(actv), ptr(x_v), Nt, n, ptr(g16), st))
    with KERNEL_TIMER.region("painn_message_tc"):
        check(lib().ld_painn_message_bf16_tc(ptr(row_ptr), ptr(dst), ptr(rij), Nt, n, n_rbf, radial_kind, float(rmax),
                                             float(eps), ptr(w[0]), ptr(mlp_dist.b[0]), ptr(w[1]), ptr(mlp_dist.b[1]),
                                             ptr(w[2]), ptr(mlp_dist.b[2]), ptr(actv), ptr(x_v), ptr(g16), ptr(res_a), ptr(res_v),
                                             ptr(out_a), ptr(out_v), ptr(edge_counter), ptr(tc_status(x_v.device)), st))
    return out_a, out_v


def group_norm_cm(x, groups, eps, gamma):
    """TensGroupNorm of component-major activations x [B, N, S, C] (S = 3**inds): same statistics and result as
    group_norm on the [B, N, C, (3,)*inds] form, element for element."""
    require_cuda_f32(x, "x")
    x = x.contiguous()
    B, N, S, C = x.shape
    if C % groups != 0:
        raise RuntimeError("group_norm: channels must divide into the groups")
    y = torch.empty_like(x)
    ws = torch.empty(max(98 * B * groups, 1), dtype=torch.float32, device=x.device)
    g = gamma.detach().reshape(-1).float().contiguous()
    with KERNEL_TIMER.region("group_norm"):
        check(lib().ld_group_norm_cm(ptr(x), B, N, C, S, groups, 0, float(eps), ptr(g), None, ptr(y), ptr(ws), stream_ptr(x.device)))
    return y


def group_norm(x, groups, eps, gamma, beta=None, center=False, residual=None):
    """Per-system group norm of x [B, N, C, (3,)*inds] (fused statistics + apply kernels).
    center=True: ScalGroupNorm (mean subtracted, beta added; scalars only); center=False: TensGroupNorm (x is divided
    by the root of the group's mean squared norm, gamma applied, no beta). residual (shape of x): returns residual + norm."""
    require_cuda_f32(x, "x")
    x = x.contiguous()
    B, N, C = x.shape[0], x.shape[1], x.shape[2]
    S = 1
    for d in x.shape[3:]:
        S *= d
    if C % groups != 0:
        raise RuntimeError("group_norm: channels must divide into the groups")
    y = torch.empty_like(x)
    ws = torch.empty(max(98 * B * groups, 1), dtype=torch.float32, device=x.device)
    g = gamma.detach().reshape(-1).float().contiguous()
    b = None if beta is None else beta.detach().reshape(-1).float().contiguous()
    if residual is not None:
        require_cuda_f32(residual, "residual")
        residual = residual.contiguous()
        if residual.shape != x.shape:
            raise RuntimeError("group_norm: the residual must have the shape of x")
    with KERNEL_TIMER.region("group_norm"):
        check(lib().ld_group_norm_res(ptr(x), ptr(residual), B, N, C, S, groups, 1 if center else 0, float(eps), ptr(g), ptr(b), ptr(y),
                                      ptr(ws), stream_ptr(x.device)))
    return y
