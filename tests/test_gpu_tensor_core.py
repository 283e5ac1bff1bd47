"""tcgen05 dense layers against an FP32 torch reference of the same op. BF16 operands with FP32
accumulation: 2e-2 relative (max-norm)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def close(a, b, rel):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    scale = max(b.abs().max().item(), 1e-30)
    assert err <= rel * scale, f"max abs err {err:.3e} vs scale {scale:.3e} (rel {err / scale:.2e})"


def _status_ok():
    from ld_b200 import ops
    assert int(ops.tc_status("cuda").item()) == 0, "a bounded device-side wait ran out"


@pytest.mark.parametrize("rows,K,N", [(128, 64, 32), (1, 16, 32), (300, 128, 128), (1000, 128, 512), (517, 8, 512),
                                      (4096, 512, 512), (257, 256, 384), (129, 117, 224)])
@pytest.mark.parametrize("act", [0, 1])
def test_linear_tc(rows, K, N, act):
    from ld_b200 import ops
    g = torch.Generator().manual_seed(rows + K + N)
    W = torch.randn(N, K, generator=g) / K ** 0.5
    b = torch.randn(N, generator=g)
    x = torch.randn(rows, K, generator=g)
    want = x @ W.t() + b
    if act == 1:
        want = torch.nn.functional.silu(want)
    wp = ops.pack_weights_bf16(W.cuda())
    got = ops.linear_bf16_tc(x.cuda(), wp, N, b.cuda(), act)
    torch.cuda.synchronize()
    _status_ok()
    close(got, want, 2e-2)
    # exactness of the machinery: with BF16-representable inputs only accumulation order differs
    xb, Wb = x.bfloat16().float(), W.bfloat16().float()
    want_b = xb @ Wb.t() + b
    if act == 1:
        want_b = torch.nn.functional.silu(want_b)
    got_b = ops.linear_bf16_tc(xb.cuda(), ops.pack_weights_bf16(Wb.cuda()), N, b.cuda(), act)
    close(got_b, want_b, 2e-5)


@pytest.mark.parametrize("inds", [1, 2])
def test_tensor_linear_tc(inds):
    from ld_b200 import ops
    from oracle import reference_math as R
    g = torch.Generator().manual_seed(inds)
    W = torch.randn(64, 128, generator=g) / 128 ** 0.5
    x = torch.randn(3, 50, 128, *([3] * inds), generator=g)
    want = R.tensor_linear(inds, W, x)
    got = ops.linear_bf16_tc(x.cuda(), ops.pack_weights_bf16(W.cuda()), 64, None, 0, inds=inds)
    _status_ok()
    close(got, want, 2e-2)
    xb, Wb = x.bfloat16().float(), W.bfloat16().float()
    got_b = ops.linear_bf16_tc(xb.cuda(), ops.pack_weights_bf16(Wb.cuda()), 64, None, 0, inds=inds)
    close(got_b, R.tensor_linear(inds, Wb, xb), 2e-5)


def test_many_tiles_persistent():
    from ld_b200 import ops
    g = torch.Generator().manual_seed(5)
    W = torch.randn(128, 128, generator=g).bfloat16().float() / 8
    x = torch.randn(60000, 128, generator=g).bfloat16().float()
    got = ops.linear_bf16_tc(x.cuda(), ops.pack_weights_bf16(W.cuda()), 128)
    _status_ok()
    close(got, x @ W.t(), 2e-5)


def _message_pair(r0, n, seed, n_rbf=None, radial="painn"):
    from ld_b200 import painn
    from oracle import reference_math as R
    torch.manual_seed(seed)
    ref = R.OMessage(r0, n, n_rbf, radial)
    mine = painn.Message(r0, n, n_rbf, radial)
    mine.load_state_dict(ref.state_dict())
    mine.precision = "bf16"
    return ref, mine.cuda()


@pytest.mark.parametrize("n,B,N,r0,box,n_rbf,radial", [
    (128, 2, 300, 2.0, (9.0, 9.0, 9.0), 8, "gaussian"),
    (64, 8, 64, 3.0, None, 8, "gaussian"),       # benchmark config 0 shape
    (128, 1, 700, 2.5, (10.0, 10.0, 10.0), None, "painn"),
    (96, 3, 40, 1.0, None, 16, "gaussian"),
    (128, 1, 5, 2.0, None, 16, "gaussian"),
])
def test_message_tc_vs_oracle(n, B, N, r0, box, n_rbf, radial):
    """BF16 tensor-core message against the FP32 CPU oracle (2e-2) and against the FP32 GPU kernel"""
    from ld_b200 import graph_layers as GL
    from oracle import reference_math as R
    ref, mine = _message_pair(r0, n, seed=n + N, n_rbf=n_rbf, radial=radial)
    g = torch.Generator().manual_seed(2000 + n)
    if box is None:
        pos = torch.cumsum(torch.randn(B, N, 3, generator=g) / 3 ** 0.5, dim=1)
    else:
        pos = torch.rand(B, N, 3, generator=g) * torch.tensor(box)
    x_a = torch.randn(B, N, n, generator=g)
    x_v = torch.randn(B, N, n, 3, generator=g)
    o = R.radius_graph(pos, r0, box)
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    with torch.no_grad():
        ra, rv = ref(o["src"], o["dst"], x_a, x_v, o["rij"])
        graph = GL.Graph.radius_graph(r0, box, pos.cuda())
        ga, gv = mine(graph, x_a.cuda(), x_v.cuda(), graph.rij, edge_counter=counter)
        ga2, gv2 = mine(graph, x_a.cuda(), x_v.cuda(), graph.rij, residual=True)
    torch.cuda.synchronize()
    _status_ok()
    assert int(counter.item()) == o["E"]
    close(ga, ra, 2e-2)
    close(gv, rv, 2e-2)
    close(ga2, x_a + ra, 2e-2)
    close(gv2, x_v + rv, 2e-2)


def test_message_tc_empty_and_isolated():
    from ld_b200 import graph_layers as GL
    from oracle import reference_math as R
    ref, mine = _message_pair(1.0, 128, seed=3, n_rbf=8, radial="gaussian")
    pos = torch.arange(6, dtype=torch.float32).reshape(1, 6, 1).repeat(1, 1, 3) * 10
    x_a, x_v = torch.randn(1, 6, 128), torch.randn(1, 6, 128, 3)
    with torch.no_grad():
        graph = GL.Graph.radius_graph(1.0, None, pos.cuda())
        a, v = mine(graph, x_a.cuda(), x_v.cuda(), graph.rij)
    assert a.abs().max() == 0 and v.abs().max() == 0
    pos[0, 1] = pos[0, 0] + 0.5
    o = R.radius_graph(pos, 1.0, None)
    with torch.no_grad():
        graph = GL.Graph.radius_graph(1.0, None, pos.cuda())
        a, v = mine(graph, x_a.cuda(), x_v.cuda(), graph.rij)
        ra, rv = ref(o["src"], o["dst"], x_a, x_v, o["rij"])
    _status_ok()
    close(a, ra, 2e-2)
    close(v, rv, 2e-2)


def test_message_tc_deterministic():
    from ld_b200 import graph_layers as GL
    _, mine = _message_pair(2.0, 128, seed=4, n_rbf=8, radial="gaussian")
    g = torch.Generator().manual_seed(44)
    pos = (torch.rand(2, 1500, 3, generator=g) * 12.0).cuda()
    x_a, x_v = torch.randn(2, 1500, 128, generator=g).cuda(), torch.randn(2, 1500, 128, 3, generator=g).cuda()
    with torch.no_grad():
        graph = GL.Graph.radius_graph(2.0, (12.0, 12.0, 12.0), pos)
        a1, v1 = mine(graph, x_a, x_v, graph.rij)
        a2, v2 = mine(graph, x_a, x_v, graph.rij)
    assert torch.equal(a1, a2) and torch.equal(v1, v2)


def test_denoiser_bf16_vs_oracle():
    """whole denoiser with every Message and MLP on the tensor-core path, against the FP32 CPU oracle"""
    from ld_b200 import painn
    from oracle import reference_math as R
    n, B, N, r0 = 128, 2, 60, 2.5
    torch.manual_seed(5)
    ref = R.OSE3ITO(r0, n, N, 4, 1, 2, 8, "gaussian")
    mine = painn.SE3ITO(r0, n, N, 4, 1, 2, n_rbf=8, radial="gaussian")
    mine.load_state_dict(ref.state_dict())
    painn.set_precision(mine.cuda(), "bf16")
    g = torch.Generator().manual_seed(78)
    box = (8.0, 8.0, 9.0)
    x0 = torch.rand(B, N, 3, generator=g) * torch.tensor(box)
    x1 = x0 + 0.3 * torch.randn(B, N, 3, generator=g)
    types = torch.randint(0, 4, (N,), generator=g)
    s_, t_ = torch.full((B,), 0.2), torch.full((B,), 0.7)
    empty = torch.zeros(0, dtype=torch.int64)
    with torch.no_grad():
        want = ref((s_, t_), x0, x1, box, types, empty, empty)
        got = mine((s_.cuda(), t_.cuda()), x0.cuda(), x1.cuda(), box, types.cuda(), painn.empty_bond_graph(B, N, "cuda"))
    _status_ok()
    close(got, want, 2e-2)


@pytest.mark.parametrize("inds,rows,K,N", [(1, 700, 640, 64), (2, 129, 640, 32), (0, 300, 64, 128), (2, 5, 8, 32)])
def test_linear_component_major_bf16_input_matches_fp32_input(inds, rows, K, N):
    """BF16 activations stored [rows, 3**inds, K] give bit-identical results to the same values passed as FP32
    [rows, K, (3,)*inds]: the tensor-core path rounds its operands to BF16 either way"""
    from ld_b200 import ops
    g = torch.Generator().manual_seed(K + N + inds)
    S = 3 ** inds
    x16 = torch.randn(rows, S, K, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(N, K, generator=g) * K ** -0.5).cuda()
    Wp = ops.pack_weights_bf16(W)
    x32 = x16.float().permute(0, 2, 1).reshape(rows, K, *([3] * inds)).contiguous()
    a = ops.linear_bf16_tc_cm(x16, Wp, N, inds)
    b = ops.linear_bf16_tc(x32, Wp, N, inds=inds)
    assert a.shape == b.shape and torch.equal(a, b)
    assert int(ops.tc_status("cuda").item()) == 0


@pytest.mark.parametrize("rows,S,K,N,bias,act", [(148 * 128 * 3 + 77, 1, 640, 64, False, 0), (40000, 9, 640, 32, False, 0),
                                                 (30011, 3, 256, 128, True, 2), (1000, 1, 64, 96, True, 1), (1, 1, 640, 64, False, 0)])
def test_streaming_rows_gemm_against_float_reference(rows, S, K, N, bias, act):
    """the streaming kernel for BF16 rows (weights resident in shared memory, six chunks of asynchronous copies in
    flight, accumulators of two tiles alternating): many tiles per block, a ragged last tile, bias and activation,
    against the FP32 product of the same BF16-rounded operands (1e-5 of the output scale; the sums differ only in order)"""
    from ld_b200 import ops
    g = torch.Generator().manual_seed(rows % 1000 + K + N)
    x16 = torch.randn(rows, S, K, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(N, K, generator=g) * K ** -0.5).cuda()
    b = torch.randn(N, generator=g).cuda() if bias else None
    Wp = ops.pack_weights_bf16(W)
    inds = {1: 0, 3: 1, 9: 2}[S]
    got = ops.linear_bf16_tc_cm(x16, Wp, N, inds, bias=b, act=act)
    again = ops.linear_bf16_tc_cm(x16, Wp, N, inds, bias=b, act=act)
    torch.cuda.synchronize()
    assert int(ops.tc_status("cuda").item()) == 0
    assert torch.equal(got, again)
    want = x16.float() @ W.to(torch.bfloat16).float().t()
    if bias:
        want = want + b
    if act == 1:
        want = torch.nn.functional.silu(want)
    elif act == 2:
        want = torch.nn.functional.leaky_relu(want, 0.1)
    want = want.permute(0, 2, 1).reshape(got.shape)
    close(got, want, 1e-5)


def test_bounded_wait_runs_out_and_returns():
    """A launch of the tensor-core linear whose weight panels are never requested: every wait gives up after 64 polls,
    all blocks leave through the failure path (status flag set, tensor memory released, no trap), the host check
    raises and clears the word, and the next launch on the same device is correct."""
    from ld_b200 import ops
    from ld_b200._lib import lib, check, ptr, stream_ptr, HotpathError, LD_ERR_TIMEOUT, LD_FLAG_TIMEOUT
    torch.cuda.synchronize()
    ops.check_tc_status("cuda")                       # clean before
    g = torch.Generator().manual_seed(5)
    rows, K, N = 200, 128, 64
    W = torch.randn(N, K, generator=g) / K ** 0.5
    x = torch.randn(rows, K, generator=g).cuda()
    wp = ops.pack_weights_bf16(W.cuda())
    y = torch.full((rows, N), 7.0, device="cuda")
    status = ops.tc_status("cuda")
    check(lib().ld_linear_bf16_tc_selftest_timeout(ptr(x), rows, K, ptr(wp), N, ptr(y), ptr(status), stream_ptr(x.device)))
    torch.cuda.synchronize()                          # the kernel returned by itself
    assert int(status.item()) & LD_FLAG_TIMEOUT
    assert torch.all(y == 7.0)                        # nothing was written
    with pytest.raises(HotpathError) as err:
        ops.check_tc_status("cuda")
    assert err.value.status == LD_ERR_TIMEOUT
    assert int(status.item()) == 0                    # reported once, then cleared
    # tensor memory was released and the context is intact: the regular launch works, several times over
    for _ in range(3):
        got = ops.linear_bf16_tc(x, wp, N)
    torch.cuda.synchronize()
    _status_ok()
    close(got, x.cpu() @ W.t(), 2e-2)
    # the non-blocking form used inside rollout loops reports a flagged step on a later call
    check(lib().ld_linear_bf16_tc_selftest_timeout(ptr(x), rows, K, ptr(wp), N, ptr(y), ptr(status), stream_ptr(x.device)))
    ops.check_tc_status("cuda", block=False)          # requests a copy of the word
    torch.cuda.synchronize()
    with pytest.raises(HotpathError):
        ops.check_tc_status("cuda", block=False)      # the copy has arrived and shows the flag
    assert int(status.item()) == 0
