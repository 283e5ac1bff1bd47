"""Dense proximity attention kernels (forward and the five gradients) through the C ABI against the
reference-generated golden vectors and the CPU oracle. FP32: 2e-5 of the largest entry of each tensor."""
import pytest
import torch

from oracle import reference_math as R

pytestmark = pytest.mark.gpu


def close(a, b, rel=2e-5):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    scale = max(b.abs().max().item(), 1e-30)
    assert err <= rel * scale, f"max abs err {err:.3e} vs scale {scale:.3e} (rel {err / scale:.2e})"


def run(ins, r0sq, box, cot):
    from ld_b200 import proxattn as PA
    g_in = [t.detach().cuda().requires_grad_(True) for t in ins]
    out = PA.proxattn(*g_in, r0sq.cuda()) if box is None else PA.proxattn_periodic(*g_in, r0sq.cuda(), box)
    grads = torch.autograd.grad((out * cot.cuda()).sum(), g_in)
    return out, grads


def test_against_reference_golden(golden):
    p = golden["proxattn"]
    for box, ko, kg in ((None, "out", "grads"), (p["box"], "out_periodic", "grads_periodic")):
        out, grads = run(p["inputs"], p["r0sq"], box, p["cotangent"])
        close(out, p[ko])
        for mine, ref in zip(grads, p[kg]):
            close(mine, ref)


@pytest.mark.parametrize("dim", [16, 32, 64, 128])
@pytest.mark.parametrize("Z,N,heads", [(5, 1, 5), (4, 64, 2), (3, 130, 1), (10, 257, 5)])
@pytest.mark.parametrize("periodic", [False, True])
def test_vs_oracle(dim, Z, N, heads, periodic):
    g = torch.Generator().manual_seed(1000 * dim + N + int(periodic))
    ins = [torch.randn(Z, N, dim, generator=g) for _ in range(3)] + [2 * torch.rand(Z, N, 3, generator=g) for _ in range(2)]
    r0sq = 0.2 + torch.rand(heads, generator=g)
    box = (2.2, 1.9, 2.7) if periodic else None
    cot = torch.randn(Z, N, dim, generator=g)
    ref_in = [t.clone().requires_grad_(True) for t in ins]
    ref_out = R.proxattn(*ref_in, r0sq, box)
    ref_grads = torch.autograd.grad((ref_out * cot).sum(), ref_in)
    out, grads = run(ins, r0sq, box, cot)
    close(out, ref_out)
    for mine, ref in zip(grads, ref_grads):
        close(mine, ref, rel=5e-5)


def test_empty_and_argument_errors():
    from ld_b200 import proxattn as PA
    r0sq = torch.tensor([0.5, 0.7]).cuda()
    e = torch.zeros(4, 0, 16).cuda()
    assert PA.proxattn(e, e, e, torch.zeros(4, 0, 3).cuda(), torch.zeros(4, 0, 3).cuda(), r0sq).shape == (4, 0, 16)
    q = torch.zeros(4, 8, 24).cuda()
    x = torch.zeros(4, 8, 3).cuda()
    with pytest.raises(RuntimeError, match="dim must be one of"):
        PA.proxattn(q, q, q, x, x, r0sq)
    q = torch.zeros(3, 8, 16).cuda()
    x = torch.zeros(3, 8, 3).cuda()
    with pytest.raises(RuntimeError, match="multiple of the number of heads"):
        PA.proxattn(q, q, q, x, x, r0sq)


def test_deterministic_and_linear_in_v():
    """size-independent properties on a larger case (Z = 8, N = 1500, dim = 64): bit-identical reruns, and
    linearity in V: out(V1 + V2) = out(V1) + out(V2) to rounding"""
    from ld_b200 import proxattn as PA
    g = torch.Generator().manual_seed(5)
    Z, N, dim = 8, 1500, 64
    q, k, v1, v2 = (torch.randn(Z, N, dim, generator=g).cuda() for _ in range(4))
    x, y = (3 * torch.rand(Z, N, 3, generator=g)).cuda(), (3 * torch.rand(Z, N, 3, generator=g)).cuda()
    r0sq = torch.tensor([0.3, 0.9]).cuda()
    a = PA.proxattn(q, k, v1, x, y, r0sq)
    assert torch.equal(a, PA.proxattn(q, k, v1, x, y, r0sq))
    b = PA.proxattn(q, k, v2, x, y, r0sq)
    close(PA.proxattn(q, k, v1 + v2, x, y, r0sq), a + b, rel=1e-5)


@pytest.mark.parametrize("dim", [16, 32, 64, 128])
@pytest.mark.parametrize("Z,N,heads", [(5, 1, 5), (4, 128, 2), (3, 130, 1), (6, 517, 3)])
@pytest.mark.parametrize("periodic", [False, True])
def test_tf32_tensor_core_forward(dim, Z, N, heads, periodic):
    """forward on the tensor cores in TF32 (10-bit mantissas on both products): 3e-3 of the largest output,
    the accuracy class of the reference's Triton kernel; the backward of that call is the FP32 one"""
    from ld_b200 import ops, proxattn as PA
    g = torch.Generator().manual_seed(77 * dim + N + int(periodic))
    ins = [torch.randn(Z, N, dim, generator=g) for _ in range(3)] + [2 * torch.rand(Z, N, 3, generator=g) for _ in range(2)]
    r0sq = 0.2 + torch.rand(heads, generator=g)
    box = (2.2, 1.9, 2.7) if periodic else None
    want = R.proxattn(*ins, r0sq, box)
    g_in = [t.cuda().requires_grad_(True) for t in ins]
    if periodic:
        got = PA.proxattn_periodic(*g_in, r0sq.cuda(), box, precision="tf32")
    else:
        got = PA.proxattn(*g_in, r0sq.cuda(), precision="tf32")
    close(got, want, rel=3e-3)
    assert int(ops.tc_status(got.device).item()) == 0
    cot = torch.randn(Z, N, dim, generator=g)
    grads = torch.autograd.grad((got * cot.cuda()).sum(), g_in)
    ref_in = [t.clone().requires_grad_(True) for t in ins]
    ref_grads = torch.autograd.grad((R.proxattn(*ref_in, r0sq, box) * cot).sum(), ref_in)
    for mine, ref in zip(grads, ref_grads):
        close(mine, ref, rel=5e-5)


def test_attention_modules_against_reference_golden():
    """ProbePoints2, ProximityFlashAttention and ProximityFlashAttentionPeriodic with the reference's state dicts
    against outputs of the reference's own classes (golden: its torch definition of the operator underneath), FP32
    kernels at 2e-5; the TF32 tensor-core forward at 3e-3; gradients flow to inputs and weights"""
    import os
    from ld_b200 import attention_layers as AL
    gold = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_golden_attention.pt"))
    adim, vdim, chan = gold["dims"]
    ax, vx, pos, pos2 = (gold[k].cuda() for k in ("ax", "vx", "pos", "pos2"))
    probe = AL.ProbePoints2(2, len(gold["r0_list"]), adim, vdim).cuda()
    probe.load_state_dict(gold["probe_state"])
    att = AL.ProximityFlashAttention(gold["r0_list"], adim, vdim, chan).cuda()
    att.load_state_dict(gold["att_state"])
    attp = AL.ProximityFlashAttentionPeriodic(gold["r0_list"], adim, vdim, chan).cuda()
    attp.load_state_dict(gold["attp_state"])
    with torch.no_grad():
        pts = probe(ax, vx, [pos, pos2])
        close(pts, gold["probe_out"], 2e-6)
        for got, want in zip(att(ax, vx, pts, pts + 0.1), gold["att_out"]):
            close(got, want, 2e-5)
        for got, want in zip(attp(ax, vx, pts, pts + 0.1, gold["box"]), gold["attp_out"]):
            close(got, want, 2e-5)
        att.precision = "tf32"
        for got, want in zip(att(ax, vx, pts, pts + 0.1), gold["att_out"]):
            close(got, want, 3e-3)
        att.precision = "fp32"
    axg = ax.clone().requires_grad_(True)
    ay, vy = att(axg, vx, pts, pts + 0.1)
    (ay.square().sum() + vy.square().sum()).backward()
    assert axg.grad is not None and torch.isfinite(axg.grad).all() and axg.grad.abs().max() > 0
    assert att.W_aq.grad is not None and torch.isfinite(att.W_aq.grad).all()
