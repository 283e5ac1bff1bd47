"""Dense-weight l<=2 products (Ant16) and the TensorProds modules on the GPU: against vectors from the
reference's own einsum refimpl / classes (tests/golden) and against the CPU oracle at larger sizes.
Tolerance 1e-5 relative (FP32), gradients of weights 3e-5 (sums over the batch)."""
import pytest
import torch

from oracle import reference_math as R

pytestmark = pytest.mark.gpu
ORDER = ["000", "110", "220", "011", "101", "121", "211", "111", "022", "202", "112", "222", "212"]
SFX = {0: (), 1: (3,), 2: (3, 3)}


def close(a, b, rel=1e-5):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape
    if b.numel() == 0:
        return
    err = (a - b).abs().max().item()
    scale = max(b.abs().max().item(), 1e-30)
    assert err <= rel * scale + 1e-7, f"max abs err {err:.3e} vs scale {scale:.3e}"


def run_autograd(inputs, cotangents):
    from ld_b200.codegen_tensor_products import Ant16
    ins = [t.cuda().requires_grad_(True) for t in inputs]
    outs = Ant16.apply(*ins)
    grads = torch.autograd.grad(sum((y * c.cuda()).sum() for y, c in zip(outs, cotangents)), ins)
    return outs, grads


def test_ant16_golden(golden):
    a = golden["ant16"]
    outs, grads = run_autograd(a["inputs"], a["cotangents"])
    for mine, ref in zip(outs, a["outputs"]):
        close(mine, ref)
    for mine, ref in zip(grads, a["grads"]):
        close(mine, ref, rel=2e-5)


def make_inputs(nb, d0, d1, d2, dl, seed):
    g = torch.Generator().manual_seed(seed)
    dims = {0: d0, 1: d1, 2: d2}
    ins = [torch.randn(nb, dims[r], *SFX[r], generator=g) for r in (0, 1, 2)]
    for name in ORDER:
        rl, rr, ro = (int(ch) for ch in name)
        ins.append(torch.randn(dims[ro], dl, dims[rr], generator=g) * (dl * dims[rr]) ** -0.5)
        ins.append(torch.randn(nb, dl, *SFX[rl], generator=g))
    return ins


@pytest.mark.parametrize("shape", [(10, 64, 48, 32, 16), (1, 1, 1, 1, 1), (257, 32, 32, 16, 8), (0, 8, 8, 8, 4)])
def test_ant16_vs_oracle(shape):
    ins = make_inputs(*shape, seed=sum(shape))
    ref_in = [t.clone().requires_grad_(True) for t in ins]
    ref_out = R.ant16(*ref_in)
    g = torch.Generator().manual_seed(5)
    cot = [torch.randn(t.shape, generator=g) for t in ref_out]
    ref_grads = torch.autograd.grad(sum((y * c).sum() for y, c in zip(ref_out, cot)), ref_in)
    outs, grads = run_autograd(ins, cot)
    for mine, ref in zip(outs, ref_out):
        close(mine, ref)
    for mine, ref in zip(grads, ref_grads):
        close(mine, ref, rel=3e-5)


def test_ant16_chunked_rows(monkeypatch):
    """a small scratch bound forces several row chunks; results must not depend on the chunking"""
    from ld_b200 import ant16
    ins = make_inputs(300, 16, 16, 8, 4, seed=9)
    g = torch.Generator().manual_seed(6)
    ref_out = R.ant16(*ins)
    cot = [torch.randn(t.shape, generator=g) for t in ref_out]
    whole = run_autograd(ins, cot)
    monkeypatch.setattr(ant16, "SCRATCH_BYTES", 64 << 10)
    parts = run_autograd(ins, cot)
    for a, b in zip(whole[0] + tuple(whole[1]), parts[0] + tuple(parts[1])):
        close(a, b, rel=3e-5)
    for mine, ref in zip(parts[0], ref_out):
        close(mine, ref)


def test_dropin_entry_points_match_reference_order(golden):
    """the sixteen codegen_tensops_cuda names: forward groups and the chiral backward's zero dx_2"""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "learned-dynamics_b200", "dropin"))
    import codegen_tensops_cuda as cg
    a = golden["ant16"]
    ins = [t.cuda() for t in a["inputs"]]
    x_0, x_1, x_2 = ins[:3]
    pl = ins[3:]
    y_0, = cg.ant16_o0_cuda(x_0, x_1, x_2, *pl[0:6])
    y_1, = cg.ant16_o1_cuda(x_0, x_1, x_2, *pl[6:14])
    y_1c, y_2c = cg.ant16_oc_cuda(x_1, x_2, *pl[14:16], *pl[24:26])
    y_2, = cg.ant16_o2_cuda(x_0, x_1, x_2, *pl[16:24])
    close(y_0, a["outputs"][0])
    close(y_1 + y_1c, a["outputs"][1])
    close(y_2 + y_2c, a["outputs"][2])
    dx_1, dx_2 = cg.ant16_oc_backward_cuda(a["cotangents"][1].cuda(), a["cotangents"][2].cuda(), *pl[14:16], *pl[24:26])
    assert dx_1.shape == x_1.shape and dx_2.shape == x_2.shape and float(dx_2.abs().max()) == 0.0
    with pytest.raises(RuntimeError):
        cg.ant16_o0_cuda(x_0.cpu(), x_1, x_2, *pl[0:6])
    with pytest.raises(RuntimeError):
        cg.ant16_o0_cuda(x_0, x_1, x_2, pl[0], pl[1][:, :2], *pl[2:6])


def test_avd_tensor_prods_golden(golden):
    from ld_b200.tensor_products import AVDFullTensorProds
    a = golden["avd_tensor_prods"]
    mod = AVDFullTensorProds(*a["dims"]).cuda()
    mod.load_state_dict(a["state"])
    with torch.no_grad():
        outs = mod(*[t.cuda() for t in a["inputs"]])
    for mine, ref in zip(outs, a["out"]):
        close(mine, ref, rel=2e-5)


@pytest.mark.parametrize("ranks", [(0, 0, 0), (1, 0, 1), (1, 1, 0), (1, 1, 2), (2, 0, 2), (2, 1, 1), (2, 2, 0), (2, 2, 2),
                                   (0, 1, 1), (1, 2, 1), (2, 1, 3), (2, 2, 4), (0, 2, 2), (1, 2, 3)])
def test_tensor_prod_bare_forward_backward(ranks):
    from ld_b200.tensor_products import TensorProdBare
    il, ir, io = ranks
    g = torch.Generator().manual_seed(il * 9 + ir * 3 + io)
    x_l = torch.randn(7, 33, *([3] * il), generator=g)
    x_r = torch.randn(7, 33, *([3] * ir), generator=g)
    xl_r, xr_r = x_l.clone().requires_grad_(True), x_r.clone().requires_grad_(True)
    y_ref = R.tensor_prod_bare(il, ir, io, xl_r, xr_r)
    cot = torch.randn(y_ref.shape, generator=g)
    y_ref.backward(cot)
    xl_g, xr_g = x_l.cuda().requires_grad_(True), x_r.cuda().requires_grad_(True)
    y = TensorProdBare(il, ir, io)(xl_g, xr_g)
    y.backward(cot.cuda())
    close(y, y_ref)
    close(xl_g.grad, xl_r.grad)
    close(xr_g.grad, xr_r.grad)
