"""CPU check of the product / adjoint / radial formulas shared with the CUDA kernels (tp_math.h)."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import reference_math as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# field order of struct BeeOut: scalar outputs, then rank-1, rank-2, then the two Levi-Civita products
SIZES = [1, 1, 1, 3, 3, 3, 3, 9, 9, 9, 9, 3, 9]


@pytest.fixture(scope="module")
def host(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("tp") / "libhost_tp.so")
    subprocess.check_call(["g++", "-O1", "-ffp-contract=off", "-fPIC", "-shared", "-I",
                           os.path.join(ROOT, "learned-dynamics_b200", "csrc"), "-o", so,
                           os.path.join(ROOT, "tests", "host_tp_math.cpp")])
    return ctypes.CDLL(so)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _operands(n, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, 1, *([3] * l), generator=g) for l in (0, 1, 2, 0, 1, 2)]


def test_bee_forward_matches_einsum(host):
    n = 50
    ops = _operands(n, 0)
    ref = torch.cat([t.reshape(n, -1) for t in R.bee(*ops)], dim=1).numpy()
    arrs = [np.ascontiguousarray(t.numpy().reshape(n, -1)) for t in ops]
    out = np.zeros((n, 63), dtype=np.float32)
    host.host_bee_fwd(*[_p(a) for a in arrs], n, _p(out))
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("left", [1, 0])
def test_bee_adjoints_match_autograd(host, left):
    n = 40
    ops = [t.requires_grad_(True) for t in _operands(n, 1)]
    ys = R.bee(*ops)
    g = torch.Generator().manual_seed(2)
    gy = [torch.randn(y.shape, generator=g) for y in ys]
    sum((y * q).sum() for y, q in zip(ys, gy)).backward()
    want = ops[0:3] if left else ops[3:6]
    given = ops[3:6] if left else ops[0:3]
    ref = torch.cat([t.grad.reshape(n, -1) for t in want], dim=1).numpy()
    gflat = np.ascontiguousarray(torch.cat([q.reshape(n, -1) for q in gy], dim=1).numpy())
    arrs = [np.ascontiguousarray(t.detach().numpy().reshape(n, -1)) for t in given]
    d = np.zeros((n, 13), dtype=np.float32)
    host.host_bee_bw(left, *[_p(a) for a in arrs], _p(gflat), n, _p(d))
    np.testing.assert_allclose(d, ref, rtol=1e-5, atol=1e-5)


def test_radial_features(host):
    d = np.linspace(0.0, 6.0, 97, dtype=np.float32)
    r = torch.zeros(97, 3)
    r[:, 0] = torch.from_numpy(d)
    for kind, fn, n, rmax in ((0, R.radial_encode_painn, 16, 3.0), (0, R.radial_encode_painn, 7, 5.0),
                              (1, R.radial_encode_gaussian, 8, 3.0), (1, R.radial_encode_gaussian, 16, 5.0)):
        out = np.zeros((97, n), dtype=np.float32)
        host.host_radial(kind, n, ctypes.c_float(rmax), _p(d), 97, _p(out))
        np.testing.assert_allclose(out, fn(r, n, rmax).numpy(), rtol=1e-5, atol=2e-6)
