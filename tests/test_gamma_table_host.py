"""The fused l<=2 edge kernel forms the 63 product components of an (edge, channel) as one small matrix product with a
13 x 63 matrix of monomials of the edge direction. This checks that table (exported by the library, no GPU needed)
against the reference's einsum definitions of the Bee products (managan/codegen_tensor_products.py:235-249) with right
operands (pa, pa * rhat, pa * rhat rhat^T), as Messages.forward builds them (archs/diffuser_atoms15.py:239-243)."""
import ctypes

import torch

from oracle import reference_math as R


def test_gamma_table_reproduces_bee_products():
    from ld_b200 import _lib
    buf = (ctypes.c_int * (4 * 128))()
    n = _lib.lib().ld_bee_gamma_table(ctypes.cast(buf, ctypes.c_void_p))
    assert n == 115
    ent = [tuple(buf[4 * i: 4 * i + 4]) for i in range(n)]
    assert len({(o, m) for o, m, _, _ in ent}) == n          # one entry per position
    g = torch.Generator().manual_seed(0)
    rows, chan = 7, 5
    l0 = torch.randn(rows, chan, generator=g, dtype=torch.float64)
    l1 = torch.randn(rows, chan, 3, generator=g, dtype=torch.float64)
    l2 = torch.randn(rows, chan, 3, 3, generator=g, dtype=torch.float64)
    pa = torch.randn(rows, chan, generator=g, dtype=torch.float64)
    rh = torch.randn(rows, 3, generator=g, dtype=torch.float64) * 0.5
    # monomials in the kernel's order: 1, r_x, r_y, r_z, then r_x r_y for (x, y) = 00, 01, 02, 11, 12, 22
    mono = torch.stack([torch.ones(rows, dtype=torch.float64), rh[:, 0], rh[:, 1], rh[:, 2], rh[:, 0] * rh[:, 0],
                        rh[:, 0] * rh[:, 1], rh[:, 0] * rh[:, 2], rh[:, 1] * rh[:, 1], rh[:, 1] * rh[:, 2],
                        rh[:, 2] * rh[:, 2]], dim=1)
    G = torch.zeros(rows, 16, 64, dtype=torch.float64)
    for o, m, k, neg in ent:
        G[:, m, o] = -mono[:, k] if neg else mono[:, k]
    left = torch.cat([l0[..., None], l1, l2.reshape(rows, chan, 9), torch.zeros(rows, chan, 3, dtype=torch.float64)], dim=-1)
    D = pa[..., None] * torch.einsum("rcm, rmo -> rco", left, G)
    phi_v = pa[..., None] * rh[:, None, :]
    phi_d = pa[..., None, None] * rh[:, None, None, :] * rh[:, None, :, None]
    (y000, y110, y220, y011, y101, y121, y211, y022, y202, y112, y222, y111, y212) = R.bee(l0, l1, l2, pa, phi_v, phi_d)
    want = torch.cat([y000[..., None], y110[..., None], y220[..., None], y011, y101, y121, y211, y111,
                      y022.reshape(rows, chan, 9), y202.reshape(rows, chan, 9), y112.reshape(rows, chan, 9),
                      y222.reshape(rows, chan, 9), y212.reshape(rows, chan, 9)], dim=-1)
    assert torch.allclose(D[..., :63], want, rtol=1e-12, atol=1e-12)
    assert torch.all(D[..., 63] == 0)
