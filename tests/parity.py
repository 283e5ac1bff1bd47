"""Comparison helpers shared by the GPU parity tests.

`close` is a max-norm check: max|a - b| <= rel * max|b|. It bounds the error relative to the largest
entry of the expected tensor, so entries much smaller than that are checked in absolute terms only.
`close_elem` adds an element-wise check, |a - b| <= rtol * |b| + atol_rel * max|b| for every entry."""
import torch


def rel_err(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape, (a.shape, b.shape)
    return (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)


def close(a, b, rel):
    e = rel_err(a, b)
    assert e <= rel, f"max-norm relative error {e:.3e} > {rel:.1e}"
    return e


def close_elem(a, b, rtol, atol_rel):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape, (a.shape, b.shape)
    scale = max(b.abs().max().item(), 1e-30)
    excess = (a - b).abs() - (rtol * b.abs() + atol_rel * scale)
    assert excess.max().item() <= 0, f"element-wise check failed by {excess.max().item():.3e} (scale {scale:.3e})"
