"""Generates tests/golden/reference_golden_attention.pt from the REFERENCE's own Python on CPU:
managan/attention_layers.py (ProbePoints2, ProximityFlashAttention, ProximityFlashAttentionPeriodic; imported as they
are). Their Triton operators `proxattn` / `proxattn_periodic` need a GPU, so the module's two names are pointed at the
reference's own torch definitions of the same operators (`refimpl_proxattn` in managan/triton_kernels/proxattn.py and
proxattn_periodic.py). Only inputs, weights and outputs are stored.

    python tests/golden/make_golden_attention.py /path/to/learned-dynamics      (or set LD_REFERENCE_DIR)"""
import importlib
import os
import sys

import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LD_REFERENCE_DIR", "")
if not os.path.isdir(os.path.join(REF, "managan")):
    sys.exit("usage: make_golden_attention.py /path/to/learned-dynamics (a checkout of the reference repository)")
OUT = os.path.dirname(os.path.abspath(__file__))
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

al = importlib.import_module("managan.attention_layers")
pa = importlib.import_module("managan.triton_kernels.proxattn")
pap = importlib.import_module("managan.triton_kernels.proxattn_periodic")
al.proxattn = pa.refimpl_proxattn
al.proxattn_periodic = lambda Q, K, V, X, Y, r0sq, box: pap.refimpl_proxattn(Q, K, V, X, Y, r0sq, torch.tensor(box))

g = torch.Generator().manual_seed(515)
batch, nodes, adim, vdim, chan = 2, 37, 24, 16, 8
r0_list = [1.0, 2.5, 4.0]
box = (6.0, 7.0, 8.0)
ax = torch.randn(batch, nodes, adim, generator=g)
vx = torch.randn(batch, nodes, vdim, 3, generator=g)
pos = torch.rand(batch, nodes, 3, generator=g) * torch.tensor(box)
pos2 = pos + 0.3 * torch.randn(batch, nodes, 3, generator=g)


def init_all(mod, seed):
    torch.manual_seed(seed)
    mod.self_init()
    with torch.no_grad():        # the reference's self_init leaves the two output maps uninitialised
        for name in ("W_ao", "W_vo"):
            if hasattr(mod, name):
                getattr(mod, name).normal_(std=getattr(mod, name).shape[-1] ** -0.5)
    return mod


probe = init_all(al.ProbePoints2(2, len(r0_list), adim, vdim), 1)
torch.manual_seed(2)
with torch.no_grad():
    probe.lin_mix.weight.normal_(std=adim ** -0.5)
att = init_all(al.ProximityFlashAttention(r0_list, adim, vdim, chan), 3)
attp = init_all(al.ProximityFlashAttentionPeriodic(r0_list, adim, vdim, chan), 4)
with torch.no_grad():
    pts = probe(ax, vx, [pos, pos2])                       # (batch, heads, nodes, 3)
    ay, vy = att(ax, vx, pts, pts + 0.1)
    ayp, vyp = attp(ax, vx, pts, pts + 0.1, box)
out = {"ax": ax, "vx": vx, "pos": pos, "pos2": pos2, "r0_list": r0_list, "box": box, "dims": (adim, vdim, chan),
       "probe_state": {k: v.clone() for k, v in probe.state_dict().items()}, "probe_out": pts,
       "att_state": {k: v.clone() for k, v in att.state_dict().items()}, "att_out": (ay, vy),
       "attp_state": {k: v.clone() for k, v in attp.state_dict().items()}, "attp_out": (ayp, vyp)}
torch.save(out, os.path.join(OUT, "reference_golden_attention.pt"))
print("wrote", os.path.join(OUT, "reference_golden_attention.pt"))
