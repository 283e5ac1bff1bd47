"""Generates tests/golden/reference_golden_radial.pt from the REFERENCE's own Python on CPU:
managan/layers_common.py (radial_encode, VecLinear; imported as it is) and radial_encode_edge of
archs/diffuser_atoms5.py (the function definition alone is compiled from the file by AST, because
importing that arch needs the CUDA-only extension modules). Only inputs, weights and outputs are stored.

    python tests/golden/make_golden_radial.py /path/to/learned-dynamics      (or set LD_REFERENCE_DIR)"""
import ast
import os
import sys

import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LD_REFERENCE_DIR", "")
if not os.path.isdir(os.path.join(REF, "managan")):
    sys.exit("usage: make_golden_radial.py /path/to/learned-dynamics (a checkout of the reference repository)")
OUT = os.path.dirname(os.path.abspath(__file__))
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

import managan.layers_common as lcm  # noqa: E402

ns = {"torch": torch}
tree = ast.parse(open(os.path.join(REF, "archs/diffuser_atoms5.py")).read())
for node in ast.walk(tree):
    if isinstance(node, ast.FunctionDef) and node.name == "radial_encode_edge":
        exec(compile(ast.Module(body=[node], type_ignores=[]), "<reference radial_encode_edge>", "exec"), ns)
radial_encode_edge = ns["radial_encode_edge"]

g = torch.Generator().manual_seed(2024)
r_vec = torch.randn(257, 3, generator=g) * 1.5          # some beyond rmax: the envelope clamps them to zero
r_len = torch.rand(5, 61, generator=g) * 1.2
torch.manual_seed(7)
vl = lcm.VecLinear(24, 40)
vl.self_init()
v_in = torch.randn(3, 17, 24, 3, generator=g)
with torch.no_grad():
    out = {
        "r_vec": r_vec, "r_len": r_len,
        "edge_n8_rmax4": radial_encode_edge(r_vec, 8, 4.0),
        "edge_n16_rmax2p5": radial_encode_edge(r_vec, 16, 2.5),
        "cos_n8": lcm.radial_encode(r_len, 8, 1.0),
        "cos_n12": lcm.radial_encode(r_len, 12, 3.0),
        "veclinear_state": {k: v.clone() for k, v in vl.state_dict().items()},
        "veclinear_in": v_in, "veclinear_out": vl(v_in),
    }
torch.save(out, os.path.join(OUT, "reference_golden_radial.pt"))
print("wrote", os.path.join(OUT, "reference_golden_radial.pt"))
