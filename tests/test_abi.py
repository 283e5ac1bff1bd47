"""The C-ABI library loads without a GPU and exports every symbol include/ld_hotpath.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ld_hotpath.h")).read()
    return sorted(set(re.findall(r"\b(ld_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from ld_b200.build import build_library
    from ld_b200 import _lib
    path = build_library()
    L = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 19
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/ld_hotpath.h but not exported"
    # the Python binding covers the same set
    bound = set(_lib.SIGNATURES) | {"ld_last_error", "ld_status_string", "ld_packed_weight_elems"}
    assert set(names) == bound, set(names) ^ bound


def test_status_strings():
    from ld_b200 import _lib
    L = _lib.lib()
    assert L.ld_status_string(0) == b"ok"
    assert b"cutoff" in L.ld_status_string(_lib.LD_ERR_BOX_TOO_SMALL)


def test_argument_errors_without_gpu():
    """pure host-side validation paths (no kernel launch)"""
    import ctypes as C
    from ld_b200 import _lib
    L = _lib.lib()
    n = C.c_size_t(0)
    box = (C.c_float * 3)(5.0, 5.0, 5.0)
    rc = L.ld_radius_graph_workspace_size(2, 10, 1, 3.0, C.cast(box, C.c_void_p), 0, 0, C.byref(n))
    assert rc == _lib.LD_ERR_BOX_TOO_SMALL
    rc = L.ld_radius_graph_workspace_size(2, 10, 1, 1.0, C.cast(box, C.c_void_p), 0, 0, C.byref(n))
    assert rc == 0 and n.value > 0
    rc = L.ld_radius_graph_workspace_size(2, 10, 0, 1.0, None, 1, 0, C.byref(n))
    assert rc == _lib.LD_ERR_SHAPE  # reference-compatible grid is periodic only
    assert L.ld_tensor_linear(3, None, 1, 1, None, None, 4, 4, 4, None) == _lib.LD_ERR_UNSUPPORTED
