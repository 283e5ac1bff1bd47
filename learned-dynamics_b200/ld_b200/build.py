"""Builds libld_hotpath.so (all CUDA kernels + the C ABI) in-tree with nvcc for sm_100a.

Every .cu under csrc/ is compiled to an object file of its own (in parallel, only when the source
or a header is newer than the object) and the objects are linked into one shared library."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libld_hotpath.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


# LD_PHASE_COUNTERS=1 in the environment selects the diagnostics variant (cycle counters inside the fused tensor-core
# kernels): a library of its own, built and loaded only while the variable is set
if os.environ.get("LD_PHASE_COUNTERS", "0") == "1":
    NVCC_FLAGS.append("-DLD_PHASE_COUNTERS")
    OBJ_DIR = os.path.join(CSRC, "build_prof")
    LIB_PATH = os.path.join(HERE, "libld_hotpath_prof.so")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]


def _obj(src):
    return os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")


def build_library(force=False, verbose=False):
    """Compile every .cu under csrc/ and link them into one shared library. Returns its path."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = max(os.path.getmtime(h) for h in _headers())
    todo = []
    for src in sources():
        obj = _obj(src)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            todo.append(src)
    objs = [_obj(s) for s in sources()]
    if not todo and os.path.exists(LIB_PATH) and all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(o) for o in objs):
        return LIB_PATH

    def compile_one(src):
        cmd = [nvcc, "-c", "-o", _obj(src)] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [src]
        return src, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, todo))
    failed = [(s, r) for s, r in results if r.returncode != 0]
    for s, r in results:
        if r.returncode != 0 or verbose:
            sys.stderr.write(f"==== {os.path.basename(s)}\n" + r.stdout + r.stderr)
    if failed:
        raise RuntimeError("nvcc failed on " + ", ".join(os.path.basename(s) for s, _ in failed))
    res = subprocess.run([nvcc, "-shared", "-o", LIB_PATH] + NVCC_FLAGS + objs + ["-lcudart"], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libld_hotpath.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="-f" in sys.argv, verbose="-v" in sys.argv))
