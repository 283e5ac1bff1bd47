"""TEST INFRASTRUCTURE ONLY. Compiles the C restatement of the radius-graph predicate into
oracle/liboracle.so (gcc, no FMA contraction)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build(force=False):
    src = os.path.join(HERE, "radius_graph_oracle.c")
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-o", LIB, src, "-lm"])
    return LIB


if __name__ == "__main__":
    print(build(force=True))
