"""Builds the C restatement of the oracle (oracle/attn_oracle_c.c -> oracle/_build/liboracle.so) with gcc.

Test infrastructure: the library is the timed CPU baseline of bench.py and is checked against the numpy oracle
by tests/test_oracle_c.py.  It is this repository's own port of the reference's algebra, not the reference compiled
(the reference's implementation of this path is HIP for an AMD GPU and cannot be built with gcc or nvcc).

    python -m oracle.build [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "attn_oracle_c.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "liboracle.so")


def build_oracle(force=False):
    if not os.path.exists(SRC):
        return LIB if os.path.exists(LIB) else None
    os.makedirs(OUT_DIR, exist_ok=True)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-o", LIB, SRC, "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return LIB


if __name__ == "__main__":
    print(build_oracle("--force" in sys.argv))
