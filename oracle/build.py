"""Build recipe for the CPU oracle (test infrastructure, never imported by the package).

`python -m oracle.build` compiles oracle/bm_oracle.c into oracle/libbm_oracle.so.
The flags matter for parity:
  -ffp-contract=off   gcc must not fuse a*b+c on its own; every fused
                      multiply-add in the oracle is an explicit fmaf()
  -march=x86-64-v3    fmaf() becomes one vfmadd instruction (hardware FMA is
                      exact by definition, so the result does not depend on it,
                      only the speed does) and the int8 dot products vectorise
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "bm_oracle.c")
OUT = os.path.join(HERE, "libbm_oracle.so")
HDR = os.path.join(HERE, "..", "bitmtp_b200", "csrc", "bm_math.h")


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(p) > t for p in (SRC, HDR, __file__))


def build_oracle(force: bool = False, verbose: bool = False) -> str:
    """Compile the oracle if its sources are newer than the library; return the .so path."""
    if not force and not _stale():
        return OUT
    # The system gcc ships libgomp; a $CC wrapper may not, so it is not consulted.
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    cmd = [
        cc, "-O3", "-std=gnu11", "-fopenmp", "-fPIC", "-shared",
        "-ffp-contract=off", "-fno-fast-math", "-march=x86-64-v3", "-fvisibility=hidden",
        "-Wall", "-Wno-unknown-pragmas", SRC, "-o", OUT + ".tmp", "-lm",
    ]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    os.replace(OUT + ".tmp", OUT)
    return OUT


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv, verbose=True))
