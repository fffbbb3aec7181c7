"""Build recipe for the oracle's C restatement (test infrastructure).

`python oracle/build.py` compiles oracle_c.c into oracle/liboracle_c.so with
strict floating point (no fast math, no FMA contraction), matching the reference
kernels' own build flags (kernels/exact-rowwise-int8/build_extension.py:12-19).

The reference's kernels themselves are HIP sources that need hipcc, the DTK
runtime and torch's HIP headers; none of that exists on this toolchain, so there
is no oracle/_ref build: the reference is treated as unbuildable here.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "oracle_c.c"
OUT = HERE / "liboracle_c.so"


def build(force: bool = False) -> Path:
    if OUT.exists() and not force and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    cmd = ["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           "-o", str(OUT), str(SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
