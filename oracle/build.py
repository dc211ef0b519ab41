"""Compile the plain-C oracle (bi_oracle.c) into oracle/_build/liboracle.so with gcc.

Test infrastructure only. The reference project is Python with Metal kernel strings, so
there is no reference C/C++ source to compile next to it (no oracle/_ref).
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "bi_oracle.c"
OUT = HERE / "_build" / "liboracle.so"
# -ffp-contract=off: the only fused operations are the fmaf() calls the source spells out.
FLAGS = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-std=c11", "-Wall", "-fopenmp"]


def build(force: bool = False) -> Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    r = subprocess.run(["gcc", *FLAGS, str(SRC), "-o", str(OUT), "-lm"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
