"""Builds the C/OpenMP oracle port into oracle/_build/liboracle_v2x2ssd.so (gcc).

There is nothing to compile from the reference itself for this path (it is pure
Python/torch; its only native code is the vendored causal-conv1d CUDA extension),
so no ``oracle/_ref`` artefact exists.
"""

from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "csrc" / "v2x2ssd_cpu.c"
OUT = HERE / "_build" / "liboracle_v2x2ssd.so"


def build(force: bool = False) -> Path:
    OUT.parent.mkdir(exist_ok=True)
    if force or not OUT.exists() or OUT.stat().st_mtime < SRC.stat().st_mtime:
        subprocess.run(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c11",
                        str(SRC), "-o", str(OUT)], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
