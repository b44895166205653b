"""In-tree build of the C-ABI CUDA library (sm_100a only).

``python -m slinoss_b200.build`` compiles ``csrc/*.cu`` with nvcc into
``slinoss_b200/_lib/libslinoss_b200.so``.  The library links only the CUDA
runtime (statically), exports the ``sl_*`` symbols declared in
``include/slinoss_b200.h`` and has no dependency on torch.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB_PATH = LIB_DIR / "libslinoss_b200.so"
SOURCES = ["abi.cu", "scan_simt.cu", "scan_tc.cu", "decode.cu", "scanprep_conv.cu", "mixer_tail.cu",
           "scan_bwd_static.cu", "mixer_step.cu", "ffn_rowwise.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xptxas=-v", "-Xcompiler", "-fPIC", "-Xcompiler",
    "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built.")


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        h.update(name.encode())
        h.update((CSRC / name).read_bytes())
    h.update((PKG.parent / "include" / "slinoss_b200.h").read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if sources changed; returns the path of the .so."""
    LIB_DIR.mkdir(exist_ok=True)
    stamp = LIB_DIR / "build.sha256"
    digest = _digest()
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == digest:
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in SOURCES:
        obj = LIB_DIR / (src + ".o")
        objs.append(str(obj))
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                            text=True)))
    log = []
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        log.append(f"==== {src}\n{out}")
        failed |= pr.returncode != 0
    (LIB_DIR / "build.log").write_text("\n".join(log))
    if verbose or failed:
        sys.stderr.write("\n".join(log))
    if failed:
        raise RuntimeError("nvcc failed; see slinoss_b200/_lib/build.log")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH), *objs]
    subprocess.run(link, check=True)
    stamp.write_text(digest)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
