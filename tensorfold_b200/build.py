"""Builds the C-ABI CUDA library in-tree (``tensorfold_b200/lib/libtfb200.so``) with nvcc for sm_100a.

``python -m tensorfold_b200.build`` rebuilds it; nothing is built at import time, and there is no fallback: the
package's operators fail loudly when the library is missing.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "lib" / "libtfb200.so"
UNIT = CSRC / "tfb200.cu"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-shared"]


def sources() -> list[Path]:
    return sorted(p for p in CSRC.iterdir() if p.suffix in (".cu", ".cuh", ".h"))


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    return any(p.stat().st_mtime > built for p in sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel into one shared library; returns its path."""

    if not force and not stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built here")
    LIB.parent.mkdir(parents=True, exist_ok=True)
    tmp = LIB.with_suffix(".so.tmp")
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(tmp), str(UNIT)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr, file=sys.stderr)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
