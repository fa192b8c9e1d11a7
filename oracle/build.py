"""TEST INFRASTRUCTURE: compiles the C restatements (``cpu_moe.c``, ``cpu_exl3.c``) into
``oracle/lib/liboracle_cpu.so`` with gcc."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRCS = [HERE / "cpu_moe.c", HERE / "cpu_exl3.c"]
LIB = HERE / "lib" / "liboracle_cpu.so"

# x86-64-v3 (AVX2 + FMA) rather than -march=native: the library is built in one container and run on another host.
CFLAGS = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared", "-std=c11"]


def build(force: bool = False) -> Path:
    if not force and LIB.exists() and all(LIB.stat().st_mtime >= src.stat().st_mtime for src in SRCS):
        return LIB
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found: the CPU oracle cannot be built")
    LIB.parent.mkdir(parents=True, exist_ok=True)
    tmp = LIB.with_suffix(".so.tmp")
    proc = subprocess.run([gcc, *CFLAGS, "-o", str(tmp), *map(str, SRCS), "-lm"], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("gcc failed:\n" + proc.stdout + proc.stderr)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
