"""TEST INFRASTRUCTURE: compiles the REFERENCE's own packed-code header as C++ into ``oracle/_ref/``.

The reference keeps its bit-extraction expression in a Metal header held as a Python string
(``src/tensorfold/kernels/qwen/dense/v1/affine_rows.py:12-24``, ``_HEADER``); its own test compiles that string as
plain C++ behind a small shim (``tests/test_affine_rows.py:82-101``).  This script does the same from the source where
it lies under the mounted reference tree: the string is read with ``ast`` (the module itself needs MLX), written to a
temporary file and compiled to ``oracle/_ref/libaffine_header.so`` exporting ``decode(words, index, bits)``.
Nothing of the reference is copied into the repository: ``oracle/_ref/`` is git-ignored.  Where the reference tree is
not mounted (the GPU box) this is a no-op and the prebuilt file, if any, is used.
"""

from __future__ import annotations

import ast
import os
import shutil
import subprocess
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "libaffine_header.so"
# the reference checkout: $TENSORFOLD_REFERENCE, else a folder named "reference" beside this repository
REFERENCE = Path(os.environ.get("TENSORFOLD_REFERENCE") or HERE.parents[1] / "reference")
SOURCE = REFERENCE / "src/tensorfold/kernels/qwen/dense/v1/affine_rows.py"
BITS = (2, 3, 4, 5, 6, 8)

SHIM = ("#include <cstdint>\n#include <cstring>\nusing uint = std::uint32_t;\n#define device\n#define thread\n"
        "template <typename T, typename U> T as_type(U u) { T t; std::memcpy(&t, &u, sizeof t); return t; }\n")


def header_text() -> str:
    tree = ast.parse(SOURCE.read_text())
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(getattr(t, "id", "") == "_HEADER" for t in node.targets):
            return ast.literal_eval(node.value)
    raise RuntimeError(f"{SOURCE}: no _HEADER string")


def build(force: bool = False) -> Path | None:
    if not SOURCE.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force:
        return OUT
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        return None
    switches = "".join(f"case {b}: return code_at<{b}>(words + index / 32 * {b}, index % 32);" for b in BITS)
    text = (SHIM + header_text() + '\nextern "C" uint decode(const uint* words, int index, int bits) { switch(bits) {'
            + switches + "default: return 0;} }\n")
    OUT.parent.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "header.cpp"
        src.write_text(text)
        subprocess.run([cxx, "-std=c++17", "-shared", "-fPIC", "-O1", str(src), "-o", str(OUT)], check=True,
                       capture_output=True, timeout=60)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
