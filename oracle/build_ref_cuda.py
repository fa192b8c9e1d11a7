"""TEST INFRASTRUCTURE: compiles the REFERENCE's own CUDA extension for the grouped 4-bit experts, for sm_100, into
``oracle/_ref/``.

The reference builds ``experts.cpp``, ``experts.cu``, ``experts_prefill.cu`` and ``experts_pack.cu``
(``src/tensorfold/cuda/experts.py:18-25``) with torch's JIT for the GPU present (``src/tensorfold/cuda/build.py:49-69``:
``-gencode=arch=compute_XY,code=sm_XY`` of that GPU, ``-O3``).  This recipe runs the same torch build on the same four
files where they lie under the mounted reference tree, for ``compute_100`` / ``sm_100`` - what that build would pick on a
B200 - and leaves the module in ``oracle/_ref/experts_ext/``.  It is the reference's kernels recompiled, unmodified:
the second, device-side checker of the parity tests (``tests/test_reference_cuda_gpu.py``) and the "reference kernels on
the same GPU" figure of ``bench.py``.  Nothing of the reference is copied into the repository (``oracle/_ref/`` is
git-ignored); where the reference tree is not mounted (the GPU box) this is a no-op and the prebuilt module is used.
"""

from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref" / "experts_ext"
NAME = "tf_reference_experts"
REFERENCE = Path(os.environ.get("TENSORFOLD_REFERENCE", "/root/reference"))
SOURCES = [REFERENCE / "src/tensorfold/cuda" / f for f in ("experts.cpp", "experts.cu", "experts_prefill.cu",
                                                           "experts_pack.cu")]


def module_path() -> Path:
    return OUT_DIR / f"{NAME}.so"


def build(force: bool = False) -> Path | None:
    """Build (or find) the module; returns its path, or None when it can be neither built nor found."""

    out = module_path()
    if not all(s.exists() for s in SOURCES):
        return out if out.exists() else None
    newest = max(s.stat().st_mtime for s in SOURCES)
    if out.exists() and out.stat().st_mtime >= newest and not force:
        return out
    from torch.utils import cpp_extension

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    was = os.environ.get("TORCH_CUDA_ARCH_LIST")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"       # one architecture: the B200's (no GPU is needed to compile)
    try:
        cpp_extension.load(name=NAME, sources=[str(s) for s in SOURCES], extra_cuda_cflags=["-O3"],
                           build_directory=str(OUT_DIR), with_cuda=True, is_python_module=False, verbose=False)
    finally:
        if was is None:
            os.environ.pop("TORCH_CUDA_ARCH_LIST", None)
        else:
            os.environ["TORCH_CUDA_ARCH_LIST"] = was
    return out if out.exists() else None


def load():
    """The built module (``pack``, ``plan``, ``run``, ``prefill``), or None when it was never built."""

    path = module_path()
    if not path.exists():
        return None
    import torch  # noqa: F401  (the module links against torch's libraries)

    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[NAME] = mod
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
