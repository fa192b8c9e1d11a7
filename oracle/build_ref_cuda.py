"""TEST INFRASTRUCTURE: compiles the REFERENCE's own CUDA extensions for the grouped 4-bit experts and for the routed
EXL3 experts, for sm_100, into ``oracle/_ref/``.

The reference builds ``experts.cpp``, ``experts.cu``, ``experts_prefill.cu`` and ``experts_pack.cu``
(``src/tensorfold/cuda/experts.py:18-25``) with torch's JIT for the GPU present (``src/tensorfold/cuda/build.py:49-69``:
``-gencode=arch=compute_XY,code=sm_XY`` of that GPU, ``-O3``).  This recipe runs the same torch build on the same four
files where they lie under the mounted reference tree, for ``compute_100`` / ``sm_100`` - what that build would pick on a
B200 - and leaves the module in ``oracle/_ref/experts_ext/``; the EXL3 extension (``src/tensorfold/cuda/exl3/experts.py:
24-30``: ``experts.cpp``, ``experts.cu``, ``experts_cb0/1/2.cu``) goes to ``oracle/_ref/exl3_ext/`` the same way.  They
are the reference's kernels recompiled, unmodified:
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
# the reference checkout: $TENSORFOLD_REFERENCE, else a folder named "reference" beside this repository
REFERENCE = Path(os.environ.get("TENSORFOLD_REFERENCE") or HERE.parents[1] / "reference")
CUDA = REFERENCE / "src/tensorfold/cuda"
# target -> (module name, build directory, sources)
TARGETS = {
    "experts": ("tf_reference_experts", HERE / "_ref" / "experts_ext",
                [CUDA / f for f in ("experts.cpp", "experts.cu", "experts_prefill.cu", "experts_pack.cu")]),
    "exl3": ("tf_reference_exl3", HERE / "_ref" / "exl3_ext",
             [CUDA / "exl3" / f for f in ("experts.cpp", "experts.cu", "experts_cb0.cu", "experts_cb1.cu",
                                          "experts_cb2.cu")]),
}


def module_path(target: str = "experts") -> Path:
    name, out_dir, _ = TARGETS[target]
    return out_dir / f"{name}.so"


def build(target: str = "experts", force: bool = False) -> Path | None:
    """Build (or find) a module; returns its path, or None when it can be neither built nor found."""

    name, out_dir, sources = TARGETS[target]
    out = module_path(target)
    if not all(s.exists() for s in sources):
        return out if out.exists() else None
    newest = max(s.stat().st_mtime for s in sources)
    if out.exists() and out.stat().st_mtime >= newest and not force:
        return out
    from torch.utils import cpp_extension

    out_dir.mkdir(parents=True, exist_ok=True)
    was = os.environ.get("TORCH_CUDA_ARCH_LIST")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"       # one architecture: the B200's (no GPU is needed to compile)
    try:
        cpp_extension.load(name=name, sources=[str(s) for s in sources], extra_cuda_cflags=["-O3"],
                           build_directory=str(out_dir), with_cuda=True, is_python_module=False, verbose=False)
    finally:
        if was is None:
            os.environ.pop("TORCH_CUDA_ARCH_LIST", None)
        else:
            os.environ["TORCH_CUDA_ARCH_LIST"] = was
    return out if out.exists() else None


def load(target: str = "experts"):
    """A built module (experts: ``pack``, ``plan``, ``run``, ``prefill``; exl3: ``grouped``, ``dequant``, ``group``,
    ``rot_in``, ``gateup_epilogue``, ``down_epilogue``, ``combine``, ``down_combine``), or None when never built."""

    path = module_path(target)
    if not path.exists():
        return None
    import torch  # noqa: F401  (the module links against torch's libraries)

    name = TARGETS[target][0]
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    for t in TARGETS:
        print(t, build(t, force="--force" in sys.argv))
