"""The C-ABI library loads on a CPU-only host and exports every symbol ``include/tfb200.h`` declares."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared() -> list[str]:
    text = (ROOT / "include" / "tfb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tfb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared()
    assert {"tfb_router", "tfb_select_rows", "tfb_plan", "tfb_experts_run", "tfb_combine", "tfb_pack"} <= set(names)


def test_library_exports_every_declared_symbol():
    from tensorfold_b200 import build

    lib = ctypes.CDLL(str(build.build()))
    for name in declared():
        assert hasattr(lib, name), name


def test_binding_covers_the_header():
    from tensorfold_b200 import _lib

    bound = set(_lib.SIGNATURES) | {"tfb_last_error", "tfb_version", "tfb_set_pdl", "tfb_select_plan_max_rows",
                                     "tfb_set_wait_limit_ms", "tfb_route_max_rows", "tfb_decode_kslices"}
    assert set(declared()) == bound


def test_bad_arguments_are_refused_before_any_launch():
    from tensorfold_b200 import _lib

    with pytest.raises(ValueError, match="null pointer"):
        _lib.call("tfb_plan", 0, 0, 1, 16, 0, 0, 0, 0)
    with pytest.raises(ValueError, match="1..1024 experts"):
        _lib.call("tfb_select_rows", 8, 8, 8, 8, 1, 5000, 2, 0, 0)
    with pytest.raises(ValueError, match="groups of 64"):
        _lib.call("tfb_pack", 8, 8, 8, 32, 8, 1, 32, 64, 0)
