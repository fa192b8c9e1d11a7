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


def test_new_entry_points_refuse_bad_arguments_before_any_launch():
    """The entry points added beside the reference's four (fused forms, EXL3 launches, the rows either side of the
    path): a bad argument is refused by name, with no CUDA call made (this runs without a GPU)."""

    from tensorfold_b200 import _lib

    cases = [
        ("tfb_add_moe_norm", (16, 16, 0, 16, 16, 16, 16, 16, 1, 100, 4, 2, 1e-5, 0), "multiple of 64"),
        ("tfb_add_moe_norm", (16, 16, 0, 16, 16, 16, 16, 16, 1, 128, 4, 5, 1e-5, 0), "5 routed of 4 slots"),
        ("tfb_add_moe_norm", (0, 16, 0, 16, 16, 16, 16, 16, 1, 128, 4, 2, 1e-5, 0), "null pointer"),
        ("tfb_exl3_rot_out", (16, 16, 0, 16, 100, 0, 1, 128, 0), "rows at least N apart"),
        ("tfb_exl3_rot_out", (16, 16, 0, 16, 128, 3, 1, 128, 0), "out_type"),
        ("tfb_experts_run_slices", (64, 16, 64, 0, 16, 1, 1, 16, 16, 16, 16, 32, -1, 1, 0, 8, 0), "bad row count"),
        ("tfb_experts_run_tile", (64, 4, 16, 64, 0, 16, 1, 1, 16, 16, 16, 16, 32, 0.0, 1, 0, 8, 0), "no kernel for epilogue 4"),
        ("tfb_exl3_prologue", (16, 128, 0, 16, 16, 0, 16, 0, 1, 128, 1, 4, 7, 16, 16, 16, 16, 0, 0, 0, 0, 0, 0),
         "sort is 0"),
        ("tfb_exl3_prologue", (16, 128, 0, 16, 16, 0, 16, 0, 1, 128, 1, 4, 16, 16, 16, 16, 16, 0, 0, 0, 16, 4, 0),
         "the width order needs"),
        ("tfb_exl3_down", (16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 128, 128, 1, 0, 1, 0, 24, 0, 4, 0), "items of 16 or 32"),
        ("tfb_exl3_down", (16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 128, 128, 1, 0, 1, 0, 16, 0, 3, 0), "column tiles"),
        ("tfb_exl3_down", (16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 128, 128, 1, 0, 1, 0, 16, 40, 4, 0), "k2_all"),
    ]
    for name, args, why in cases:
        with pytest.raises(ValueError, match=why):
            _lib.call(name, *args)
    assert _lib.lib().tfb_decode_kslices(32) == 4 and _lib.lib().tfb_decode_kslices(12) == 2
    assert _lib.lib().tfb_decode_kslices(4) == 1
