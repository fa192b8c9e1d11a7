"""ctypes binding of the C-ABI library (``include/tfb200.h``).  No CPU path exists behind these calls."""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from functools import lru_cache
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtfb200.so"

ERR_ARG, ERR_CUDA, ERR_DEVICE = -1, -2, -3

P, I, L, F = c_void_p, c_int, c_int64, c_float

# name -> argument types (every entry point returns int status, except tfb_last_error / tfb_version / tfb_set_pdl)
SIGNATURES: dict[str, tuple] = {
    "tfb_router": (P, L, P, P, I, I, I, P),
    "tfb_router_prompt": (P, L, P, P, I, I, I, P),
    "tfb_select_rows": (P, I, P, P, I, I, I, I, P),
    "tfb_select_sigmoid": (P, I, P, P, P, I, I, I, I, F, I, P),
    "tfb_plan": (P, L, I, I, P, P, P, P),
    "tfb_select_plan": (P, I, P, P, I, I, I, I, I, P, P, P, P),
    "tfb_select_plan_window": (P, I, P, P, I, I, I, I, I, I, I, P, P, P, P),
    "tfb_plan_window": (P, L, I, I, I, P, P, P, P),
    "tfb_route": (P, L, P, P, I, I, I, I, I, I, P, P, I, I, I, P, P, P, P, P),
    "tfb_experts_down_combine": (I, P, L, P, I, I, P, P, P, P, I, L, I, I, P, I, P, I, P, P),
    "tfb_plan_split": (P, L, I, I, I, I, I, P, P, P, P, P, P),
    "tfb_combine_window": (P, I, P, P, I, I, P, I, I, I, I, P),
    "tfb_combine": (P, I, P, P, I, I, I, I, P),
    "tfb_add_moe_norm": (P, P, I, P, P, P, P, P, I, I, I, I, F, P),
    "tfb_pack": (P, P, P, I, P, I, I, I, P),
    "tfb_unpack": (P, I, P, P, P, I, I, I, P),
    "tfb_dequant": (P, I, I, I, P, I, I, I, P),
    "tfb_group_sums": (P, L, P, I, I, I, P),
    "tfb_experts_run": (I, I, P, L, I, P, I, I, P, P, P, P, I, F, L, I, P),
    "tfb_experts_run_tile": (I, I, P, L, I, P, I, I, P, P, P, P, I, F, L, I, I, P),
    "tfb_experts_run_slices": (I, P, L, I, P, I, I, P, P, P, P, I, I, L, I, I, P),
    "tfb_experts_prefill": (I, I, P, L, I, P, I, I, P, P, P, P, I, F, L, I, P),
    "tfb_exl3_dequant": (P, P, I, I, I, I, P),
    "tfb_exl3_group": (P, P, P, P, P, P, P, I, I, I, I, I, P),
    "tfb_exl3_group_static": (P, P, P, P, I, I, I, I, I, P),
    "tfb_exl3_prologue": (P, L, I, P, P, P, P, P, I, I, I, I, I, P, P, P, P, P, P, P, P, I, P),
    "tfb_exl3_gateup": (P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, F, I, P, P, I, I, I, P),
    "tfb_exl3_rot_out": (P, P, P, P, L, I, I, I, P),
    "tfb_exl3_down": (P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, I, I, I, P),
    "tfb_peer_stage": (P, P, L, L, P),
    "tfb_peer_gather": (P, I, I, I, P, P, P, P, P),
    "tfb_combine_push": (P, P, P, I, I, P, L, I, I, I, I, I, P, P),
    "tfb_peer_sum": (P, I, L, I, I, I, P, I, P, P, I, P, P, P),
    "tfb_peer_push": (P, P, L, I, I, I, I, P, P),
    "tfb_window_picks": (P, P, I, I, P, P, I, P),
    "tfb_kernel_status": (P, P),
}


class MissingLibrary(RuntimeError):
    pass


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise MissingLibrary(f"{LIB_PATH} is not built: run `python -m tensorfold_b200.build` (there is no fallback)")
    handle = ctypes.CDLL(str(LIB_PATH))
    handle.tfb_last_error.restype = c_char_p
    handle.tfb_last_error.argtypes = ()
    handle.tfb_version.restype = c_int
    handle.tfb_set_pdl.argtypes = (c_int,)
    handle.tfb_set_pdl.restype = c_int
    handle.tfb_set_wait_limit_ms.argtypes = (c_int,)
    handle.tfb_set_wait_limit_ms.restype = c_int
    handle.tfb_route_max_rows.argtypes = (c_int,)
    handle.tfb_route_max_rows.restype = c_int
    handle.tfb_decode_kslices.argtypes = (c_int,)
    handle.tfb_decode_kslices.restype = c_int
    handle.tfb_select_plan_max_rows.restype = c_int
    handle.tfb_select_plan_max_rows.argtypes = ()
    for name, args in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.argtypes = args
        fn.restype = c_int
    return handle


def call(name: str, *args) -> None:
    """Call an entry point; a bad argument raises ValueError, anything else RuntimeError, with the library's text."""

    handle = lib()
    rc = getattr(handle, name)(*args)
    if rc == 0:
        return
    text = handle.tfb_last_error().decode("utf-8", "replace")
    if rc == ERR_ARG:
        raise ValueError(text)
    raise RuntimeError(text)


def kernel_status(stream: int = 0) -> int:
    """The device status word (0: every kernel since the last read finished its waits); clears it."""

    out = c_int(0)
    call("tfb_kernel_status", ctypes.addressof(out), stream)
    return out.value


def set_pdl(on: bool) -> bool:
    return bool(lib().tfb_set_pdl(1 if on else 0))


def set_wait_limit_ms(ms: int) -> int:
    """How long an expert-parallel barrier waits for the other ranks; returns the previous limit."""

    was = lib().tfb_set_wait_limit_ms(int(ms))
    if was < 0:
        raise ValueError(lib().tfb_last_error().decode("utf-8", "replace"))
    return was


ST_WAIT_TIMEOUT, ST_BAD_INDEX = 1, 2
_WHERE = {0: "a kernel's copy pipeline", 1: "the tokens barrier", 2: "the results barrier"}


def describe_status(status: int) -> str:
    """The status word in words: which wait ran out and, for a barrier between ranks, which rank never arrived."""

    if status == 0:
        return "ok"
    code, where, rank = status & 0xFF, (status >> 8) & 0xFF, (status >> 16) & 0xFF
    if code == ST_WAIT_TIMEOUT:
        text = f"a bounded wait ran out at {_WHERE.get(where, f'site {where}')}"
        return text + (f": rank {rank} had not arrived" if where in (1, 2) else "")
    if code == ST_BAD_INDEX:
        return "a table held an index no kernel exists for"
    return f"unknown status word {status:#x}"


class StepFailed(RuntimeError):
    """A kernel recorded a failure on the device; ``status`` is the word ``describe_status`` reads."""

    def __init__(self, status: int) -> None:
        super().__init__(describe_status(status))
        self.status = status


def check_status(stream: int = 0) -> None:
    """Raise ``StepFailed`` unless every kernel since the last read completed its waits."""

    status = kernel_status(stream)
    if status != 0:
        raise StepFailed(status)
