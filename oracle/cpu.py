"""TEST INFRASTRUCTURE: ctypes front of ``cpu_moe.c`` over numpy arrays (bf16 / fp16 carried as uint16 bit patterns)."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_int64, c_uint16, c_uint32, c_void_p
from functools import lru_cache

import numpy as np

from . import build as _build


class Matrix(Structure):
    _fields_ = [("words", c_void_p), ("scales", c_void_p), ("biases", c_void_p)]


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    h = ctypes.CDLL(str(_build.build()))
    h.tfo_code_at.restype = c_uint32
    h.tfo_code_at.argtypes = (c_void_p, c_int, c_int)
    h.tfo_router_logits.argtypes = (c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int)
    h.tfo_router_logits.restype = None
    h.tfo_topk_rows.argtypes = (c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int)
    h.tfo_topk_rows.restype = None
    h.tfo_plan.argtypes = (c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p)
    h.tfo_plan.restype = c_int
    h.tfo_affine_rows.argtypes = (c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                  c_int)
    h.tfo_affine_rows.restype = None
    h.tfo_dequant.argtypes = (c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p)
    h.tfo_dequant.restype = None
    h.tfo_moe_layer.argtypes = (c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, Matrix, Matrix, Matrix, c_int,
                                c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p)
    h.tfo_moe_layer.restype = c_int
    h.tfo_threads.restype = c_int
    h.tfo_set_threads.argtypes = (c_int,)
    return h


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _c(a, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype != dtype:
        raise TypeError(f"expected {dtype}, got {a.dtype}")
    return a


def threads() -> int:
    return lib().tfo_threads()


def set_threads(n: int) -> None:
    lib().tfo_set_threads(n)


def router_logits(x_bits: np.ndarray, w_bits: np.ndarray) -> np.ndarray:
    x, w = _c(x_bits, np.uint16), _c(w_bits, np.uint16)
    t, d = x.shape
    out = np.empty((t, w.shape[0]), dtype=np.float32)
    lib().tfo_router_logits(_p(x), d, _p(w), _p(out), t, d, w.shape[0])
    return out


def topk_rows(logits: np.ndarray, experts: int, top_k: int, shared: bool):
    lg = _c(logits, np.float32)
    t, nl = lg.shape
    slots = top_k + (1 if shared else 0)
    pick = np.empty((t, slots), dtype=np.int32)
    wts = np.empty((t, slots), dtype=np.float32)
    lib().tfo_topk_rows(_p(lg), nl, _p(pick), _p(wts), t, experts, top_k, 1 if shared else 0)
    return pick, wts


def plan(picks: np.ndarray, experts: int, tile: int):
    pk = _c(picks, np.int32).reshape(-1)
    members = np.full((pk.size,), -1, dtype=np.int32)
    items = np.zeros((pk.size + experts, 3), dtype=np.int32)
    counts = np.zeros((2,), dtype=np.int32)
    n = lib().tfo_plan(_p(pk), pk.size, experts, tile, _p(members), _p(items), _p(counts))
    valid = int(((pk >= 0) & (pk < experts)).sum())
    return items[:n].copy(), members[:valid].copy(), counts


def affine_rows(x_bits, words, scales_bits, biases_bits, gs: int, fp16_scales: bool, out_bf16: bool = True):
    x, w = _c(x_bits, np.uint16), _c(words, np.uint32)
    s, b = _c(scales_bits, np.uint16), _c(biases_bits, np.uint16)
    r, k = x.shape
    n = w.shape[0]
    out = np.empty((r, n), dtype=np.float32)
    lib().tfo_affine_rows(_p(x), r, _p(w), _p(s), _p(b), 1 if fp16_scales else 0, n, k, gs, _p(out),
                          1 if out_bf16 else 0)
    return out


def dequant(words, scales_bits, biases_bits, gs: int, fp16_scales: bool, prefill: bool) -> np.ndarray:
    w, s, b = _c(words, np.uint32), _c(scales_bits, np.uint16), _c(biases_bits, np.uint16)
    k = w.shape[-1] * 8
    rows = w.size // w.shape[-1]
    out = np.empty((*w.shape[:-1], k), dtype=np.float32)
    lib().tfo_dequant(_p(w), _p(s), _p(b), 1 if fp16_scales else 0, rows, k, gs, 1 if prefill else 0, _p(out))
    return out


def moe_layer(x_bits, router_bits, experts: int, top_k: int, shared: bool, gate, up, down, gs: int,
              fp16_scales: bool, limit: float = 0.0, want_parts: bool = False):
    """gate/up/down: (words uint32 [E', N, K/8], scales uint16, biases uint16), E' = experts (+1 with a shared one).
    Returns out bits [T, D] uint16 (bf16), and with ``want_parts`` also (pick, wts, act bits, y)."""

    x, rt = _c(x_bits, np.uint16), _c(router_bits, np.uint16)
    t, d = x.shape
    ni = gate[0].shape[1]
    keep = []

    def mat(m):
        arrs = (_c(m[0], np.uint32), _c(m[1], np.uint16), _c(m[2], np.uint16))
        keep.append(arrs)
        return Matrix(*(a.ctypes.data for a in arrs))

    slots = top_k + (1 if shared else 0)
    out = np.empty((t, d), dtype=np.uint16)
    pick = np.empty((t, slots), dtype=np.int32) if want_parts else None
    wts = np.empty((t, slots), dtype=np.float32) if want_parts else None
    act = np.empty((t * slots, ni), dtype=np.uint16) if want_parts else None
    y = np.empty((t * slots, d), dtype=np.float32) if want_parts else None
    rc = lib().tfo_moe_layer(_p(x), t, d, _p(rt), experts, top_k, 1 if shared else 0, mat(gate), mat(up), mat(down), ni,
                             gs, 1 if fp16_scales else 0, float(limit), _p(out), _p(pick), _p(wts), _p(act), _p(y))
    if rc != 0:
        raise MemoryError("oracle moe_layer ran out of memory")
    return (out, pick, wts, act, y) if want_parts else out
