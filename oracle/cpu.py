"""TEST INFRASTRUCTURE: ctypes front of ``cpu_moe.c`` over numpy arrays (bf16 / fp16 carried as uint16 bit patterns)."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_int64, c_uint16, c_uint32, c_void_p
from functools import lru_cache

import numpy as np

from . import build as _build


class Matrix(Structure):
    _fields_ = [("words", c_void_p), ("scales", c_void_p), ("biases", c_void_p)]


class Exl3Matrices(Structure):
    """One projection of every expert: arrays of E pointers (trellis, suh, svh) and E half-bit widths."""

    _fields_ = [("trellis", c_void_p), ("k2", c_void_p), ("suh", c_void_p), ("svh", c_void_p)]


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
    h.tfo_exl3_unpack.argtypes = (c_void_p, c_int, c_int, c_int, c_int, c_void_p)
    h.tfo_exl3_unpack.restype = None
    h.tfo_exl3_routed.argtypes = (c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, Exl3Matrices,
                                  Exl3Matrices, Exl3Matrices, c_int, c_void_p)
    h.tfo_exl3_routed.restype = c_int
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


def exl3_unpack(trellis: np.ndarray, cb: int) -> np.ndarray:
    """W_q [K, N] fp16 of a trellis int16 [K/16, N/16, 8 * k2] (the C twin of ``oracle.exl3.unpack``)."""

    t = np.ascontiguousarray(trellis).view(np.uint16)
    k, n, k2 = t.shape[0] * 16, t.shape[1] * 16, t.shape[2] // 8
    out = np.empty((k, n), dtype=np.uint16)
    lib().tfo_exl3_unpack(_p(t), k, n, k2, cb, _p(out))
    return out.view(np.float16)


def _exl3_table(mats, keep):
    """mats: per expert (trellis int16, suh fp16, svh fp16), or None for an expert no row uses."""

    e = len(mats)
    ptrs = [np.zeros(e, dtype=np.uint64) for _ in range(3)]
    k2 = np.zeros(e, dtype=np.int32)
    for i, m in enumerate(mats):
        if m is None:
            continue
        arrs = (np.ascontiguousarray(m[0]).view(np.uint16), np.ascontiguousarray(m[1]).view(np.uint16),
                np.ascontiguousarray(m[2]).view(np.uint16))
        keep.append(arrs)
        for j in range(3):
            ptrs[j][i] = arrs[j].ctypes.data
        k2[i] = arrs[0].shape[-1] // 8
    keep.extend(ptrs + [k2])
    return Exl3Matrices(ptrs[0].ctypes.data, k2.ctypes.data, ptrs[1].ctypes.data, ptrs[2].ctypes.data)


def exl3_routed(x: np.ndarray, pick: np.ndarray, wts: np.ndarray, gate, up, down, cb: int, dims: int,
                width: int) -> np.ndarray:
    """The routed EXL3 layer in fp32 on the host cores (the C twin of ``oracle.exl3.routed``): out [R, D]."""

    xf, pk, w = _c(np.asarray(x, dtype=np.float32), np.float32), _c(pick, np.int32), _c(wts, np.float32)
    r, slots = pk.shape
    keep: list = []
    out = np.empty((r, dims), dtype=np.float32)
    rc = lib().tfo_exl3_routed(_p(xf), _p(pk), _p(w), r, slots, len(gate), dims, width, _exl3_table(gate, keep),
                               _exl3_table(up, keep), _exl3_table(down, keep), cb, _p(out))
    if rc != 0:
        raise MemoryError("tfo_exl3_routed: out of memory")
    return out
