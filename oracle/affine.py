"""TEST INFRASTRUCTURE: numpy restatement of the MLX affine 4-bit group-64 format and float64 layer references.

Format (``src/tensorfold/families/qwen3_5_moe/cuda/weights.py:20-29``; ``code_at`` in
``src/tensorfold/kernels/qwen/dense/v1/affine_rows.py:14-21``): element k of a row is bits [4 (k % 8), +4) of word
k // 8; value = scale[k // 64] * q + bias[k // 64].
"""

from __future__ import annotations

import numpy as np


def bf16_bits(f: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""

    u = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_value(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(f: np.ndarray) -> np.ndarray:
    return bf16_value(bf16_bits(f))


def half_value(bits: np.ndarray, fp16: bool) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    return b.view(np.float16).astype(np.float32) if fp16 else bf16_value(b)


def codes(words: np.ndarray) -> np.ndarray:
    """uint32 words [..., K/8] -> codes uint8 [..., K]."""

    w = np.ascontiguousarray(words).view(np.uint32)
    sh = (np.arange(8, dtype=np.uint32) * 4)
    return ((w[..., None] >> sh) & 0xF).astype(np.uint8).reshape(*w.shape[:-1], -1)


def pack_codes(q: np.ndarray) -> np.ndarray:
    """codes [..., K] -> uint32 words [..., K/8]."""

    q = np.asarray(q, dtype=np.uint64).reshape(*q.shape[:-1], -1, 8)
    sh = np.arange(8, dtype=np.uint64) * 4
    return (q << sh).sum(-1).astype(np.uint32)


def dequant64(words, scales_bits, biases_bits, gs: int, fp16: bool) -> np.ndarray:
    """float64 q * s + b (exact), as the float64 twin in tests/cuda/test_experts.py:26-30."""

    q = codes(words).astype(np.float64)
    s = half_value(scales_bits, fp16).astype(np.float64).repeat(gs, -1)
    b = half_value(biases_bits, fp16).astype(np.float64).repeat(gs, -1)
    return q * s + b


def silu_gate(g: np.ndarray, u: np.ndarray, limit: float = 0.0) -> np.ndarray:
    """bf16(bf16(silu(bf16 g)) * bf16 u) in float64 inputs (src/tensorfold/cuda/experts.cuh:57-65;
    tests/cuda/test_experts.py:178-182)."""

    gv = round_bf16(g.astype(np.float32)).astype(np.float64)
    uv = round_bf16(u.astype(np.float32)).astype(np.float64)
    if limit:
        gv, uv = np.minimum(gv, limit), np.clip(uv, -limit, limit)
    s = round_bf16((gv / (1.0 + np.exp(-gv))).astype(np.float32)).astype(np.float64)
    return round_bf16((s * uv).astype(np.float32)).astype(np.float64)


def layer64(x_bits, pick, wts, gate, up, down, gs: int, fp16: bool, limit: float = 0.0, prefill: bool = False):
    """The fp64-accumulated reference of one layer given the routing: per pair act and y, and the combined out.

    gate/up/down = (words [E', N, K/8], scales bits, biases bits).  ``prefill`` rounds the dequantised weights to
    bf16 first (tests/cuda/test_experts.py:174-176).  Returns (act [P, NI], y [P, D], out [T, D]) in float64."""

    from . import cpu

    x = bf16_value(x_bits).astype(np.float64)
    t, slots = pick.shape
    p = t * slots
    ni, d = gate[0].shape[1], x.shape[1]
    act = np.zeros((p, ni))
    y = np.zeros((p, d))
    flat = pick.reshape(-1)

    def weights(m, e):
        if prefill:
            return cpu.dequant(m[0][e], m[1][e], m[2][e], gs, fp16, True).astype(np.float64)
        return dequant64(m[0][e], m[1][e], m[2][e], gs, fp16)

    for e in np.unique(flat):
        idx = np.nonzero(flat == e)[0]
        xr = x[idx // slots]
        a = silu_gate(xr @ weights(gate, e).T, xr @ weights(up, e).T, limit)
        act[idx] = a
        y[idx] = a @ weights(down, e).T
    out = (wts.astype(np.float64).reshape(t, slots, 1) * y.reshape(t, slots, d)).sum(1)
    return act, y, out
