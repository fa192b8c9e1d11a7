"""TEST INFRASTRUCTURE: numpy restatement of the EXL3 trellis format and of the routed EXL3 layer.

Follows the reference's format description and decoder (``src/tensorfold/cuda/exl3/format.py:16-19,31-48`` codebooks,
``:58-66`` window ends, ``:69-77`` tile positions, ``:95-116`` 16-bit states, ``:119-132`` unpack, ``:145-180``
Hadamard rotation and layer), written independently and pinned against that module's outputs by the fixtures in
``tests/golden/`` (made by ``tests/golden/make_exl3_golden.py`` where the reference tree is mounted).
"""

from __future__ import annotations

import numpy as np

CB_3INST, CB_MCG, CB_MUL1 = 0, 1, 2
HAD = 128


def _half(bits: np.ndarray) -> np.ndarray:
    return bits.astype(np.uint16).view(np.float16)


def codebook(cb: int) -> np.ndarray:
    """fp16 value of every 16-bit state, [65536]."""

    s = np.arange(65536, dtype=np.uint64)
    if cb == CB_MUL1:
        x = (s * 0x83DCD12D) & 0xFFFFFFFF
        h = 1024 + (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + ((x >> 24) & 255)
        scale = float(_half(np.array([0x1EEE]))[0])
        bias = float(_half(np.array([0xC931]))[0])
        return (h.astype(np.float64) * scale + bias).astype(np.float16)          # one rounding, as an fp16 fma
    x = (s * 0xCBAC1FED) & 0xFFFFFFFF if cb == CB_MCG else (s * 89226354 + 64248484) & 0xFFFFFFFF
    x = (x & 0x8FFF8FFF) ^ 0x3B603B60
    lo, hi = _half(x & 0xFFFF).astype(np.float64), _half(x >> 16).astype(np.float64)
    return (lo + hi).astype(np.float16)                                          # one fp16 rounding of the exact sum


def window_end(p: np.ndarray | int, k2: int):
    """One past the last stream bit of value p's 16-bit window, for K2 half-bits a value."""

    p = np.asarray(p)
    return (p >> 1) * k2 + np.where(p & 1, k2, k2 >> 1)


def tile_states(words32: np.ndarray, k2: int) -> np.ndarray:
    """[..., 4 * k2] uint32 tile words -> [..., 256] 16-bit states in stream order (MSB-first circular stream)."""

    w = np.ascontiguousarray(words32).astype(np.uint64)
    tw = 4 * k2
    assert w.shape[-1] == tw
    first = window_end(np.arange(256), k2) - 16 + 32 * tw
    i0, off = (first // 32) % tw, first % 32
    pair = (w[..., i0] << 32) | w[..., (i0 + 1) % tw]
    return ((pair >> (48 - off).astype(np.uint64)) & 0xFFFF).astype(np.uint32)


def tile_positions():
    p = np.arange(256)
    lane, j = p // 8, p % 8
    return 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1), lane // 4 + 8 * (j >> 2)


def unpack(trellis: np.ndarray, cb: int) -> np.ndarray:
    """trellis int16 [K/16, N/16, 8 * k2] -> W_q fp16 [K, N]."""

    t = np.ascontiguousarray(trellis)
    kt, nt, w16 = t.shape
    k2 = w16 // 8
    words = t.view(np.uint16).astype(np.uint32)
    words = words[..., 0::2] | (words[..., 1::2] << 16)
    vals = codebook(cb)[tile_states(words, k2)]                                  # [kt, nt, 256]
    rows, cols = tile_positions()
    out = np.empty((kt, 16, nt, 16), dtype=np.float16)
    out[:, rows, :, cols] = vals.transpose(2, 0, 1)
    return out.reshape(kt * 16, nt * 16)


def hadamard() -> np.ndarray:
    i = np.arange(HAD)
    par = np.array([bin(v).count("1") & 1 for v in range(HAD)])
    return np.where(par[i[:, None] & i[None, :]] == 1, -1.0, 1.0) / np.sqrt(HAD)


def rotate(x: np.ndarray) -> np.ndarray:
    """H / sqrt(128) on every block of 128 of the last axis, float64."""

    s = x.shape
    return (x.reshape(*s[:-1], s[-1] // HAD, HAD) @ hadamard()).reshape(s)


def linear(x, trellis, suh, svh, cb):
    """y = rot(rot(x * suh) @ W_q) * svh in float64 (format.py:174-180)."""

    wq = unpack(trellis, cb).astype(np.float64)
    return rotate(rotate(x * suh.astype(np.float64)) @ wq) * svh.astype(np.float64)


def routed(x, pick, wts, gate, up, down, cb):
    """float64 routed output [R, D]; gate/up/down: per-expert (trellis, suh, svh); picks >= E are skipped
    (the reference's own check: tests/cuda/test_exl3_experts.py:137-161)."""

    x = np.asarray(x, dtype=np.float64)
    out = np.zeros_like(x)
    e_count = len(gate)
    for r in range(x.shape[0]):
        for j in range(pick.shape[1]):
            e = int(pick[r, j])
            if e < 0 or e >= e_count:
                continue
            g = linear(x[r], *gate[e], cb)
            u = linear(x[r], *up[e], cb)
            a = g / (1.0 + np.exp(-g)) * u
            out[r] += float(wts[r, j]) * linear(a, *down[e], cb)
    return out


def group(pick: np.ndarray, experts: int):
    """Distinct routed experts (< E) ascending and, per expert, its members row * 32 + slot in row order
    (src/tensorfold/cuda/exl3/experts.cu:19-72; tests/cuda/test_group_kernel_smem.py:53-64)."""

    r, slots = pick.shape
    uids = sorted({int(e) for e in pick.reshape(-1) if 0 <= e < experts})
    members = np.full((len(uids), r), -1, dtype=np.int32)
    for u, e in enumerate(uids):
        rows, sl = np.nonzero(pick == e)
        order = np.lexsort((sl, rows))
        codes = rows[order] * 32 + sl[order]
        members[u, :min(r, codes.size)] = codes[:r]
    return np.array(uids, dtype=np.int32), members
