"""Test infrastructure only: numpy restatement of the reference's sigmoid-plus-bias selection
(``src/tensorfold/families/glm5_next/cuda/glue.py:351-378`` ``_topk``; the Nemotron twin is
``src/tensorfold/families/nemotron_h/cuda/glue.py:56-88``).  The reference's own tests pin the picks against the sort by
(-choice, id) and the weights by ``allclose``; the exp's last bits are Triton's, so weights are tolerance-checked."""

from __future__ import annotations

import numpy as np


def sigmoid_topk(logits: np.ndarray, bias: np.ndarray, top_k: int, scale: float, norm: bool, shared_slots: int = 1):
    """logits [T, >= E] fp32, bias [E] fp32 -> pick [T, top_k + shared_slots] int32, wts fp32, and each row's smallest
    gap between consecutive choices around the cut (rows with a gap near the exp's rounding are not comparable)."""

    logits = np.asarray(logits, dtype=np.float32)
    e = bias.shape[0]
    rows = logits.shape[0]
    slots = top_k + shared_slots
    pick = np.zeros((rows, slots), dtype=np.int32)
    wts = np.zeros((rows, slots), dtype=np.float32)
    gap = np.zeros((rows,), dtype=np.float64)
    for r in range(rows):
        score = (np.float32(1) / (np.float32(1) + np.exp(-logits[r, :e], dtype=np.float32))).astype(np.float32)
        choice = (score + bias.astype(np.float32)).astype(np.float32)
        order = sorted(range(e), key=lambda i: (-choice[i], i))
        total = np.float32(0)
        for k in range(top_k):
            pick[r, k] = order[k]
            wts[r, k] = score[order[k]]
            total = np.float32(total + score[order[k]])
        if norm:
            wts[r, :top_k] = wts[r, :top_k] / np.float32(total + np.float32(1e-20))
        wts[r, :top_k] = wts[r, :top_k] * np.float32(scale)
        for j in range(shared_slots):
            pick[r, top_k + j] = e + j
            wts[r, top_k + j] = 1.0
        top = choice[order[:top_k + 1]].astype(np.float64)
        gap[r] = np.min(top[:-1] - top[1:]) if e > top_k else 1.0
    return pick, wts, gap
