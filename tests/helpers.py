"""Shared by the tests: torch <-> numpy bit views and small builders."""

from __future__ import annotations

import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    """A bf16 / fp16 tensor's bit patterns as uint16 numpy."""

    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def words_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().numpy().view(np.uint32)


def triple_np(m):
    return words_np(m[0]), bits(m[1]), bits(m[2])


def from_bits(b: np.ndarray, dtype=torch.bfloat16) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(b).view(np.int16)).view(dtype)


def rel_l2(got, want) -> float:
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
