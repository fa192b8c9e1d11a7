"""Routed EXL3 experts of any codebook, a width per expert matrix; rows never depend on the window.

Mirrors the operator surface of the reference's ``src/tensorfold/cuda/exl3/experts.py`` (prepare, prepare_stacked,
Exl3RoutedExperts, Scratch, routed, dequant, default_config, codebook_id, k2_of) over the C-ABI library.  The
trellises are referenced in place by device pointer; the returned object keeps them alive.  ``routed`` allocates
nothing (unless ``out`` is None) and never synchronises, so it can be captured in a CUDA graph.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Sequence

import torch

from .. import _lib

CB_3INST, CB_MCG, CB_MUL1 = 0, 1, 2
ACT_BF16, ACT_F32 = 0, 1          # SwiGLU with the GLM family's bf16 roundings / in fp32
K2_SUPPORTED = tuple(range(2, 17))   # half-bits a value: 1..8 bits and every half-integer rate between
LAUNCHES_PER_CALL = 6             # kernels one ``routed`` call enqueues (grouping included)

# (16-column tiles a block, K-slice warps, K splits across blocks, tiles in flight): this library's one setting.
# The split is by shape only; partial sums meet in warp order inside the block, so there is one split.
CONFIG = (4, 4, 1, 1)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def codebook_id(name: str) -> int:
    ids = {"3inst": CB_3INST, "mcg": CB_MCG, "mul1": CB_MUL1}
    if name not in ids:
        raise ValueError(f"unknown EXL3 codebook {name!r}")
    return ids[name]


def k2_of(trellis: torch.Tensor) -> int:
    """Half-bits a value of a trellis int16 [K/16, N/16, 8 * K2]."""

    w = trellis.shape[-1]
    if w % 8:
        raise ValueError(f"trellis last dim {w} is not a multiple of 8")
    k2 = w // 8
    if k2 not in K2_SUPPORTED:
        raise ValueError(f"unsupported EXL3 bit width {k2 / 2}")
    return k2


@dataclass
class Exl3RoutedExperts:
    """One layer's routed experts: trellis pointers and widths per projection, stacked suh / svh."""

    gate_ptr: torch.Tensor    # int64 [E]
    up_ptr: torch.Tensor
    down_ptr: torch.Tensor
    gate_k2: torch.Tensor     # int32 [E]
    up_k2: torch.Tensor
    down_k2: torch.Tensor
    suh_g: torch.Tensor       # fp16 [E, D]
    suh_u: torch.Tensor
    svh_g: torch.Tensor       # fp16 [E, I]
    svh_u: torch.Tensor
    suh_d: torch.Tensor       # fp16 [E, I]
    svh_d: torch.Tensor       # fp16 [E, D]
    count: int
    dims: int
    width: int
    cb: int
    k2_gu: tuple[int, int]
    k2_d: tuple[int, int]
    trellis_bytes: torch.Tensor   # int64 [E], gate + up + down trellis bytes of each expert
    keep: list = field(default_factory=list, repr=False)

    def nbytes_read(self, ids: Sequence[int]) -> int:
        return int(self.trellis_bytes[list(ids)].sum())


def prepare(gate: Sequence[tuple], up: Sequence[tuple], down: Sequence[tuple], codebook: int | str,
            device="cuda") -> Exl3RoutedExperts:
    """A layer from per-expert (trellis, suh, svh) triples, trellises referenced in place, each at its own width."""

    cb = codebook_id(codebook) if isinstance(codebook, str) else int(codebook)
    if cb not in (CB_3INST, CB_MCG, CB_MUL1):
        raise ValueError("codebook must be 0 (3inst), 1 (mcg) or 2 (mul1)")
    e_count = len(gate)
    if not (len(up) == len(down) == e_count) or e_count == 0:
        raise ValueError("gate, up and down need the same, non-zero number of experts")
    d, i = gate[0][0].shape[0] * 16, gate[0][0].shape[1] * 16
    if d % 128 or i % 128:
        raise ValueError(f"EXL3 experts need K and N in multiples of 128, not {d} and {i}")
    keep = []

    def table(mats, k, n):
        ptrs, k2s = [], []
        for t, _, _ in mats:
            if t.dtype != torch.int16 or not t.is_contiguous() or t.device.type != "cuda":
                raise ValueError("trellis must be a contiguous CUDA int16 tensor")
            if t.shape[0] * 16 != k or t.shape[1] * 16 != n:
                raise ValueError(f"expert shape {tuple(t.shape)} does not match [{k // 16}, {n // 16}, *]")
            k2s.append(k2_of(t))
            ptrs.append(t.data_ptr())
            keep.append(t)
        return (torch.tensor(ptrs, dtype=torch.int64, device=device),
                torch.tensor(k2s, dtype=torch.int32, device=device), k2s)

    gp, gk, gks = table(gate, d, i)
    upp, uk, uks = table(up, d, i)
    dp, dk, dks = table(down, i, d)

    def stack(mats, j, n):
        out = torch.empty((e_count, n), dtype=torch.float16, device=device)
        for e, m in enumerate(mats):
            out[e].copy_(m[j].reshape(-1))
        return out

    tb = torch.tensor([(d * i // 256) * (gks[e] + uks[e] + dks[e]) * 16 for e in range(e_count)], dtype=torch.int64)
    return Exl3RoutedExperts(gp, upp, dp, gk, uk, dk, stack(gate, 1, d), stack(up, 1, d), stack(gate, 2, i),
                             stack(up, 2, i), stack(down, 1, i), stack(down, 2, d), e_count, d, i, cb,
                             (min(gks + uks), max(gks + uks)), (min(dks), max(dks)), tb, keep)


def prepare_stacked(gt, ut, dt, suh_g, suh_u, svh_g, svh_u, suh_d, svh_d, codebook: int | str) -> Exl3RoutedExperts:
    """A uniform-width layer stacked per projection: trellis [E, K/16, N/16, 16 bits] (int16, or int32 words)."""

    def as16(t):
        return t.view(torch.int16) if t.dtype == torch.int32 else t

    gt, ut, dt = as16(gt), as16(ut), as16(dt)
    e_count = gt.shape[0]
    return prepare([(gt[e], suh_g[e], svh_g[e]) for e in range(e_count)],
                   [(ut[e], suh_u[e], svh_u[e]) for e in range(e_count)],
                   [(dt[e], suh_d[e], svh_d[e]) for e in range(e_count)], codebook, device=gt.device)


def default_config(K: int, N: int, gateup: bool) -> tuple[int, int, int, int]:
    """The tile setting for a K -> N projection: one setting, the shape only decides whether it divides."""

    nt, w, sk, pf = CONFIG
    if K % (16 * sk * w) or N % (16 * nt):
        raise ValueError(f"no tile setting divides K={K}, N={N}")
    return CONFIG


class Scratch:
    """Buffers for up to ``rows`` rows of ``slots`` slots; slots whose pick is not a routed expert are the caller's."""

    def __init__(self, ex: Exl3RoutedExperts, rows: int, slots: int, cfg_gu=None, cfg_d=None, device="cuda") -> None:
        d, i = ex.dims, ex.width
        self.cfg_gu = cfg_gu or default_config(d, i, True)
        self.cfg_d = cfg_d or default_config(i, d, False)
        if slots > 32:
            raise ValueError("at most 32 slots")
        p = rows * slots
        self.xg = torch.zeros((p, d), dtype=torch.float16, device=device)
        self.xu = torch.zeros((p, d), dtype=torch.float16, device=device)
        self.xd = torch.zeros((p, i), dtype=torch.float16, device=device)
        self.z = torch.zeros((max(2 * i, d) * p,), dtype=torch.float32, device=device)
        self.y = torch.zeros((p, d), dtype=torch.float32, device=device)
        maxu = min(p, ex.count)
        self.ids = torch.zeros((maxu,), dtype=torch.int32, device=device)
        self.count = torch.zeros((1,), dtype=torch.int32, device=device)
        self.members_buf = torch.full((maxu * rows,), -1, dtype=torch.int32, device=device)
        self.sort_members = torch.zeros((p,), dtype=torch.int32, device=device)
        self.sort_items = torch.zeros((max(1, maxu), 3), dtype=torch.int32, device=device)
        self.sort_counts = torch.zeros((2,), dtype=torch.int32, device=device)
        self.rows, self.slots, self.count_experts = rows, slots, ex.count

    def window(self, R: int):
        """(ids, members) sized for R rows: the grids only span what R rows can use."""

        maxu = min(R * self.slots, self.count_experts)
        return self.ids[:maxu], self.members_buf[:maxu * R].view(maxu, R)


def group(pick: torch.Tensor, s: Scratch, R: int, experts: int) -> None:
    """Distinct routed experts (< E) in id order into ``s.ids`` / ``s.count``, their members into ``s.members_buf``."""

    ids, members = s.window(R)
    with torch.cuda.device(pick.device):
        _lib.call("tfb_exl3_group", pick.data_ptr(), ids.data_ptr(), s.count.data_ptr(), members.data_ptr(),
                  s.sort_members.data_ptr(), s.sort_items.data_ptr(), s.sort_counts.data_ptr(), R, s.slots, experts,
                  ids.shape[0], R, _stream(pick))


def routed(x: torch.Tensor, pick: torch.Tensor, wts: torch.Tensor | None, ex: Exl3RoutedExperts, s: Scratch,
           out: torch.Tensor | None, R: int, limit: float = math.inf, act_mode: int = ACT_F32,
           group_first: bool = True) -> torch.Tensor:
    """Routed experts of R rows (picks >= E skipped): y per slot [R * slots, D] fp32, or ``out`` [R, D] fp32 = the
    wts-weighted slot-order sum when ``wts`` is given; no host sync."""

    d, i, e_count, slots = ex.dims, ex.width, ex.count, s.slots
    p = R * slots
    if R > s.rows:
        raise ValueError(f"{R} rows but the scratch holds {s.rows}")
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or x.stride(1) != 1 or x.shape[1] != d:
        raise ValueError("x must be CUDA bf16 or fp16 [R, D] with unit-stride rows")
    if pick.dtype != torch.int32 or not pick.is_contiguous() or pick.shape != (R, slots):
        raise ValueError(f"pick must be contiguous int32 [{R}, {slots}]")
    ids, members = s.window(R)
    st = _stream(x)
    lim = float(min(limit, 3.0e38))
    with torch.cuda.device(x.device):
        if group_first:
            group(pick, s, R, e_count)
        _lib.call("tfb_exl3_rot_in", x.data_ptr(), x.stride(0), 1 if x.dtype == torch.float16 else 0, pick.data_ptr(),
                  ex.suh_g.data_ptr(), ex.suh_u.data_ptr(), s.xg.data_ptr(), s.xu.data_ptr(), R, d, slots, e_count, st)
        _lib.call("tfb_exl3_grouped", s.xg.data_ptr(), s.xu.data_ptr(), ex.gate_ptr.data_ptr(), ex.up_ptr.data_ptr(),
                  ex.gate_k2.data_ptr(), ex.up_k2.data_ptr(), ids.data_ptr(), s.count.data_ptr(), members.data_ptr(),
                  s.z.data_ptr(), 2, d, i, p, slots, ex.cb, R, ids.shape[0], st)
        _lib.call("tfb_exl3_gateup_epilogue", s.z.data_ptr(), pick.data_ptr(), ex.svh_g.data_ptr(),
                  ex.svh_u.data_ptr(), ex.suh_d.data_ptr(), s.xd.data_ptr(), p, i, e_count, lim, act_mode, st)
        _lib.call("tfb_exl3_grouped", s.xd.data_ptr(), s.xd.data_ptr(), ex.down_ptr.data_ptr(), ex.down_ptr.data_ptr(),
                  ex.down_k2.data_ptr(), ex.down_k2.data_ptr(), ids.data_ptr(), s.count.data_ptr(),
                  members.data_ptr(), s.z.data_ptr(), 1, i, d, p, slots, ex.cb, R, ids.shape[0], st)
        if wts is None:
            _lib.call("tfb_exl3_down_epilogue", s.z.data_ptr(), pick.data_ptr(), ex.svh_d.data_ptr(), s.y.data_ptr(),
                      0, 0, R, d, e_count, slots, st)
            return s.y[:p]
        if out is None:
            out = torch.empty((R, d), dtype=torch.float32, device=x.device)
        _lib.call("tfb_exl3_down_epilogue", s.z.data_ptr(), pick.data_ptr(), ex.svh_d.data_ptr(), s.y.data_ptr(),
                  wts.data_ptr(), out.data_ptr(), R, d, e_count, slots, st)
    return out


def dequant(trellis: torch.Tensor, codebook: int | str) -> torch.Tensor:
    """W_q [K, N] fp16 of one matrix through the kernels' own lane decode; for tests."""

    cb = codebook_id(codebook) if isinstance(codebook, str) else int(codebook)
    k2 = k2_of(trellis)
    k, n = trellis.shape[0] * 16, trellis.shape[1] * 16
    t = trellis.contiguous()
    out = torch.empty((k, n), dtype=torch.float16, device=trellis.device)
    with torch.cuda.device(trellis.device):
        _lib.call("tfb_exl3_dequant", t.data_ptr(), out.data_ptr(), k, n, k2, cb, _stream(trellis))
    return out
