"""Routed EXL3 experts of any codebook, a width per expert matrix; rows never depend on the window.

Mirrors the operator surface of the reference's ``src/tensorfold/cuda/exl3/experts.py`` (prepare, prepare_stacked,
Exl3RoutedExperts, Scratch, routed, dequant, default_config, codebook_id, k2_of) over the C-ABI library.  The
trellises are referenced in place by device pointer; the returned object keeps them alive.  ``routed`` allocates
nothing (unless ``out`` is None) and never synchronises, so it can be captured in a CUDA graph.

One ``routed`` call is three launches (``csrc/exl3.cu``): a prologue that sorts the pairs by expert and rotates the
inputs, the gate/up projection with its epilogue fused in, the down projection with its output rotation fused in -
plus the slot-order combine when weights are given.
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
LAUNCHES_PER_CALL = 4             # kernels one ``routed`` call with weights enqueues (3 without)
ITEM_PAIRS = 16                   # pairs an item of the sort holds: two mma tiles share one decoded weight tile
WIDE_ITEM_PAIRS = 32              # the same with four mma tiles, for calls with many pairs an expert
WIDE_FROM = 12                    # pairs an expert on average from which a call sorts into the wide items

# (16-column tiles a block, K-slice warps, K splits across blocks, tiles in flight): this library's one setting.
# The split is by shape only; partial sums meet in warp order inside the block, so there is one split.
CONFIG = (4, 4, 1, 1)
_CODEBOOKS = {"3inst": CB_3INST, "mcg": CB_MCG, "mul1": CB_MUL1}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def codebook_id(name: str) -> int:
    try:
        return _CODEBOOKS[name]
    except KeyError:
        raise ValueError(f"unknown EXL3 codebook {name!r}") from None


def _codebook(codebook: int | str) -> int:
    cb = codebook_id(codebook) if isinstance(codebook, str) else int(codebook)
    if cb not in _CODEBOOKS.values():
        raise ValueError("codebook must be 0 (3inst), 1 (mcg) or 2 (mul1)")
    return cb


def k2_of(trellis: torch.Tensor) -> int:
    """Half-bits a value of a trellis int16 [K/16, N/16, 8 * K2]."""

    k2, rest = divmod(trellis.shape[-1], 8)
    if rest:
        raise ValueError(f"trellis last dim {trellis.shape[-1]} is not a multiple of 8")
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

    @property
    def mixed(self) -> bool:
        """The tensors of a projection differ in width: the kernels then run the items width by width."""

        return self.k2_gu[0] != self.k2_gu[1] or self.k2_d[0] != self.k2_d[1]


class _Projection:
    """The experts' matrices of one projection (K -> N): checked, then one pointer table, one width table and the two
    scale vectors stacked - each made in a single pass over the experts."""

    def __init__(self, mats: Sequence[tuple], k: int, n: int, device) -> None:
        for t, _, _ in mats:
            if t.dtype != torch.int16 or not t.is_contiguous() or t.device.type != "cuda":
                raise ValueError("trellis must be a contiguous CUDA int16 tensor")
            if (t.shape[0] * 16, t.shape[1] * 16) != (k, n):
                raise ValueError(f"expert shape {tuple(t.shape)} does not match [{k // 16}, {n // 16}, *]")
            if t.data_ptr() % 16:
                raise ValueError("trellises must start on a 16-byte boundary (the kernels copy them in 16-byte units)")
        self.trellises = [t for t, _, _ in mats]
        self.widths = [k2_of(t) for t in self.trellises]
        self.ptr = torch.tensor([t.data_ptr() for t in self.trellises], dtype=torch.int64).to(device)
        self.k2 = torch.tensor(self.widths, dtype=torch.int32).to(device)
        self.suh = torch.stack([m[1].reshape(k) for m in mats]).to(device=device, dtype=torch.float16).contiguous()
        self.svh = torch.stack([m[2].reshape(n) for m in mats]).to(device=device, dtype=torch.float16).contiguous()


def prepare(gate: Sequence[tuple], up: Sequence[tuple], down: Sequence[tuple], codebook: int | str,
            device="cuda") -> Exl3RoutedExperts:
    """A layer from per-expert (trellis, suh, svh) triples, trellises referenced in place, each at its own width."""

    cb = _codebook(codebook)
    if len(gate) == 0 or len({len(gate), len(up), len(down)}) != 1:
        raise ValueError("gate, up and down need the same, non-zero number of experts")
    dims, width = (16 * s for s in gate[0][0].shape[:2])
    if dims % 128 or width % 128:
        raise ValueError(f"EXL3 experts need K and N in multiples of 128, not {dims} and {width}")
    g, u, d = _Projection(gate, dims, width, device), _Projection(up, dims, width, device), \
        _Projection(down, width, dims, device)
    # a tile of 256 values takes 16 * K2 bytes, so an expert's three trellises take (tiles a matrix) * 16 * sum(K2)
    tile_bytes = (dims // 16) * (width // 16) * 16
    trellis_bytes = ((g.k2 + u.k2 + d.k2).to(torch.int64) * tile_bytes).cpu()
    return Exl3RoutedExperts(g.ptr, u.ptr, d.ptr, g.k2, u.k2, d.k2, g.suh, u.suh, g.svh, u.svh, d.suh, d.svh,
                             len(gate), dims, width, cb, (min(g.widths + u.widths), max(g.widths + u.widths)),
                             (min(d.widths), max(d.widths)), trellis_bytes, g.trellises + u.trellises + d.trellises)


def prepare_stacked(gt, ut, dt, suh_g, suh_u, svh_g, svh_u, suh_d, svh_d, codebook: int | str) -> Exl3RoutedExperts:
    """A uniform-width layer stacked per projection: trellis [E, K/16, N/16, 16 bits] (int16, or int32 words)."""

    def triples(t, suh, svh):
        t16 = t.view(torch.int16) if t.dtype == torch.int32 else t      # 32-bit words are pairs of the same int16
        return list(zip(t16.unbind(0), suh.unbind(0), svh.unbind(0)))

    return prepare(triples(gt, suh_g, svh_g), triples(ut, suh_u, svh_u), triples(dt, suh_d, svh_d), codebook,
                   device=gt.device)


def default_config(K: int, N: int, gateup: bool) -> tuple[int, int, int, int]:
    """The tile setting for a K -> N projection: one setting, the shape only decides whether it divides."""

    tiles, warps, splits, _ = CONFIG
    if K % (16 * splits * warps) or N % (16 * tiles):
        raise ValueError(f"no tile setting divides K={K}, N={N}")
    return CONFIG


def item_pairs(pairs: int, experts: int) -> int:
    """Pairs an item of a call's sort holds: a function of the call's shape alone (a pair's bits depend on neither)."""

    return WIDE_ITEM_PAIRS if pairs >= WIDE_FROM * experts else ITEM_PAIRS


COMPACT_MIXED = True              # projections of mixed widths run the trellis kernel's build with short loops (same bits)
CROWDED_BLOCKS = 592              # thread blocks from which an SM of a B200 holds four of a launch at once
FILL_BLOCKS = 1480                # thread blocks that fill a B200 twice over (148 SMs x 5 blocks x 2)


def col_tiles(pairs: int, experts: int, n: int, mats: int, k2_all: int = 0, per_item: int = ITEM_PAIRS) -> int:
    """16-column tiles a block of the trellis kernel takes: 4, or 2 while the launch would have too few blocks to
    keep every SM busy (few experts in use) - a function of the call's shape; no result depends on it.  Only for
    projections whose tensors all have 4.00 bits (the kernel built for that width; a row of two narrower tiles is a
    bulk copy of 64-192 bytes, too small to stream well: a mixed-width layer at one token lost a quarter) and for
    items of 16 pairs."""

    few = min(pairs, experts) * (n // 64) * mats < FILL_BLOCKS
    return 2 if few and k2_all == 8 and per_item == ITEM_PAIRS else 4


def max_items(pairs: int, experts: int) -> int:
    """Items the sort of ``pairs`` pairs over ``experts`` experts can make: one an expert in use, one more for every
    full ``ITEM_PAIRS`` pairs past an expert's first (u experts in use: at most u + (pairs - u) // ITEM_PAIRS)."""

    used = min(pairs, experts)
    return used + (pairs - used) // ITEM_PAIRS


class Scratch:
    """Buffers for up to ``rows`` rows of ``slots`` slots; slots whose pick is not a routed expert are the caller's."""

    def __init__(self, ex: Exl3RoutedExperts, rows: int, slots: int, cfg_gu=None, cfg_d=None, device="cuda") -> None:
        if slots > 32:
            raise ValueError("at most 32 slots")
        self.cfg_gu = cfg_gu or default_config(ex.dims, ex.width, True)
        self.cfg_d = cfg_d or default_config(ex.width, ex.dims, False)
        self.rows, self.slots, self.count_experts = rows, slots, ex.count
        pairs, experts_seen = rows * slots, min(rows * slots, ex.count)

        def buf(shape, dtype, fill=0):
            return torch.full(shape, fill, dtype=dtype, device=device)

        # rotated inputs of gate, up and down; partial sums (gate and up side by side, or down); per-pair outputs
        self.xg, self.xu = buf((pairs, ex.dims), torch.float16), buf((pairs, ex.dims), torch.float16)
        self.xd = buf((pairs, ex.width), torch.float16)
        self.z = buf((pairs * max(2 * ex.width, ex.dims),), torch.float32)
        self.y = buf((pairs, ex.dims), torch.float32)
        # the `group` operator's tables (distinct experts, how many, their members) and its sort temporaries
        self.ids, self.count = buf((experts_seen,), torch.int32), buf((1,), torch.int32)
        self.members_buf = buf((experts_seen * rows,), torch.int32, -1)
        self.tmp_members, self.tmp_items = buf((pairs,), torch.int32), buf((max(1, experts_seen), 3), torch.int32)
        self.tmp_counts = buf((2,), torch.int32)
        # what the kernels read: pairs sorted by expert, items of up to ITEM_PAIRS pairs, and the arrival counters of
        # the fused epilogues (one a (item, 128 columns); the kernels leave them zero)
        items = max_items(pairs, ex.count)
        self.sort_members, self.sort_items = buf((pairs,), torch.int32), buf((max(1, items), 3), torch.int32)
        self.sort_counts = buf((2,), torch.int32)
        self.arrive = buf((max(1, items) * (max(ex.width, ex.dims) // 128),), torch.int32)
        # the items once more in the order of each projection's widths (gate, up, down), for layers of mixed widths
        self.by_width = buf((3, max(1, items), 4), torch.int32)

    def window(self, R: int):
        """(ids, members) sized for R rows: the grids only span what R rows can use."""

        maxu = min(R * self.slots, self.count_experts)
        return self.ids[:maxu], self.members_buf[:maxu * R].view(maxu, R)


def group(pick: torch.Tensor, s: Scratch, R: int, experts: int) -> None:
    """Distinct routed experts (< E) in id order into ``s.ids`` / ``s.count``, their members into ``s.members_buf``
    (the reference's tables), and the sort the kernels read into ``s.sort_*`` - so a following
    ``routed(..., group_first=False)`` finds its pairs grouped."""

    ids, members = s.window(R)
    with torch.cuda.device(pick.device):
        _lib.call("tfb_exl3_group", pick.data_ptr(), ids.data_ptr(), s.count.data_ptr(), members.data_ptr(),
                  s.tmp_members.data_ptr(), s.tmp_items.data_ptr(), s.tmp_counts.data_ptr(), R, s.slots, experts,
                  ids.shape[0], R, _stream(pick))
        _lib.call("tfb_plan", pick.data_ptr(), R * s.slots, experts, ITEM_PAIRS, s.sort_members.data_ptr(),
                  s.sort_items.data_ptr(), s.sort_counts.data_ptr(), _stream(pick))


def routed(x: torch.Tensor, pick: torch.Tensor, wts: torch.Tensor | None, ex: Exl3RoutedExperts, s: Scratch,
           out: torch.Tensor | None, R: int, limit: float = math.inf, act_mode: int = ACT_F32,
           group_first: bool = True, share: float = 1.0) -> torch.Tensor:
    """Routed experts of R rows (picks >= E skipped): y per slot [R * slots, D] fp32, or ``out`` [R, D] fp32 = the
    wts-weighted slot-order sum when ``wts`` is given; no host sync.  ``share``: the fraction of the slots that the
    caller expects to hold one of these experts (an expert-parallel rank: its experts over all experts) - it only
    steers which build of the kernels a call of mixed widths uses, never a result."""

    dims, width, slots = ex.dims, ex.width, s.slots
    pairs = R * slots
    if R > s.rows:
        raise ValueError(f"{R} rows but the scratch holds {s.rows}")
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or x.stride(1) != 1 or x.shape[1] != dims:
        raise ValueError("x must be CUDA bf16 or fp16 [R, D] with unit-stride rows")
    if pick.dtype != torch.int32 or not pick.is_contiguous() or pick.shape != (R, slots):
        raise ValueError(f"pick must be contiguous int32 [{R}, {slots}]")
    if act_mode not in (ACT_BF16, ACT_F32):
        raise ValueError("act_mode is ACT_BF16 or ACT_F32")
    st, items = _stream(x), max_items(pairs, ex.count)
    # `group` sorts into the narrow items; an expert-parallel rank expects only its share of the pairs
    per_item = item_pairs(int(pairs * share), ex.count) if group_first else ITEM_PAIRS
    sort = (s.sort_members.data_ptr(), s.sort_items.data_ptr(), s.sort_counts.data_ptr())
    # the one width of a projection's tensors; or -1: they differ and the launch is large enough for blocks of several
    # widths to share an SM (the kernels then run a build with short loops); or 0: they differ, a small launch
    def width_of(k2: tuple[int, int], n: int, mats: int) -> int:
        if k2[0] == k2[1]:
            return k2[0]
        crowded = min(pairs * share, ex.count) * (n // 64) * mats >= CROWDED_BLOCKS
        return -1 if COMPACT_MIXED and crowded else 0

    k2_gu, k2_d = width_of(ex.k2_gu, width, 2), width_of(ex.k2_d, dims, 1)
    # a layer of mixed widths: the prologue lays the items out width by width, once a projection
    order = [s.by_width[m].data_ptr() for m in range(3)] if ex.mixed and group_first else [0, 0, 0]
    with torch.cuda.device(x.device):
        _lib.call("tfb_exl3_prologue", x.data_ptr(), x.stride(0), int(x.dtype == torch.float16), pick.data_ptr(),
                  ex.suh_g.data_ptr(), ex.suh_u.data_ptr(), s.xg.data_ptr(), s.xu.data_ptr(), R, dims, slots, ex.count,
                  per_item if group_first else 0, *sort, s.count.data_ptr(), ex.gate_k2.data_ptr(), ex.up_k2.data_ptr(),
                  ex.down_k2.data_ptr(), order[0], s.by_width.shape[1], st)
        tables = (sort[1], sort[2], sort[0], s.z.data_ptr(), s.arrive.data_ptr())
        _lib.call("tfb_exl3_gateup", s.xg.data_ptr(), s.xu.data_ptr(), ex.gate_ptr.data_ptr(), ex.up_ptr.data_ptr(),
                  ex.gate_k2.data_ptr(), ex.up_k2.data_ptr(), *tables, ex.svh_g.data_ptr(), ex.svh_u.data_ptr(),
                  ex.suh_d.data_ptr(), s.xd.data_ptr(), dims, width, pairs, ex.cb, items, float(min(limit, 3.0e38)),
                  act_mode, order[0], order[1], per_item, k2_gu, col_tiles(pairs, ex.count, width, 2, k2_gu, per_item),
                  st)
        _lib.call("tfb_exl3_down", s.xd.data_ptr(), ex.down_ptr.data_ptr(), ex.down_k2.data_ptr(), *tables,
                  ex.svh_d.data_ptr(), s.y.data_ptr(), width, dims, pairs, ex.cb, items, order[2], per_item,
                  k2_d, col_tiles(pairs, ex.count, dims, 1, k2_d, per_item), st)
        if wts is None:
            return s.y[:pairs]
        if out is None:
            out = torch.empty((R, dims), dtype=torch.float32, device=x.device)
        if out.dtype != torch.float32 or not out.is_contiguous() or not wts.is_contiguous():
            raise ValueError("out must be contiguous fp32 [R, D] and wts contiguous fp32 [R, slots]")
        # slots that are not routed experts keep the y their owner put there and take part in the sum
        _lib.call("tfb_combine", s.y.data_ptr(), 0, wts.data_ptr(), out.data_ptr(), 1, R, slots, dims, st)
    return out


def dequant(trellis: torch.Tensor, codebook: int | str) -> torch.Tensor:
    """W_q [K, N] fp16 of one matrix through the kernels' own lane decode; for tests."""

    cb = _codebook(codebook)
    rows, cols = trellis.shape[0] * 16, trellis.shape[1] * 16
    words = trellis.contiguous()
    w_q = torch.empty((rows, cols), dtype=torch.float16, device=trellis.device)
    with torch.cuda.device(trellis.device):
        _lib.call("tfb_exl3_dequant", words.data_ptr(), w_q.data_ptr(), rows, cols, k2_of(trellis), cb,
                  _stream(trellis))
    return w_q
