"""Grouped MoE experts on MLX affine 4-bit group-64 weights, for B200.

Mirrors the operator surface of the reference's ``src/tensorfold/cuda/experts.py`` (names, argument order, shapes,
error behaviour) over the C-ABI library; a (row, slot) pair's bits never depend on the other rows of the call.
The inner order of a packed block is this library's own (``csrc/common.cuh``); the outer shape
``[E, N/32, K/gs, M, block]`` is the reference's, so callers may still slice experts, column blocks and groups.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

NTW = 4                  # n8 tiles a 32-column block
COLS = 8 * NTW           # output columns a block
TILE = 8                 # pairs an item holds (decode form): one mma tile of pairs
WIDE_TILE = 16           # the decode form's other item size: two mma tiles share one dequantisation
PREFILL_TILE = 192       # pairs a prompt item holds: the tensor-core tile's N
SMALL = 1024             # kept for callers that size scratch by it; this library's plan is one launch at any size
BLOCK = 288              # int32 words a block of 64 inputs x 32 columns: 1024 B of nibbles + 128 B of scale/bias

_SB = {torch.bfloat16: 0, torch.float16: 1}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")


def pack(words: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, gs: int) -> torch.Tensor:
    """MLX words [E, N, K/8], scales and biases [E, N, K/gs] (bf16 or fp16) -> int32 [E, N/32, K/gs, block]."""

    if gs != 64:
        raise ValueError(f"groups of 64 inputs, not {gs}")
    _need_cuda(words, "words")
    if words.dim() != 3 or words.element_size() != 4:
        raise ValueError("words must be 32-bit [E, N, K/8]")
    e, n, k8 = words.shape
    k = k8 * 8
    if n % COLS or k % gs or scales.shape != (e, n, k // gs) or biases.shape != scales.shape:
        raise ValueError(f"experts: shape {tuple(words.shape)} with scales {tuple(scales.shape)} does not pack")
    if scales.element_size() != 2 or biases.dtype != scales.dtype:
        raise ValueError("scales and biases must share a 2-byte dtype")
    out = torch.empty((e, n // COLS, k // gs, BLOCK), dtype=torch.int32, device=words.device)
    w, s, b = words.contiguous(), scales.contiguous(), biases.contiguous()
    with torch.cuda.device(words.device):
        _lib.call("tfb_pack", w.data_ptr(), s.data_ptr(), b.data_ptr(), gs, out.data_ptr(), e, n, k, _stream(words))
    return out


def unpack(blocks: torch.Tensor, gs: int, dtype: torch.dtype = torch.bfloat16):
    """``pack``'s inverse: blocks [E, N/32, K/gs, block] -> MLX words [E, N, K/8], scales and biases [E, N, K/gs]."""

    _need_cuda(blocks, "blocks")
    if blocks.dim() != 4 or blocks.shape[-1] != BLOCK or blocks.dtype != torch.int32:
        raise ValueError(f"blocks must be int32 [E, N/32, K/gs, {BLOCK}]")
    e, nb, kg, _ = blocks.shape
    n, k = nb * COLS, kg * gs
    blocks = blocks.contiguous()
    words = torch.empty((e, n, k // 8), dtype=torch.int32, device=blocks.device)
    scales = torch.empty((e, n, kg), dtype=dtype, device=blocks.device)
    biases = torch.empty_like(scales)
    with torch.cuda.device(blocks.device):
        _lib.call("tfb_unpack", blocks.data_ptr(), gs, words.data_ptr(), scales.data_ptr(), biases.data_ptr(), e, n, k,
                  _stream(blocks))
    return words, scales, biases


def dequantize(blocks: torch.Tensor, gs: int, *, prefill: bool = False,
               scale_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The weight values the kernels multiply by, [E, N, K]: fp32 fma(scale, q, bias) (decode form), or the prefill
    form's bf16 weights."""

    _need_cuda(blocks, "blocks")
    e, nb, kg, _ = blocks.shape
    n, k = nb * COLS, kg * gs
    blocks = blocks.contiguous()
    out = torch.empty((e, n, k), dtype=torch.bfloat16 if prefill else torch.float32, device=blocks.device)
    with torch.cuda.device(blocks.device):
        _lib.call("tfb_dequant", blocks.data_ptr(), gs, _SB[scale_dtype], 1 if prefill else 0, out.data_ptr(), e, n, k,
                  _stream(blocks))
    return out


@dataclass
class Experts:
    """One layer's experts (the shared ones included): gate and up (SwiGLU) or up (relu^2), and down."""

    up: torch.Tensor          # [E, NI/32, D/gs, M, block] int32, M = 2 (gate, then up) or 1
    down: torch.Tensor        # [E, D/32, NI/gs, 1, block]
    gs: int
    width: int                # NI: the expert's (or this rank's) intermediate width
    dims: int                 # D
    limit: float = 0.0        # SwiGLU clip (0: none)
    scale_dtype: torch.dtype = torch.bfloat16

    @property
    def count(self) -> int:
        return self.up.shape[0]

    @property
    def swiglu(self) -> bool:
        return self.up.shape[3] == 2

    def bytes_per_expert(self) -> int:
        return (self.up[0].numel() + self.down[0].numel()) * 4


def make(up: list[tuple], down: tuple, gs: int, *, limit: float = 0.0) -> Experts:
    """One layer's MLX arrays: ``up`` [gate, up] (SwiGLU) or [up] (relu^2), ``down``, each (words, scales, biases)."""

    if len(up) not in (1, 2):
        raise ValueError("experts take a gate and an up projection, or an up projection alone")
    width, dims = up[0][0].shape[1], up[0][0].shape[2] * 8
    dtype = up[0][1].dtype
    if any(m[1].dtype != dtype for m in (*up, down)):
        raise ValueError("every projection's scales must share one dtype")
    if dtype not in _SB:
        raise ValueError(f"scales must be bf16 or fp16, not {dtype}")
    u = torch.stack([pack(*m, gs) for m in up], dim=3)
    d = pack(*down, gs).unsqueeze(3)
    return Experts(u, d, gs, width, dims, float(limit), dtype)


def max_items(pairs: int, experts: int, tile: int = TILE) -> int:
    """Items a plan of ``pairs`` can hold: an expert with c pairs makes 1 + (c - 1) // tile items, so u experts in use
    make at most u + (pairs - u) // tile, which grows with u <= min(pairs, experts).  (The reference's bound,
    ``min(pairs, experts) + pairs // tile``, is the same idea with pairs not reduced; the grids sized by this one
    launch fewer blocks that find no item.)"""

    used = min(pairs, experts)
    return used + (pairs - used) // tile


class Plan:
    """Scratch grouping pairs by expert: members, items (expert, first, count), counts [items, distinct experts]."""

    def __init__(self, rows: int, slots: int, experts: int, device: torch.device | str, *,
                 prefill: bool = False, decode_tile: int = TILE, hot: int = 0) -> None:
        """``hot`` > 0 (decode plans only): experts with at least that many pairs are planned apart
        (``route_split``) and run through the prompt-form kernel, the rest through the decode form."""

        if decode_tile not in (TILE, WIDE_TILE):
            raise ValueError(f"decode items hold {TILE} or {WIDE_TILE} pairs")
        if hot and prefill:
            raise ValueError("a prompt plan has no hot experts to set apart")
        pairs = rows * slots
        self.rows, self.slots, self.experts, self.prefill = rows, slots, experts, prefill
        self.decode_tile = decode_tile
        self.tile = PREFILL_TILE if prefill else decode_tile
        self.members = torch.zeros((pairs,), dtype=torch.int32, device=device)
        self.items = torch.zeros((max_items(pairs, experts, TILE), 3), dtype=torch.int32, device=device)
        self.counts = torch.zeros((2,), dtype=torch.int32, device=device)
        self.hot = int(hot)
        if self.hot:
            big = max_items(pairs, experts, PREFILL_TILE)
            self.big_items = torch.zeros((big, 3), dtype=torch.int32, device=device)
            self.big_counts = torch.zeros((2,), dtype=torch.int32, device=device)
            # the hot experts' prompt-form launches run beside the decode-form launch, on a stream of their own
            self.side = torch.cuda.Stream(device)
            self.forked, self.joined = torch.cuda.Event(), torch.cuda.Event()
        self.rank = torch.zeros((1,), dtype=torch.int32, device=device)     # unused here; kept for the surface
        self.hist = torch.zeros((1,), dtype=torch.int32, device=device)


def route(picks: torch.Tensor, plan: Plan, tile: int = PREFILL_TILE) -> None:
    """``picks`` [R, slots] int32, contiguous: each pair's expert; a prompt plan's items hold ``tile``, its kernel's."""

    rows, slots = picks.shape
    if slots != plan.slots or rows > plan.rows:
        raise ValueError(f"picks {tuple(picks.shape)} do not fit a plan of {plan.rows} x {plan.slots}")
    if picks.dtype != torch.int32 or not picks.is_contiguous():
        raise ValueError("picks must be contiguous int32")
    _need_cuda(picks, "picks")
    plan.tile = tile if plan.prefill else plan.decode_tile
    if plan.tile < TILE:
        raise ValueError(f"items hold at least {TILE} pairs")
    with torch.cuda.device(picks.device):
        _lib.call("tfb_plan", picks.data_ptr(), rows * slots, plan.experts, plan.tile, plan.members.data_ptr(),
                  plan.items.data_ptr(), plan.counts.data_ptr(), _stream(picks))


def route_split(picks: torch.Tensor, plan: Plan, lo: int = 0) -> None:
    """``route`` for a plan made with ``hot``: experts (ids ``lo .. lo + plan.experts``) with at least ``plan.hot``
    pairs get items of up to ``PREFILL_TILE`` pairs in ``plan.big_items``; the others decode items in ``plan.items``."""

    rows, slots = picks.shape
    if not plan.hot:
        raise ValueError("the plan was made without hot=")
    if slots != plan.slots or rows > plan.rows or picks.dtype != torch.int32 or not picks.is_contiguous():
        raise ValueError(f"picks {tuple(picks.shape)} do not fit a plan of {plan.rows} x {plan.slots}")
    _need_cuda(picks, "picks")
    plan.tile = plan.decode_tile
    with torch.cuda.device(picks.device):
        _lib.call("tfb_plan_split", picks.data_ptr(), rows * slots, lo, plan.experts, plan.tile, PREFILL_TILE, plan.hot,
                  plan.members.data_ptr(), plan.items.data_ptr(), plan.counts.data_ptr(), plan.big_items.data_ptr(),
                  plan.big_counts.data_ptr(), _stream(picks))


class _BigPart:
    """The hot experts' half of a split plan, shaped like a prompt plan for ``_run``."""

    def __init__(self, plan: Plan) -> None:
        self.items, self.counts, self.members = plan.big_items, plan.big_counts, plan.members
        self.tile, self.slots, self.experts, self.prefill = PREFILL_TILE, plan.slots, plan.experts, True


class _beside:
    """The launches inside the block go to the plan's side stream, which first waits for everything enqueued on the
    current stream (the plan, the inputs); ``_rejoin`` makes the current stream wait for them.  A split plan's
    hot experts (one prompt-form pass over an expert's weights for up to 192 pairs, a long chain on few SMs) thereby
    run beside the other experts' decode-form launch instead of after it.  Captured in a CUDA graph the two become
    parallel branches.  For a plan without hot experts the block is skipped (``as hot`` is False)."""

    def __init__(self, plan, device) -> None:
        self.plan, self.device, self.ctx = plan, device, None

    def __enter__(self) -> bool:
        if not self.plan.hot:
            return False
        self.plan.forked.record(torch.cuda.current_stream(self.device))
        self.plan.side.wait_event(self.plan.forked)
        self.ctx = torch.cuda.stream(self.plan.side)
        self.ctx.__enter__()
        return True

    def __exit__(self, *exc) -> None:
        if self.ctx is not None:
            self.plan.joined.record(self.plan.side)
            self.ctx.__exit__(*exc)


def _rejoin(plan, device) -> None:
    if plan.hot:
        torch.cuda.current_stream(device).wait_event(plan.joined)


def _check_x(x: torch.Tensor, k: int) -> None:
    _need_cuda(x, "x")
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1 or x.stride(0) % 8 or x.shape[1] != k:
        raise ValueError("x: bf16 rows of K = groups * group size inputs, 16-byte aligned")


def _run(epi: int, x: torch.Tensor, slots: int, w: torch.Tensor, kg: int, nb: int, plan: Plan, out: torch.Tensor,
         n: int, limit: float, items: int, ex: Experts, prefill: bool = False) -> None:
    _check_x(x, kg * ex.gs)
    want = torch.float32 if epi == 0 else torch.bfloat16
    if prefill and plan.tile > PREFILL_TILE:
        raise ValueError(f"a prompt item holds at most {PREFILL_TILE} pairs")
    if out.dtype != want or not out.is_contiguous() or out.shape[-1] != n:
        raise ValueError("out: contiguous rows of n columns of the epilogue's dtype")
    if not w.is_contiguous():
        raise ValueError("w must be contiguous")
    with torch.cuda.device(x.device):
        if prefill:
            _lib.call("tfb_experts_prefill", ex.gs, epi, x.data_ptr(), x.stride(0), slots, w.data_ptr(), kg, nb,
                      plan.items.data_ptr(), plan.counts.data_ptr(), plan.members.data_ptr(), out.data_ptr(), n,
                      float(limit), items, _SB[ex.scale_dtype], _stream(x))
        else:
            _lib.call("tfb_experts_run_tile", ex.gs, epi, x.data_ptr(), x.stride(0), slots, w.data_ptr(), kg, nb,
                      plan.items.data_ptr(), plan.counts.data_ptr(), plan.members.data_ptr(), out.data_ptr(), n,
                      float(limit), items * nb, _SB[ex.scale_dtype], plan.tile, _stream(x))


def gate_up(x: torch.Tensor, ex: Experts, plan: Plan, out: torch.Tensor, rows: int) -> None:
    """x [R, D] bf16 (unit-stride rows) -> out [R * slots, NI] bf16, each pair's activation."""

    items = max_items(rows * plan.slots, plan.experts, plan.tile)
    epi = 2 if ex.swiglu else 1
    with _beside(plan, x.device) as hot:                     # the hot experts' pairs: other rows of the same output
        if hot:
            big = max_items(rows * plan.slots, plan.experts, PREFILL_TILE)
            _run(epi, x, plan.slots, ex.up, ex.dims // ex.gs, ex.width // COLS, _BigPart(plan), out, ex.width,
                 ex.limit, big, ex, True)
    _run(epi, x, plan.slots, ex.up, ex.dims // ex.gs, ex.width // COLS, plan, out, ex.width, ex.limit, items, ex,
         plan.prefill)
    _rejoin(plan, x.device)


def down(act: torch.Tensor, ex: Experts, plan: Plan, out: torch.Tensor, rows: int) -> None:
    """act [R * slots, NI] bf16 -> out [R * slots, D] per pair: fp32, or bf16 on a prefill plan when ``out`` is bf16."""

    items = max_items(rows * plan.slots, plan.experts, plan.tile)
    epi = 3 if plan.prefill and out.dtype == torch.bfloat16 else 0
    with _beside(plan, act.device) as hot:
        if hot:
            big = max_items(rows * plan.slots, plan.experts, PREFILL_TILE)
            _run(epi, act, 0, ex.down, ex.width // ex.gs, ex.dims // COLS, _BigPart(plan), out, ex.dims, 0.0, big, ex,
                 True)
    _run(epi, act, 0, ex.down, ex.width // ex.gs, ex.dims // COLS, plan, out, ex.dims, 0.0, items, ex, plan.prefill)
    _rejoin(plan, act.device)


def down_combine(act: torch.Tensor, ex: Experts, plan: Plan, y: torch.Tensor, rows: int, wts: torch.Tensor,
                 out: torch.Tensor, arrive: torch.Tensor) -> None:
    """``down`` (decode form) and the slot-order weighted combine in one launch: y [R * slots, D] fp32 per pair as
    ``down`` stores it, and out [R, D] (bf16 or fp32) = the sum over each row's slots of wts * y, formed by whichever
    block stores a row's last slot.  Every (row, slot) pair must be in the plan; ``arrive`` is int32 scratch
    [R, D / 32], zero before the first call (a call leaves it zero)."""

    if plan.prefill or plan.hot:
        raise ValueError("the fused combine follows the decode form of a plain plan")
    if y.dtype != torch.float32 or not y.is_contiguous() or y.shape[-1] != ex.dims:
        raise ValueError("y: contiguous fp32 rows of D columns")
    if out.dtype not in (torch.bfloat16, torch.float32) or not out.is_contiguous() or out.shape[-1] != ex.dims:
        raise ValueError("out: contiguous bf16 or fp32 rows of D columns")
    if wts.dtype != torch.float32 or not wts.is_contiguous() or wts.shape[-1] != plan.slots:
        raise ValueError("wts: contiguous fp32 [R, slots]")
    nb = ex.dims // COLS
    if arrive.dtype != torch.int32 or arrive.numel() < rows * nb:
        raise ValueError(f"arrive: int32 scratch of at least {rows * nb} entries")
    _check_x(act, ex.width)
    if not ex.down.is_contiguous():
        raise ValueError("w must be contiguous")
    items = max_items(rows * plan.slots, plan.experts, plan.tile)
    with torch.cuda.device(act.device):
        _lib.call("tfb_experts_down_combine", ex.gs, act.data_ptr(), act.stride(0), ex.down.data_ptr(),
                  ex.width // ex.gs, nb, plan.items.data_ptr(), plan.counts.data_ptr(), plan.members.data_ptr(),
                  y.data_ptr(), ex.dims, items * nb, _SB[ex.scale_dtype], plan.tile, wts.data_ptr(), plan.slots,
                  out.data_ptr(), 1 if out.dtype == torch.float32 else 0, arrive.data_ptr(), _stream(act))
