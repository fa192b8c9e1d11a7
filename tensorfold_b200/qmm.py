"""Dense 4-bit lane matmul (the projections either side of the MoE block) on the experts' kernels: the weight is one
"expert" and every input row one pair, so the arithmetic, the K slicing by shape and the row invariance are the
experts' - a row's bits never depend on how many rows run with it.

Mirrors ``tensorfold.cuda.kernels.qmm`` (``src/tensorfold/cuda/kernels/qmm.py:41-219``): ``Q4``, ``pack`` / ``unpack``,
``matmul``, ``prefill_matmul``, ``group_sums``, ``split_k``, ``bucket``.  Differences a caller can see: the packed words
use this library's block order (``unpack`` inverts it bit for bit), n is padded to 32 (the reference pads to 128),
``matmul`` adds its K slices inside the kernel in slice order (``reduce=False`` hands them out apart, as the reference
does), the slicing is the shape's and cannot be chosen per call, and the group sums the reference passes in (``xs``)
are formed inside the kernel from the same inputs, so ``xs`` is accepted and not read.
No CPU path.
"""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace

import torch

from . import _lib
from . import experts as grouped

_PLANS: dict = {}


@dataclass
class Q4:
    """Packed (n, k): blocks int32 [1, n_pad/32, k/gs, 288] (nibbles and their scales and biases together)."""

    weight: torch.Tensor
    scale_dtype: torch.dtype
    n: int
    k: int
    gs: int

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    @property
    def n_pad(self) -> int:
        return self.weight.shape[1] * grouped.COLS


def pack(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, gs: int) -> Q4:
    """MLX (n, k/8) words, (n, k/gs) scales and biases (bf16 or fp16) -> ``Q4``; n padded to 32 with zeros."""

    words = weight.view(torch.int32) if weight.dtype != torch.int32 else weight
    if words.dim() != 2 or scales.dim() != 2 or biases.shape != scales.shape:
        raise ValueError("pack: (n, k/8) words with (n, k/gs) scales and biases")
    n, k8 = words.shape
    pad = -n % grouped.COLS
    if pad:
        words = torch.cat([words, words.new_zeros((pad, k8))])
        scales = torch.cat([scales, scales.new_zeros((pad, scales.shape[1]))])
        biases = torch.cat([biases, biases.new_zeros((pad, biases.shape[1]))])
    blocks = grouped.pack(words[None], scales[None], biases[None], gs)
    return Q4(blocks, scales.dtype, n, k8 * 8, gs)


def unpack(q: Q4) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The stored MLX layout again: (n, k/8) int32 words, (n, k/gs) scales and biases."""

    words, scales, biases = grouped.unpack(q.weight, q.gs, q.scale_dtype)
    return words[0, :q.n].contiguous(), scales[0, :q.n].contiguous(), biases[0, :q.n].contiguous()


def split_k(n: int, k: int, gs: int = 64, target: int = 192) -> int:
    """K slices the kernel adds in order for an (n, k) weight: a function of the shape only, never of the rows."""

    return _lib.lib().tfb_decode_kslices(k // gs)


def bucket(m: int) -> int:
    """Rows an item holds (8 or 16); items never change bits."""

    if m < 1:
        raise ValueError("the lane matmul takes at least one row")
    return grouped.TILE if m <= grouped.TILE else grouped.WIDE_TILE


def group_sums(x: torch.Tensor, gs: int = 64) -> torch.Tensor:
    """(M, K) bf16 (rows may be strided) -> (M, K/gs) fp32 sums of each group's inputs."""

    if not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("group_sums: x must be CUDA (M, K) bf16 with unit-stride rows")
    m, k = x.shape
    xs = torch.empty((m, k // gs), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call("tfb_group_sums", x.data_ptr(), x.stride(0), xs.data_ptr(), m, k, gs,
                  torch.cuda.current_stream(x.device).cuda_stream)
    return xs


def _plan(m: int, device: torch.device, prefill: bool) -> grouped.Plan:
    """Every row is one pair of expert 0: the plan depends on (m, form) only and is made once."""

    key = (m, device.index, prefill)
    plan = _PLANS.get(key)
    if plan is None:
        plan = grouped.Plan(m, 1, 1, device, prefill=prefill, decode_tile=bucket(m))
        grouped.route(torch.zeros((m, 1), dtype=torch.int32, device=device), plan, grouped.PREFILL_TILE)
        torch.cuda.current_stream(device).synchronize()
        _PLANS[key] = plan
    return plan


def _check(x: torch.Tensor, q: Q4, what: str) -> torch.Tensor:
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != q.k:
        raise ValueError(f"{what}: x must be CUDA (M, {q.k}) bf16")
    if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8) or x.data_ptr() % 16:
        x = x.clone(memory_format=torch.contiguous_format)          # rows are read in 16-byte pieces
    return x


def _run(x: torch.Tensor, q: Q4, f32: bool, out: torch.Tensor | None, prefill: bool) -> torch.Tensor:
    m = x.shape[0]
    want = torch.float32 if f32 else torch.bfloat16
    if out is not None and (out.shape != (m, q.n) or out.dtype != want or not out.is_contiguous()):
        raise ValueError(f"out must be contiguous ({m}, {q.n}) {want}")
    padded = q.n_pad != q.n
    dst = out if out is not None and not padded else torch.empty((m, q.n_pad), dtype=want, device=x.device)
    plan = _plan(m, x.device, prefill)
    ex = SimpleNamespace(gs=q.gs, scale_dtype=q.scale_dtype)
    items = grouped.max_items(m, 1, plan.tile)
    grouped._run(0 if f32 else 3, x, 0, q.weight, q.k // q.gs, q.n_pad // grouped.COLS, plan, dst, q.n_pad, 0.0, items,
                 ex, prefill)
    if not padded:
        return dst
    if out is None:
        return dst[:, :q.n].contiguous()
    out.copy_(dst[:, :q.n])
    return out


def matmul(x: torch.Tensor, q: Q4, xs: torch.Tensor | None = None, *, sk: int | None = None, f32: bool = False,
           out: torch.Tensor | None = None, part: torch.Tensor | None = None, reduce: bool = True) -> torch.Tensor:
    """x @ q.T as (M, n) bf16, or unrounded fp32 with ``f32``: exact integer products per group, then
    ``acc = fma(xs, b, fma(p, s, acc))`` in fp32 (the decode arithmetic).  ``reduce=False`` returns the K slices apart,
    fp32 (split_k, M, n) (in ``part`` when given), for a caller that adds them in slice order inside its next kernel;
    with one slice it returns the product itself, as the reference does
    (``src/tensorfold/cuda/kernels/qmm.py:156-177``)."""

    slices = split_k(q.n, q.k, q.gs)
    if sk is not None and sk != slices:
        raise ValueError("matmul: the K slicing is the shape's (split_k), it cannot be chosen per call")
    x = _check(x, q, "matmul")
    if reduce or slices == 1:
        return _run(x, q, f32, out, False)
    return _slices(x, q, slices, part)


def _slices(x: torch.Tensor, q: Q4, slices: int, part: torch.Tensor | None) -> torch.Tensor:
    m = x.shape[0]
    need = slices * m * q.n
    padded = q.n_pad != q.n
    if part is not None and (part.dtype != torch.float32 or not part.is_contiguous() or part.numel() < need
                             or part.device != x.device):
        raise ValueError(f"part must be contiguous fp32 with at least {need} elements on x's device")
    dst = part.reshape(-1)[:need].view(slices, m, q.n) if part is not None and not padded else \
        torch.empty((slices, m, q.n_pad), dtype=torch.float32, device=x.device)
    plan = _plan(m, x.device, False)
    with torch.cuda.device(x.device):
        _lib.call("tfb_experts_run_slices", q.gs, x.data_ptr(), x.stride(0), 0, q.weight.data_ptr(), q.k // q.gs,
                  q.n_pad // grouped.COLS, plan.items.data_ptr(), plan.counts.data_ptr(), plan.members.data_ptr(),
                  dst.data_ptr(), q.n_pad, m, grouped.max_items(m, 1, plan.tile) * (q.n_pad // grouped.COLS),
                  0 if q.scale_dtype == torch.bfloat16 else 1, plan.tile, torch.cuda.current_stream(x.device).cuda_stream)
    if not padded:
        return dst
    if part is None:
        return dst[:, :, :q.n].contiguous()
    view = part.reshape(-1)[:need].view(slices, m, q.n)
    view.copy_(dst[:, :, :q.n])
    return view


def prefill_matmul(x: torch.Tensor, q: Q4, *, f32: bool = False, tile: int = 0,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """Prefill: weights rounded once to bf16, one fp32 chain over K (tcgen05); any chunking gives the same bits, not
    ``matmul``'s."""

    return _run(_check(x, q, "prefill_matmul"), q, f32, out, True)
