"""Softmax top-k MoE with an optional sigmoid-gated shared expert, on fp32 logits (ties to the lower id).

Mirrors ``src/tensorfold/cuda/moe.py`` of the reference (router, select_rows, select, moe, combine, MoEBuffers,
Routed, run) over hand-written sm_100a kernels; each row routes and runs on its own.  ``shared=True`` is the
reference's layout (router rows [E + 1, D], slot k = expert E behind a sigmoid gate); ``shared=False`` drops that
slot for layers without a shared expert.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from . import experts as grouped


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def router(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor | None = None, *, prompt: bool = False) -> torch.Tensor:
    """x [R, D] bf16, rows [NE, D] bf16 (router rows, then the shared expert's gate row if any) -> [R, NE] fp32.
    ``prompt``: the tensor-core form (the prefill arithmetic's router: its own fixed summation order, so the last bits
    differ from the decode form's; a row's bits still do not depend on the other rows)."""

    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor (this library has no CPU path)")
    if x.dtype != torch.bfloat16 or rows.dtype != torch.bfloat16 or x.dim() != 2 or rows.dim() != 2:
        raise ValueError("router: x and rows must be 2-D bf16")
    m, d = x.shape
    ne = rows.shape[0]
    if rows.shape[1] != d or x.stride(1) != 1 or not rows.is_contiguous():
        raise ValueError("router: x [R, D] with unit-stride rows, rows [NE, D] contiguous")
    if out is None:
        out = torch.empty((m, ne), dtype=torch.float32, device=x.device)
    elif out.shape != (m, ne) or out.dtype != torch.float32 or not out.is_contiguous():
        raise ValueError("router: out must be contiguous fp32 [R, NE]")
    with torch.cuda.device(x.device):
        _lib.call("tfb_router_prompt" if prompt and d % 32 == 0 else "tfb_router", x.data_ptr(), x.stride(0),
                  rows.data_ptr(), out.data_ptr(), m, d, ne, _stream(x))
    return out


class MoEBuffers:
    """Static scratch for up to ``rows`` rows (CUDA-graph safe); ``prefill`` picks the experts' prefill arithmetic."""

    def __init__(self, rows: int, cfg, device: torch.device | str, *, prefill: bool = False,
                 shared: bool = True) -> None:
        extra = 1 if shared else 0
        slots = cfg.num_experts_per_tok + extra
        self.rows, self.slots, self.shared = rows, slots, shared
        self.logits = torch.empty((rows, cfg.num_experts + extra), dtype=torch.float32, device=device)
        self.pick = torch.empty((rows, slots), dtype=torch.int32, device=device)
        self.wts = torch.empty((rows, slots), dtype=torch.float32, device=device)
        self.plan = grouped.Plan(rows, slots, cfg.num_experts + extra, device, prefill=prefill)
        self.act = torch.empty((rows, slots, cfg.moe_intermediate_size), dtype=torch.bfloat16, device=device)
        self.y = torch.empty((rows, slots, cfg.hidden_size), dtype=torch.bfloat16 if prefill else torch.float32,
                             device=device)
        # arrival counters of the kernels that finish their work in whichever block comes last (zero between calls):
        # the one-launch routing (one a group of eight rows, plus one) and the combine folded into the down projection
        self.arrive_route = torch.zeros((2 + rows // 8,), dtype=torch.int32, device=device)
        self.arrive_combine = torch.zeros((rows * (cfg.hidden_size // grouped.COLS),), dtype=torch.int32, device=device)


def select_rows(logits: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int) -> None:
    """Each row's experts and weights, rows in parallel (buf.pick, buf.wts)."""

    rows, nl = logits.shape
    shared = buf.slots == top_k + 1
    if buf.slots not in (top_k, top_k + 1) or rows > buf.rows:
        raise ValueError(f"{rows} rows of top-{top_k} do not fit buffers of {buf.rows} x {buf.slots}")
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise ValueError("logits must be contiguous fp32")
    with torch.cuda.device(logits.device):
        _lib.call("tfb_select_rows", logits.data_ptr(), nl, buf.pick.data_ptr(), buf.wts.data_ptr(), rows, experts,
                  top_k, 1 if shared else 0, _stream(logits))


def select_sigmoid(logits: torch.Tensor, bias: torch.Tensor, pick: torch.Tensor, wts: torch.Tensor, top_k: int,
                   experts: int, scale: float, norm: bool, shared_slots: int = 1) -> None:
    """The sigmoid-plus-bias routers' selection (GLM: ``glue.select``, one shared slot; Nemotron: two): each row's
    top-k experts by ``sigmoid(logit) + bias`` (ties to the lower id), weights = the picked scores, normalised in pick
    order when ``norm``, times ``scale``; then the shared slots (ids ``experts``, ``experts + 1``, weight 1)."""

    rows, nl = logits.shape
    slots = top_k + shared_slots
    if logits.dtype != torch.float32 or not logits.is_contiguous() or not logits.is_cuda:
        raise ValueError("logits must be contiguous CUDA fp32")
    if bias.dtype != torch.float32 or bias.numel() < experts or not bias.is_contiguous():
        raise ValueError("bias must be contiguous fp32 [experts]")
    for t, dt in ((pick, torch.int32), (wts, torch.float32)):
        if t.dtype != dt or not t.is_contiguous() or t.shape[0] < rows or t.shape[1] != slots:
            raise ValueError(f"pick / wts must be contiguous [{rows}, {slots}] int32 / fp32")
    with torch.cuda.device(logits.device):
        _lib.call("tfb_select_sigmoid", logits.data_ptr(), nl, bias.data_ptr(), pick.data_ptr(), wts.data_ptr(), rows,
                  experts, top_k, shared_slots, float(scale), 1 if norm else 0, _stream(logits))


# Up to this many rows the one-block kernel that selects and plans in one launch is used; above it the selection runs
# on many blocks and the plan follows as its own launch (measured inside a CUDA graph: 5.7 against 8.8 us at 64 rows).
FUSED_SELECT_ROWS = 32


def fused_select_rows() -> int:
    return min(FUSED_SELECT_ROWS, _lib.lib().tfb_select_plan_max_rows())


def select(logits: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int,
           tile: int = grouped.PREFILL_TILE) -> None:
    """Each row's experts and weights (rows in parallel), then the pairs grouped by expert, ``tile`` a prompt's item."""

    rows, nl = logits.shape
    plan = buf.plan
    if rows <= fused_select_rows() and logits.is_contiguous() and logits.dtype == torch.float32:
        shared = buf.slots == top_k + 1
        if buf.slots not in (top_k, top_k + 1) or rows > buf.rows or plan.slots != buf.slots:
            raise ValueError(f"{rows} rows of top-{top_k} do not fit buffers of {buf.rows} x {buf.slots}")
        plan.tile = tile if plan.prefill else plan.decode_tile
        with torch.cuda.device(logits.device):
            _lib.call("tfb_select_plan", logits.data_ptr(), nl, buf.pick.data_ptr(), buf.wts.data_ptr(), rows, experts,
                      top_k, 1 if shared else 0, plan.tile, plan.members.data_ptr(), plan.items.data_ptr(),
                      plan.counts.data_ptr(), _stream(logits))
        return
    select_rows(logits, buf, top_k, experts)
    grouped.route(buf.pick[:rows], plan, tile)


# Rows up to which the layer uses the one-launch routing (``route``) and the combine folded into the down projection
# (``experts.down_combine``).  Both give the separate launches' bits.  Off unless set: measured on config 2 inside a
# CUDA graph with programmatic dependent launch, a launch boundary costs about what the hand-over inside a kernel
# costs (a block's release of its results, about a microsecond), so neither makes the layer faster - one-launch
# routing: 26.5 -> 28.2 us at 1 row, 40.0 -> 39.5 at 4, 69.5 -> 69.1 at 16, 98.7 -> 99.0 at 64; folded combine:
# 26.5 -> 26.7, 40.0 -> 40.1, 69.5 -> 71.6, 98.7 -> 106.2.
FUSED_ROUTE_ROWS = 0
FUSED_COMBINE_ROWS = 0


def route_rows(router_rows: torch.Tensor) -> int:
    """Up to this many rows the router, the selection and the plan can be one launch (``route``)."""

    return _lib.lib().tfb_route_max_rows(router_rows.shape[0])


def route(x: torch.Tensor, router_rows: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int,
          tile: int = grouped.PREFILL_TILE) -> None:
    """``router`` then ``select`` for a few rows in ONE launch (the same logits, picks, weights and plan): the block
    that completes a group of eight rows selects them, the block that completes the last group plans."""

    rows, d = x.shape
    ne, plan = router_rows.shape[0], buf.plan
    shared = buf.slots == top_k + 1
    if not x.is_cuda or x.dtype != torch.bfloat16 or router_rows.dtype != torch.bfloat16 or x.stride(1) != 1 \
            or router_rows.shape[1] != d or not router_rows.is_contiguous():
        raise ValueError("route: x [R, D] bf16 with unit-stride rows, rows [NE, D] contiguous bf16")
    if buf.slots not in (top_k, top_k + 1) or rows > buf.rows or plan.slots != buf.slots or buf.logits.shape[1] != ne:
        raise ValueError(f"{rows} rows of top-{top_k} do not fit buffers of {buf.rows} x {buf.slots}")
    if rows > route_rows(router_rows):
        raise ValueError(f"route: at most {route_rows(router_rows)} rows in one launch")
    plan.tile = tile if plan.prefill else plan.decode_tile
    with torch.cuda.device(x.device):
        _lib.call("tfb_route", x.data_ptr(), x.stride(0), router_rows.data_ptr(), buf.logits.data_ptr(), rows, d, ne,
                  experts, top_k, 1 if shared else 0, buf.pick.data_ptr(), buf.wts.data_ptr(), plan.tile, 0,
                  plan.experts, plan.members.data_ptr(), plan.items.data_ptr(), plan.counts.data_ptr(),
                  buf.arrive_route.data_ptr(), _stream(x))


def _route_any(x: torch.Tensor, router_rows: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int) -> int:
    """The routing stage by the fewest launches available; returns how many it took."""

    rows = x.shape[0]
    if rows <= min(FUSED_ROUTE_ROWS, route_rows(router_rows)) and x.stride(1) == 1 \
            and buf.plan.experts == router_rows.shape[0]:
        route(x, router_rows, buf, top_k, experts)
        return 1
    router(x, router_rows, buf.logits[:rows], prompt=buf.plan.prefill)
    select(buf.logits[:rows], buf, top_k, experts)
    return 2 if rows <= fused_select_rows() else 3


def moe(x: torch.Tensor, router_rows: torch.Tensor, ex: grouped.Experts, buf: MoEBuffers, top_k: int,
        experts: int) -> MoEBuffers:
    """Route x [R, D] and run its experts into buf.y [R, slots, D] (bf16 in prefill)."""

    rows = x.shape[0]
    _route_any(x, router_rows, buf, top_k, experts)
    grouped.gate_up(x, ex, buf.plan, buf.act.view(-1, ex.width), rows)
    grouped.down(buf.act.view(-1, ex.width), ex, buf.plan, buf.y.view(-1, ex.dims), rows)
    return buf


def layer(x: torch.Tensor, m: "Routed", buf: MoEBuffers, out: torch.Tensor) -> int:
    """The whole layer on x [R, D] into ``out`` [R, D] (bf16 or fp32; device or pinned host memory): ``moe`` and
    ``combine`` with the combine folded into the down projection in the decode form - three launches for a few rows,
    five for a decode batch, six for a prompt.  buf.y still holds every slot's row.  Returns the launches made."""

    rows, ex = x.shape[0], m.experts
    launches = _route_any(x, m.router, buf, m.top_k, m.count)
    grouped.gate_up(x, ex, buf.plan, buf.act.view(-1, ex.width), rows)
    if buf.plan.prefill or buf.plan.hot or rows > FUSED_COMBINE_ROWS:
        grouped.down(buf.act.view(-1, ex.width), ex, buf.plan, buf.y.view(-1, ex.dims), rows)
        combine(buf.y[:rows], buf.wts[:rows], out)
        return launches + 3
    grouped.down_combine(buf.act.view(-1, ex.width), ex, buf.plan, buf.y.view(-1, ex.dims), rows, buf.wts, out,
                         buf.arrive_combine)
    return launches + 2


def combine(y: torch.Tensor, wts: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """y [R, S, D] (fp32, or bf16 in prefill) and wts [R, S] fp32 -> [R, D] bf16 (or fp32 when ``out`` is fp32)."""

    rows, slots, dims = y.shape
    if y.dtype not in (torch.float32, torch.bfloat16) or not y.is_contiguous() or not wts.is_contiguous():
        raise ValueError("combine: y must be contiguous fp32 or bf16, wts contiguous fp32")
    if out is None:
        out = torch.empty((rows, dims), dtype=torch.bfloat16, device=y.device)
    with torch.cuda.device(y.device):
        _lib.call("tfb_combine", y.data_ptr(), 1 if y.dtype == torch.bfloat16 else 0, wts.data_ptr(), out.data_ptr(),
                  1 if out.dtype == torch.float32 else 0, rows, slots, dims, _stream(y))
    return out


def add_moe_norm(h: torch.Tensor, y: torch.Tensor, wt: torch.Tensor, w: torch.Tensor, eps: float, top_k: int):
    """The step behind a MoE block in one launch: h [R, D] bf16, y [R * NS, D] (fp32, or bf16 in prefill), wt [R, NS]
    fp32, w [D] bf16 -> (h + delta, its RMSNorm times w, the norm's sums over groups of 64), delta = the first ``top_k``
    slots weighted plus the shared slots, summed in slot order and rounded to bf16.  Mirrors the Nemotron family's
    ``glue.add_moe_norm`` (``src/tensorfold/families/nemotron_h/cuda/glue.py:128-141``)."""

    rows, d = h.shape
    slots = wt.shape[1]
    if not h.is_cuda or h.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not h.is_contiguous() or w.numel() != d:
        raise ValueError("add_moe_norm: h [R, D] and w [D] must be contiguous CUDA bf16")
    if y.dtype not in (torch.float32, torch.bfloat16) or not y.is_contiguous() or y.numel() != rows * slots * d:
        raise ValueError("add_moe_norm: y must be contiguous fp32 or bf16 [R * NS, D]")
    if wt.dtype != torch.float32 or not wt.is_contiguous() or wt.shape[0] != rows or not 0 <= top_k <= slots:
        raise ValueError("add_moe_norm: wt must be contiguous fp32 [R, NS] with top_k <= NS")
    hn, out = torch.empty_like(h), torch.empty_like(h)
    xs = torch.empty((rows, d // 64), dtype=torch.float32, device=h.device)
    with torch.cuda.device(h.device):
        _lib.call("tfb_add_moe_norm", h.data_ptr(), y.data_ptr(), 1 if y.dtype == torch.bfloat16 else 0, wt.data_ptr(),
                  w.contiguous().data_ptr(), hn.data_ptr(), out.data_ptr(), xs.data_ptr(), rows, d, slots, top_k,
                  float(eps), _stream(h))
    return hn, out, xs


@dataclass
class Routed:
    """A layer's router rows ([E + 1, D] bf16 with the shared expert's gate row last, or [E, D]) and its experts."""

    router: torch.Tensor
    experts: grouped.Experts
    top_k: int
    shared: bool = True

    @property
    def count(self) -> int:
        return self.router.shape[0] - (1 if self.shared else 0)


class _Shape:
    def __init__(self, m: Routed) -> None:
        self.num_experts_per_tok, self.num_experts = m.top_k, m.count
        self.moe_intermediate_size, self.hidden_size = m.experts.width, m.experts.dims


_scratch: dict[tuple, MoEBuffers] = {}


def run(x: torch.Tensor, m: Routed, *, prefill: bool = False) -> torch.Tensor:
    """x [R, D] bf16 -> [R, D] bf16: its top-k experts by renormalized softmax weight (plus the shared expert)."""

    rows = x.shape[0]
    size = 1 << max(4, (rows - 1).bit_length())                 # scratch per power of two, reused by every layer
    key = (size, m.count, m.top_k, m.experts.width, m.experts.dims, prefill, m.shared, x.device)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = MoEBuffers(size, _Shape(m), x.device, prefill=prefill, shared=m.shared)
    out = torch.empty((rows, m.experts.dims), dtype=torch.bfloat16, device=x.device)
    layer(x.contiguous(), m, buf, out)
    return out


class Runner:
    """One layer at a fixed row count captured in a CUDA graph: ``runner(x)`` copies ``x`` (host or device) into the
    static input, replays the layer's launches and returns the static bf16 output [rows, D].

    The reference's families replay their decode steps from CUDA graphs the same way
    (``src/tensorfold/families/qwen3_5/cuda/forward.py`` tree_forward); the kernels read the routing on the device, so
    a replay follows the new input's experts."""

    def __init__(self, m: Routed, rows: int, *, prefill: bool = False, device=None) -> None:
        device = torch.device(device if device is not None else m.router.device)
        self.layer, self.rows, self.prefill = m, rows, prefill
        self.x = torch.zeros((rows, m.experts.dims), dtype=torch.bfloat16, device=device)
        self.buf = MoEBuffers(rows, _Shape(m), device, prefill=prefill, shared=m.shared)
        self.out = torch.zeros((rows, m.experts.dims), dtype=torch.bfloat16, device=device)
        self._stream = torch.cuda.Stream(device)
        with torch.cuda.device(device):
            self._stream.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(self._stream):
                self.launches = self._step()                       # warm up outside the capture
            torch.cuda.current_stream(device).wait_stream(self._stream)
            torch.cuda.synchronize(device)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self._stream):
                self._step()

    def _step(self) -> int:
        return layer(self.x, self.layer, self.buf, self.out)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        self.x.copy_(x, non_blocking=True)
        return self.replay()

    def bind_host(self, x_host: torch.Tensor, out_host: torch.Tensor, direct: bool = True) -> None:
        """Capture the step together with its transfers from ``x_host`` and to ``out_host`` (both pinned host memory,
        the caller's staging buffers): ``replay_host()`` is then one graph launch a step, transfers included.
        ``direct``: the rows are pulled from the pinned buffer by a kernel and the combine kernel stores the result
        rows straight into the pinned buffer (no copy-engine nodes in the graph); else two memcpy nodes."""

        want = (self.rows, self.layer.experts.dims)
        for t in (x_host, out_host):
            if t.device.type != "cpu" or not t.is_pinned() or tuple(t.shape) != want or t.dtype != torch.bfloat16:
                raise ValueError(f"host buffers must be pinned bf16 tensors of shape {want}")
        self.x_host, self.out_host = x_host, out_host
        device = self.x.device
        with torch.cuda.device(device):
            self._stream.wait_stream(torch.cuda.current_stream(device))
            self.host_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.host_graph, stream=self._stream):
                if direct:
                    _lib.call("tfb_peer_stage", x_host.data_ptr(), self.x.data_ptr(), 0,
                              self.x.numel() * self.x.element_size(), self._stream.cuda_stream)
                    layer(self.x, self.layer, self.buf, out_host)
                else:
                    self.x.copy_(x_host, non_blocking=True)
                    self._step()
                    out_host.copy_(self.out, non_blocking=True)

    def replay_host(self) -> torch.Tensor:
        """Tokens from the bound host buffer through the layer into the bound host buffer (asynchronous: synchronise
        the current stream before reading it)."""

        self.host_graph.replay()
        return self.out_host
