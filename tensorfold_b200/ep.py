"""Expert parallelism for the routed-expert layer: experts sharded over the ranks of a process group (expert ``e``
lives on rank ``e // (E / world)``), router rows and a shared expert replicated, tokens data parallel.

The reference has no expert parallelism (its only multi-GPU mode is 2-rank tensor parallelism with an all-gather of
fp32 partials, ``src/tensorfold/cuda/comm.py:69-76``); this is the sharding the routed path admits on an NVSwitch node.
Three forms of the two exchanges (tokens to the experts' owners, results back to the tokens' home ranks):

* ``PeerExpertParallel`` / ``PeerExl3ExpertParallel`` (the default, and what the benchmark times): this library's own
  kernels over NVLink peer memory (``csrc/peer.cu``) - every rank pulls all ranks' rows and selections after a flag
  barrier, and the kernel that forms a rank's per-token partial sums stores them straight into the home ranks; no
  collective-library call on the step, one CUDA graph a step.
* ``GatheredExpertParallel``: the same data flow through NCCL (all-gather of the tokens, reduce-scatter of per-pair
  rows - the exact one-GPU bits - or of per-token partial sums); the comparison arm.
* ``ExpertParallel``: counted dispatch with ``all_to_all_single`` (bf16 rows and ids out, fp32 rows back) and one host
  read of the counts a step; least link traffic, not graph-capturable.  Its index logic sits behind a small backend
  interface so CPU ranks (gloo) can exercise it with a stand-in; the product backend (``CudaBackend``) has no CPU path.

Rows are in the receiver's own memory before any expert kernel reads them.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib


class CudaBackend:
    """This rank's share of a layer on its GPU: full router rows, its slice of the routed experts, the shared expert."""

    def __init__(self, router_rows: torch.Tensor, local_experts, top_k: int, experts: int, shared_experts=None,
                 prefill_pairs: int = 24) -> None:
        from . import experts as grouped
        from . import moe

        self.moe, self.grouped = moe, grouped
        self.router_rows, self.local, self.top_k, self.experts = router_rows, local_experts, top_k, experts
        self.shared = shared_experts                      # an Experts object holding the one shared expert, or None
        self.prefill_pairs = prefill_pairs                # pairs a local expert from which the prefill form is used
        self.device = router_rows.device

    def route(self, x: torch.Tensor):
        m = self.moe
        slots = self.top_k + (1 if self.shared is not None else 0)

        class _Cfg:
            num_experts_per_tok, num_experts = self.top_k, self.experts
            moe_intermediate_size, hidden_size = self.local.width, self.local.dims

        buf = m.MoEBuffers(x.shape[0], _Cfg, self.device, shared=self.shared is not None)
        m.router(x, self.router_rows, buf.logits)
        m.select_rows(buf.logits, buf, self.top_k, self.experts)
        assert buf.slots == slots
        return buf.pick, buf.wts

    def _run(self, ex, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        g = self.grouped
        n = rows.shape[0]
        y = torch.empty((n, ex.dims), dtype=torch.float32, device=self.device)
        if n == 0:
            return y
        prefill = n >= self.prefill_pairs * ex.count
        plan = g.Plan(n, 1, ex.count, self.device, prefill=prefill)
        g.route(ids.view(n, 1).contiguous(), plan)
        act = torch.empty((n, ex.width), dtype=torch.bfloat16, device=self.device)
        g.gate_up(rows, ex, plan, act, n)
        g.down(act, ex, plan, y, n)
        return y

    def run_experts(self, rows: torch.Tensor, local_ids: torch.Tensor) -> torch.Tensor:
        return self._run(self.local, rows, local_ids)

    def run_shared(self, x: torch.Tensor) -> torch.Tensor:
        ids = torch.zeros((x.shape[0],), dtype=torch.int32, device=self.device)
        return self._run(self.shared, x, ids)

    def combine(self, y: torch.Tensor, wts: torch.Tensor) -> torch.Tensor:
        return self.moe.combine(y, wts)


@dataclass
class DispatchPlan:
    """Where a rank's routed pairs go: ``order`` sorts the pairs by owner rank (stable), ``send`` / ``recv`` are the
    per-peer row counts."""

    order: torch.Tensor
    send: list
    recv: list


class ExpertParallel:
    """One MoE layer over ``group``: ``forward(x_local)`` -> this rank's tokens' outputs [T_local, D] bf16."""

    def __init__(self, backend, experts: int, top_k: int, shared: bool, group=None) -> None:
        self.backend, self.experts, self.top_k, self.shared = backend, experts, top_k, shared
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if experts % self.world:
            raise ValueError(f"{experts} experts do not shard evenly over {self.world} ranks")
        self.per_rank = experts // self.world
        self.last_plan: DispatchPlan | None = None

    def plan_dispatch(self, pick_routed: torch.Tensor) -> DispatchPlan:
        """pick_routed [T, k]: owners, a stable sort of the pairs by owner, and the counts exchanged with the peers."""

        owner = (pick_routed.reshape(-1) // self.per_rank).to(torch.int64)
        order = torch.sort(owner, stable=True).indices
        send = torch.bincount(owner, minlength=self.world).to(torch.int64)
        recv = torch.empty_like(send)
        if self.world > 1:
            dist.all_to_all_single(recv, send, group=self.group)
        else:
            recv.copy_(send)
        return DispatchPlan(order, send.tolist(), recv.tolist())          # the one host read of a step

    def _exchange(self, rows: torch.Tensor, out_counts: list, in_counts: list) -> torch.Tensor:
        out = torch.empty((sum(in_counts), *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        if self.world > 1:
            dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=in_counts, input_split_sizes=out_counts,
                                   group=self.group)
        else:
            out.copy_(rows)
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        be, k = self.backend, self.top_k
        rows, dims = x.shape
        pick, wts = be.route(x)                                            # [T, slots], slot k = the shared expert
        slots = pick.shape[1]
        routed = pick[:, :k].contiguous()
        plan = self.plan_dispatch(routed)
        self.last_plan = plan
        pair_rows = (plan.order // k)                                      # the token of each sorted pair
        send_rows = x.index_select(0, pair_rows)
        send_ids = (routed.reshape(-1).index_select(0, plan.order) % self.per_rank).to(torch.int32)
        got_rows = self._exchange(send_rows, plan.send, plan.recv)
        got_ids = self._exchange(send_ids, plan.send, plan.recv)
        y_remote = be.run_experts(got_rows, got_ids)                       # [n_recv, D] fp32, one row a pair
        y_sorted = self._exchange(y_remote, plan.recv, plan.send)          # back in this rank's sorted-pair order
        y = torch.empty((rows, slots, dims), dtype=y_sorted.dtype, device=x.device)
        y_routed = torch.empty((rows * k, dims), dtype=y_sorted.dtype, device=x.device)
        y_routed.index_copy_(0, plan.order, y_sorted)
        y[:, :k] = y_routed.view(rows, k, dims)
        if self.shared:
            y[:, k] = be.run_shared(x)
        return be.combine(y.contiguous(), wts.contiguous())


class GatheredExpertParallel:
    """The same sharding without any host read, so the whole step can sit in a CUDA graph: every rank gathers all
    ranks' tokens (a few hundred KB), routes them all (identical bits everywhere), runs the pairs that fall on ITS
    experts into a zeroed per-pair buffer ``y_all`` [T_global * k, D] fp32, and one reduce-scatter hands each home rank
    its tokens' rows.  Every (token, slot) row is non-zero on exactly one rank, so the sum over ranks is exact and the
    home rank's slot-order combine gives the one-GPU bits.  Costs more link traffic than the counted all-to-all
    (``ExpertParallel``) and no latency of a host round trip; NCCL may reduce inside the switch (NVLS)."""

    def __init__(self, router_rows: torch.Tensor, local_experts, experts: int, top_k: int, rows_local: int,
                 group=None, reduce: str = "rows") -> None:
        """``reduce="rows"``: the per-pair fp32 rows travel (exact: the one-GPU bits).  ``reduce="tokens"``: every rank
        first sums ITS pairs of each token in slot order (weights applied) and the reduce-scatter adds the ranks'
        partial sums - k times less link traffic, the same values up to fp32 summation order across ranks."""

        from . import experts as grouped
        from . import moe

        if reduce not in ("rows", "tokens"):
            raise ValueError("reduce must be 'rows' or 'tokens'")
        self.reduce = reduce
        self.moe, self.grouped = moe, grouped
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if experts % self.world:
            raise ValueError(f"{experts} experts do not shard evenly over {self.world} ranks")
        self.per_rank, self.experts, self.top_k = experts // self.world, experts, top_k
        self.router_rows, self.local, self.rows_local = router_rows, local_experts, rows_local
        dev, d, k = router_rows.device, local_experts.dims, top_k
        rows = rows_local * self.world
        self.rows = rows

        class _Cfg:
            num_experts_per_tok, num_experts = top_k, experts
            moe_intermediate_size, hidden_size = local_experts.width, d

        self.x_all = torch.zeros((rows, d), dtype=torch.bfloat16, device=dev)
        self.buf = moe.MoEBuffers(rows, _Cfg, dev, shared=False)
        # about rows * k / experts pairs reach each local expert: from 24 on, items of 16 (one dequantisation for two
        # mma tiles) beat two passes of items of 8; below that the leaner 8-pair kernel wins (measured at 8, 16 and 32)
        wide = rows * k >= 24 * experts
        self.plan = grouped.Plan(rows, k, self.per_rank, dev, decode_tile=grouped.WIDE_TILE if wide else grouped.TILE)
        self.local_pick = torch.zeros((rows, k), dtype=torch.int32, device=dev)
        self.y_mine = torch.zeros((rows_local * k, d), dtype=torch.float32, device=dev)
        self.partial = torch.zeros((rows, d), dtype=torch.float32, device=dev)
        self.partial_mine = torch.zeros((rows_local, d), dtype=torch.float32, device=dev)
        self.out = torch.zeros((rows_local, d), dtype=torch.bfloat16, device=dev)
        self._fused_rows = moe.fused_select_rows()
        self.launches = 5 if rows <= self._fused_rows else 6

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        m, g, buf, k = self.moe, self.grouped, self.buf, self.top_k
        if self.world > 1:
            dist.all_gather_into_tensor(self.x_all, x_local.contiguous(), group=self.group)
        else:
            self.x_all.copy_(x_local)
        m.router(self.x_all, self.router_rows, buf.logits)
        lo, st = self.rank * self.per_rank, torch.cuda.current_stream(self.x_all.device).cuda_stream
        plan = self.plan
        plan.tile = plan.decode_tile
        with torch.cuda.device(self.x_all.device):
            if self.rows <= self._fused_rows:
                # selection of every token and the plan of this rank's experts in one launch
                _lib.call("tfb_select_plan_window", buf.logits.data_ptr(), buf.logits.shape[1], buf.pick.data_ptr(),
                          buf.wts.data_ptr(), self.rows, self.experts, k, 0, plan.tile, lo, self.per_rank,
                          plan.members.data_ptr(), plan.items.data_ptr(), plan.counts.data_ptr(), st)
            else:
                m.select_rows(buf.logits, buf, k, self.experts)
                _lib.call("tfb_plan_window", buf.pick.data_ptr(), self.rows * k, lo, self.per_rank, plan.tile,
                          plan.members.data_ptr(), plan.items.data_ptr(), plan.counts.data_ptr(), st)
        y_all = buf.y.view(-1, self.local.dims)
        if self.reduce == "rows":
            y_all.zero_()
        g.gate_up(self.x_all, self.local, plan, buf.act.view(-1, self.local.width), self.rows)
        g.down(buf.act.view(-1, self.local.width), self.local, plan, y_all, self.rows)
        if self.reduce == "tokens":
            # this rank's pairs of every token, weights applied, in slot order; other ranks' rows are never read
            with torch.cuda.device(self.x_all.device):
                _lib.call("tfb_combine_window", buf.y.data_ptr(), 0, buf.wts.data_ptr(), buf.pick.data_ptr(), lo,
                          self.per_rank, self.partial.data_ptr(), 1, self.rows, k, self.local.dims, st)
            if self.world > 1:
                dist.reduce_scatter_tensor(self.partial_mine, self.partial, group=self.group)
            else:
                self.partial_mine.copy_(self.partial[:self.rows_local])
            self.out.copy_(self.partial_mine)                     # one rounding to bf16
            return self.out
        if self.world > 1:
            dist.reduce_scatter_tensor(self.y_mine, y_all, group=self.group)
        else:
            self.y_mine.copy_(y_all)
        lo = self.rank * self.rows_local
        wts = buf.wts[lo:lo + self.rows_local]
        return m.combine(self.y_mine.view(self.rows_local, k, -1), wts, self.out)


class PeerWindow:
    """One rank's window of an expert-parallel layer over NVLink peer memory, and the steps every such layer shares
    (``csrc/peer.cu``): routing of the rank's own rows into the window, the pull of all ranks' rows and selections
    after the tokens barrier, and the sum of the ranks' partial results after the results barrier.

    The windows are one ``torch.distributed._symmetric_memory`` allocation a rank (plain peer mappings; multicast is
    not used).  Waits are bounded (``_lib.set_wait_limit_ms``): when a rank never arrives the status word names the
    barrier and that rank, the step's kernels leave the peers' memory alone, and the step's output is void - read
    ``_lib.kernel_status()`` (or ``_lib.check_status()``) after a step before using its output."""

    def __init__(self, router_rows: torch.Tensor, experts: int, top_k: int, rows_local: int, dims: int, shared: bool,
                 group=None, logit_bias: torch.Tensor | None = None, rows_active: int | None = None) -> None:
        """``rows_active`` (default ``rows_local``): how many of this rank's rows hold tokens.  Every rank's window has
        ``rows_local`` rows; a batch smaller than the rank count (one token on eight GPUs) leaves some ranks with
        none.  The other rows are never routed: their slots carry an id no rank owns, so no expert runs for them."""

        import ctypes
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if experts % self.world:
            raise ValueError(f"{experts} experts do not shard evenly over {self.world} ranks")
        if router_rows.shape[0] != experts + (1 if shared else 0):
            raise ValueError("router rows: one an expert, plus the shared expert's gate row when there is one")
        self.per_rank, self.experts, self.top_k, self.shared = experts // self.world, experts, top_k, shared
        self.lo = self.rank * self.per_rank
        self.router_rows, self.rows_local, self.dims = router_rows, rows_local, dims
        self.logit_bias = logit_bias                              # [experts] fp32 added to the routed logits, or None
        self.slots = slots = top_k + (1 if shared else 0)
        self.rows_active = rows_local if rows_active is None else int(rows_active)
        if not 0 <= self.rows_active <= rows_local:
            raise ValueError(f"rows_active must lie in 0..{rows_local}")
        dev, d = router_rows.device, dims
        self.device = dev
        self.rows = rows = rows_local * self.world

        def up(n: int) -> int:
            return (n + 255) // 256 * 256

        x_bytes, s_bytes = rows_local * d * 2, rows_local * slots * 4
        if x_bytes % 16 or s_bytes % 16 or 2 * self.world * 4 > 256:
            raise ValueError("rows_local * dims must be a multiple of 8, rows_local * slots of 4, and at most 32 ranks")
        self.x_offset = 256
        self.pick_offset = self.x_offset + up(x_bytes)
        self.wts_offset = self.pick_offset + up(s_bytes)
        self.p_offset = self.wts_offset + up(s_bytes)
        self.x_bytes = x_bytes
        self.window = win = symm.empty(self.p_offset + rows * d * 4, dtype=torch.uint8, device=dev)
        win.zero_()
        torch.cuda.synchronize(dev)
        self.handle = symm.rendezvous(win, self.group)
        self.windows = torch.tensor(list(self.handle.buffer_ptrs), dtype=torch.int64, device=dev)
        self.step = torch.zeros(1, dtype=torch.int32, device=dev)
        # this rank's rows inside its window: a caller may write them here and run the layer without an argument
        self.tokens = win[self.x_offset:self.x_offset + x_bytes].view(torch.bfloat16).view(rows_local, d)
        self.pick_mine = win[self.pick_offset:self.pick_offset + s_bytes].view(torch.int32).view(rows_local, slots)
        self.wts_mine = win[self.wts_offset:self.wts_offset + s_bytes].view(torch.float32).view(rows_local, slots)
        self.pick_mine[self.rows_active:] = experts + 1           # rows without a token: an id outside every window
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)                                  # every window is zeroed before any flag is written
        self.logits = torch.zeros((rows_local, router_rows.shape[0]), dtype=torch.float32, device=dev)
        self.x_all = torch.zeros((rows, d), dtype=torch.bfloat16, device=dev)
        self.pick_all = torch.zeros((rows, slots), dtype=torch.int32, device=dev)
        self.wts_all = torch.zeros((rows, slots), dtype=torch.float32, device=dev)
        self._seg = (
            (ctypes.c_int64 * 3)(self.x_offset, self.pick_offset, self.wts_offset),
            (ctypes.c_int64 * 3)(x_bytes, s_bytes, s_bytes),
            (ctypes.c_void_p * 3)(self.x_all.data_ptr(), self.pick_all.data_ptr(), self.wts_all.data_ptr()),
        )

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def route_own(self, x_local: torch.Tensor | None) -> None:
        """Stage ``x_local`` (unless the caller wrote ``tokens`` itself), then router and selection of the own rows."""

        from . import moe

        st = self._stream()
        if x_local is not None:
            if tuple(x_local.shape) != tuple(self.tokens.shape) or x_local.dtype != torch.bfloat16:
                raise ValueError("x_local must be bf16 [rows_local, D]")
            if not x_local.is_cuda and not x_local.is_pinned():
                raise ValueError("host rows must be in pinned memory (a kernel reads them)")
            x_local = x_local.contiguous()
            _lib.call("tfb_peer_stage", x_local.data_ptr(), self.window.data_ptr(), self.x_offset, self.x_bytes, st)
        n = self.rows_active
        if n == 0:
            return
        moe.router(self.tokens[:n], self.router_rows, self.logits[:n])
        if self.logit_bias is not None:
            self.logits[:n, :self.experts].add_(self.logit_bias)
        _lib.call("tfb_select_rows", self.logits.data_ptr(), self.logits.shape[1], self.pick_mine.data_ptr(),
                  self.wts_mine.data_ptr(), n, self.experts, self.top_k, 1 if self.shared else 0, st)

    def gather(self) -> None:
        """Tokens barrier, then all ranks' rows and selections into ``x_all``, ``pick_all``, ``wts_all``."""

        _lib.call("tfb_peer_gather", self.windows.data_ptr(), self.rank, self.world, 3, self._seg[0], self._seg[1],
                  self._seg[2], self.step.data_ptr(), self._stream())

    def push(self, partial: torch.Tensor) -> None:
        """partial [rows, D] fp32 (this rank's experts' share of every token) to the tokens' home ranks."""

        _lib.call("tfb_peer_push", partial.data_ptr(), self.windows.data_ptr(), self.p_offset, self.rank,
                  self.rows_local, self.rows, self.dims, self.step.data_ptr(), self._stream())

    def sum(self, out: torch.Tensor, extra: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> None:
        """Results barrier, then out [rows_local, D] (bf16 or fp32) = the ranks' shares in rank order (+ the shared
        expert's rows ``extra`` weighted by the own rows' last slot, + the ``residual`` rows, bf16)."""

        ew = self.wts_mine.data_ptr() + 4 * self.top_k if extra is not None else 0
        if residual is not None and (residual.dtype != torch.bfloat16 or not residual.is_contiguous()
                                     or tuple(residual.shape) != (self.rows_local, self.dims)):
            raise ValueError("the residual rows are contiguous bf16 [rows_local, D]")
        _lib.call("tfb_peer_sum", self.windows.data_ptr(), self.rank, self.p_offset, self.world, self.rows_local,
                  self.dims, out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                  extra.data_ptr() if extra is not None else 0, ew, self.slots,
                  residual.data_ptr() if residual is not None else 0, self.step.data_ptr(), self._stream())


class PeerExpertParallel:
    """The expert-parallel step of the affine 4-bit experts with both exchanges done by this library's own kernels over
    NVLink peer memory (``PeerWindow``): no collective-library call on the step.  Every rank routes ITS rows (router
    and selection, as on one GPU) with the selections written into its window beside the rows; a flag barrier; every
    rank pulls all ranks' rows and selections, plans the pairs of its experts and runs them; the per-token partial sums
    of a rank's experts (slot order, weights applied) are stored straight into the home rank's window by the kernel that
    forms them; a second flag barrier; the home rank adds the ranks' rows in rank order and rounds once.  A shared
    expert (``shared_experts``: an ``Experts`` of one expert, replicated; the router's last row is its gate) runs on
    the rank's own rows with no exchange and joins the final sum.  Values equal
    ``GatheredExpertParallel(reduce="tokens")`` up to fp32 summation order across ranks (here fixed: rank 0, 1, ...)."""

    def __init__(self, router_rows: torch.Tensor, local_experts, experts: int, top_k: int, rows_local: int,
                 group=None, shared_experts=None, logit_bias: torch.Tensor | None = None, hot_pairs: int = 0,
                 rows_active: int | None = None) -> None:
        """``hot_pairs`` > 0: a rank's experts with at least that many pairs run through the prompt-form kernel (one
        pass over the expert's weights for up to 192 pairs) instead of one decode item per 8 pairs - for skewed
        routing, where one rank's busiest experts otherwise set the step time.  Those pairs then carry the prompt
        form's arithmetic (weights rounded once to bf16), so a token's bits depend on its experts' load."""

        from . import experts as grouped
        from . import moe

        self.moe, self.grouped = moe, grouped
        shared = shared_experts is not None
        self.win = w = PeerWindow(router_rows, experts, top_k, rows_local, local_experts.dims, shared, group,
                                  logit_bias, rows_active)
        self.local, self.shared_ex, self.rows_local, self.top_k = local_experts, shared_experts, rows_local, top_k
        self.world, self.rank, self.rows, self.tokens = w.world, w.rank, w.rows, w.tokens
        dev, d, rows, slots = w.device, w.dims, w.rows, w.slots
        self.act = torch.zeros((rows * slots, local_experts.width), dtype=torch.bfloat16, device=dev)
        self.y = torch.zeros((rows * slots, d), dtype=torch.float32, device=dev)
        wide = rows * top_k >= 24 * experts
        self.plan = grouped.Plan(rows, slots, w.per_rank, dev,
                                 decode_tile=grouped.WIDE_TILE if wide else grouped.TILE, hot=hot_pairs)
        self.out = torch.zeros((rows_local, d), dtype=torch.bfloat16, device=dev)
        self.launches = 8 + (2 if hot_pairs else 0)               # + 1 when forward() is given rows to stage
        if shared:
            if shared_experts.count != 1 or shared_experts.dims != d:
                raise ValueError("shared_experts holds the one replicated expert of the layer's width")
            # every own row is one pair of expert 0: the plan never changes
            wide_s = rows_local >= 12
            self.plan_s = grouped.Plan(rows_local, 1, 1, dev, decode_tile=grouped.WIDE_TILE if wide_s else grouped.TILE)
            grouped.route(torch.zeros((rows_local, 1), dtype=torch.int32, device=dev), self.plan_s)
            self.act_s = torch.zeros((rows_local, shared_experts.width), dtype=torch.bfloat16, device=dev)
            self.y_s = torch.zeros((rows_local, d), dtype=torch.float32, device=dev)
            self.launches += 2
            # the shared expert needs nothing from the exchange and is needed only by the final sum: its two launches
            # run on a stream of their own beside the gather, the plan and the routed experts
            self.side_s = torch.cuda.Stream(dev)
            self.forked_s, self.joined_s = torch.cuda.Event(), torch.cuda.Event()
            torch.cuda.synchronize(dev)

    def forward(self, x_local: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """``x_local`` [rows_local, D] bf16 (device memory, or pinned host memory that the staging kernel reads over
        PCIe), or None when the caller has written its rows into ``self.tokens``.  ``out`` [rows_local, D] bf16:
        where the last kernel stores the result (device or pinned host memory); default ``self.out``."""

        g, w, k, d = self.grouped, self.win, self.top_k, self.win.dims
        out = self.out if out is None else out
        if tuple(out.shape) != tuple(self.out.shape) or out.dtype != self.out.dtype or not out.is_contiguous():
            raise ValueError("out must be contiguous bf16 [rows_local, D]")
        if not out.is_cuda and not out.is_pinned():
            raise ValueError("a host result buffer must be pinned memory (a kernel stores into it)")
        plan = self.plan
        plan.tile = plan.decode_tile
        with torch.cuda.device(w.device):
            st = w._stream()
            w.route_own(x_local)
            if self.shared_ex is not None:                         # own rows only; beside everything up to the sum
                cur = torch.cuda.current_stream(w.device)
                self.forked_s.record(cur)
                self.side_s.wait_event(self.forked_s)
                with torch.cuda.stream(self.side_s):
                    g.gate_up(w.tokens, self.shared_ex, self.plan_s, self.act_s, self.rows_local)
                    g.down(self.act_s, self.shared_ex, self.plan_s, self.y_s, self.rows_local)
                self.joined_s.record(self.side_s)
            w.gather()
            if plan.hot:
                g.route_split(w.pick_all, plan, w.lo)
            else:
                _lib.call("tfb_plan_window", w.pick_all.data_ptr(), self.rows * w.slots, w.lo, w.per_rank, plan.tile,
                          plan.members.data_ptr(), plan.items.data_ptr(), plan.counts.data_ptr(), st)
            g.gate_up(w.x_all, self.local, plan, self.act, self.rows)
            g.down(self.act, self.local, plan, self.y, self.rows)
            _lib.call("tfb_combine_push", self.y.data_ptr(), w.wts_all.data_ptr(), w.pick_all.data_ptr(), w.lo,
                      w.per_rank, w.windows.data_ptr(), w.p_offset, w.rank, self.rows_local, self.rows, w.slots, d,
                      w.step.data_ptr(), st)
            if self.shared_ex is not None:
                torch.cuda.current_stream(w.device).wait_event(self.joined_s)
            w.sum(out, self.y_s if self.shared_ex is not None else None)
        return out


class PeerExl3ExpertParallel:
    """The same step for EXL3 routed experts (``exl3.experts.routed`` on the rank's experts): selections are renumbered
    to the rank's window (other ranks' slots become skipped ids with weight 0), the routed call forms the rank's
    weighted slot-order share of every token, which is pushed to the home ranks; the sum is fp32 like the one-GPU
    call's output."""

    def __init__(self, router_rows: torch.Tensor, local_ex, experts: int, top_k: int, rows_local: int, group=None,
                 limit: float = float("inf"), rows_active: int | None = None) -> None:
        from .exl3 import experts as exl3

        self.exl3 = exl3
        self.win = w = PeerWindow(router_rows, experts, top_k, rows_local, local_ex.dims, False, group,
                                  rows_active=rows_active)
        self.local, self.rows_local, self.top_k, self.limit = local_ex, rows_local, top_k, limit
        self.world, self.rank, self.rows, self.tokens = w.world, w.rank, w.rows, w.tokens
        dev, d, rows = w.device, w.dims, w.rows
        self.scratch = exl3.Scratch(local_ex, rows, top_k, device=dev)
        self.scratch.y.zero_()                                     # skipped slots are read with weight 0: keep them finite
        self.pick_local = torch.zeros((rows, top_k), dtype=torch.int32, device=dev)
        self.wts_local = torch.zeros((rows, top_k), dtype=torch.float32, device=dev)
        self.partial = torch.zeros((rows, d), dtype=torch.float32, device=dev)
        self.out = torch.zeros((rows_local, d), dtype=torch.float32, device=dev)
        self.out_next = torch.zeros((rows_local, d), dtype=torch.bfloat16, device=dev)
        self.launches = 7 + exl3.LAUNCHES_PER_CALL               # + 1 when forward() is given rows to stage
        torch.cuda.synchronize(dev)

    def forward(self, x_local: torch.Tensor | None = None, residual: bool = False) -> torch.Tensor:
        """The layer's output [rows_local, D] fp32; with ``residual`` the next hidden state bf16(h + layer(h)) instead
        (h = the rank's rows as staged in the window), formed by the kernel that adds the ranks' shares."""

        w = self.win
        with torch.cuda.device(w.device):
            w.route_own(x_local)
            w.gather()
            _lib.call("tfb_window_picks", w.pick_all.data_ptr(), w.wts_all.data_ptr(), w.lo, w.per_rank,
                      self.pick_local.data_ptr(), self.wts_local.data_ptr(), self.rows * self.top_k, w._stream())
            self.exl3.routed(w.x_all, self.pick_local, self.wts_local, self.local, self.scratch, self.partial,
                             self.rows, limit=self.limit, share=w.per_rank / w.experts)
            w.push(self.partial)
            if residual:
                w.sum(self.out_next, residual=w.tokens)
                return self.out_next
            w.sum(self.out)
        return self.out
