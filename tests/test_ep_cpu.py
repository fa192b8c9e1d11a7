"""Expert parallelism's host logic on two CPU ranks (gloo): dispatch, owner-side compute, return and slot-order
combine give every token the single-rank result, bit for bit, for even and skewed routing."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


class FakeBackend:
    """A stand-in for the GPU arithmetic: experts are random dense maps, routing a fixed seeded rule."""

    def __init__(self, experts, top_k, dims, first, count, shared, skew):
        g = torch.Generator().manual_seed(7)
        self.w = torch.randn((experts + 1, dims, dims), generator=g) * 0.1     # every rank can build all; uses its own
        self.router = torch.randn((experts + 1, dims), generator=g)
        self.first, self.count, self.top_k, self.experts, self.shared, self.skew = first, count, top_k, experts, shared, skew

    def route(self, x):
        logits = x.float() @ self.router.t()
        if self.skew:
            logits[:, : self.experts] += -1.1 * torch.log(torch.arange(1, self.experts + 1).float())
        top = torch.topk(logits[:, : self.experts], self.top_k, dim=1)
        wts = torch.softmax(top.values, dim=1)
        pick = top.indices.to(torch.int32)
        if self.shared:
            pick = torch.cat([pick, torch.full((x.shape[0], 1), self.experts, dtype=torch.int32)], 1)
            wts = torch.cat([wts, torch.sigmoid(logits[:, self.experts:])], 1)
        return pick, wts.float()

    def run_experts(self, rows, local_ids):
        assert ((local_ids >= 0) & (local_ids < self.count)).all()
        w = self.w[self.first + local_ids.long()]
        return torch.einsum("nd,nde->ne", rows.float(), w)

    def run_shared(self, x):
        return x.float() @ self.w[self.experts]

    def combine(self, y, wts):
        acc = torch.zeros((y.shape[0], y.shape[2]))
        for s in range(y.shape[1]):
            acc = acc + wts[:, s:s + 1] * y[:, s]
        return acc.to(torch.bfloat16)


def _worker(rank, world, port, shared, skew, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tensorfold_b200.ep import ExpertParallel

    experts, top_k, dims, rows = 8, 3, 16, 11
    g = torch.Generator().manual_seed(100)
    x_all = torch.randn((world * rows, dims), generator=g).to(torch.bfloat16)
    per = experts // world
    ep = ExpertParallel(FakeBackend(experts, top_k, dims, rank * per, per, shared, skew), experts, top_k, shared)
    got = ep.forward(x_all[rank * rows:(rank + 1) * rows])
    solo = ExpertParallel.__new__(ExpertParallel)                  # the same layer on one rank holding every expert
    solo.backend = FakeBackend(experts, top_k, dims, 0, experts, shared, skew)
    solo.experts, solo.top_k, solo.shared, solo.group, solo.world, solo.rank, solo.per_rank = \
        experts, top_k, shared, None, 1, 0, experts
    want = solo.forward(x_all[rank * rows:(rank + 1) * rows])
    ok = torch.equal(got, want) and sum(ep.last_plan.send) == rows * top_k
    out.put((rank, bool(ok), ep.last_plan.send))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("shared,skew", [(False, False), (True, True)])
def test_two_ranks_match_one(shared, skew):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, shared, skew, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    if skew:                                                       # skewed routing loads rank 0's experts more
        sends = {r: s for r, _, s in results}
        assert sends[0][0] > sends[0][1]
