"""Router, selection, plan and combine on the GPU against the CPU oracle: indices and sort order bit for bit."""

import numpy as np
import pytest
import torch

from helpers import bits

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _logits(t, ne, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn((t, ne), generator=g)


@pytest.mark.parametrize("t,d,ne", [(1, 2048, 128), (5, 768, 13), (64, 2048, 129), (300, 256, 50), (17, 6144, 257)])
def test_router_logits_bit_exact(t, d, ne):
    from oracle import cpu
    from tensorfold_b200 import moe

    g = torch.Generator().manual_seed(t + d)
    x = torch.randn((t, d), generator=g).to(torch.bfloat16)
    w = (torch.randn((ne, d), generator=g) * 0.02).to(torch.bfloat16)
    got = moe.router(x.to(DEV), w.to(DEV)).cpu().numpy()
    assert np.array_equal(got, cpu.router_logits(bits(x), bits(w)))


@pytest.mark.parametrize("t,d,ne", [(1, 2048, 128), (300, 256, 50), (17, 6144, 257), (2048, 2048, 129), (70, 96, 9)])
def test_prompt_router_on_the_tensor_cores(t, d, ne):
    """The prompt form's router: the fp32-fma router's logits up to summation order (1e-5 of the largest), the same
    top-8 wherever the eighth and ninth logits are further apart than that, and a row's bits independent of the rows
    it is computed with."""

    from tensorfold_b200 import moe

    g = torch.Generator().manual_seed(700 + t)
    x = torch.randn((t, d), generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((ne, d), generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    want = moe.router(x, w)
    got = moe.router(x, w, prompt=True)
    tol = 1e-5 * float(want.abs().max())
    assert float((got - want).abs().max()) <= tol
    k = min(8, ne - 1)
    a, b = got.cpu().numpy(), want.cpu().numpy()
    for r in range(0, t, max(1, t // 40)):
        order = sorted(range(ne), key=lambda i: (-b[r, i], i))
        if b[r, order[k - 1]] - b[r, order[k]] > 4 * tol:
            assert sorted(range(ne), key=lambda i: (-a[r, i], i))[:k] == order[:k]
    for lo, hi in ((0, 1), (t // 2, t // 2 + 1), (max(0, t - 19), t)):
        assert torch.equal(moe.router(x[lo:hi], w, prompt=True), got[lo:hi])


def test_router_rows_do_not_depend_on_the_window():
    from tensorfold_b200 import moe

    g = torch.Generator().manual_seed(3)
    x = torch.randn((40, 512), generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((33, 512), generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    full = moe.router(x, w)
    for a, b in ((0, 1), (7, 8), (3, 20), (39, 40)):
        assert torch.equal(moe.router(x[a:b], w), full[a:b])
    wide = torch.zeros((40, 1024), dtype=torch.bfloat16, device=DEV)          # strided rows
    wide[:, :512] = x
    assert torch.equal(moe.router(wide[:, :512], w), full)


class _Cfg:
    def __init__(self, e, k, ni=64, d=64):
        self.num_experts, self.num_experts_per_tok, self.moe_intermediate_size, self.hidden_size = e, k, ni, d


@pytest.mark.parametrize("t,e,k,shared", [(1, 128, 8, False), (64, 128, 8, False), (40, 64, 10, True),
                                         (33, 256, 8, True), (9, 160, 8, False), (20, 1000, 6, True), (7, 5, 5, False)])
def test_select_rows_against_the_oracle(t, e, k, shared):
    from oracle import cpu
    from tensorfold_b200 import moe

    logits = _logits(t, e + (1 if shared else 0), 100 + t + e)
    logits[0, :] = 0.0
    if t > 2:
        logits[2, : min(e, 12)] = 1.25
    buf = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=shared)
    moe.select_rows(logits.to(DEV), buf, k, e)
    pick, wts = buf.pick.cpu().numpy(), buf.wts.cpu().numpy()
    want_pick, want_wts = cpu.topk_rows(logits.numpy(), e, k, shared)
    assert np.array_equal(pick, want_pick)                                     # indices: bit exact
    ln = logits.numpy()
    for r in range(t):
        assert pick[r, :k].tolist() == sorted(range(e), key=lambda i: (-ln[r, i], i))[:k]
    assert pick[0, :k].tolist() == list(range(k))                              # ties go to the lower id
    # weights: bf16 values within one bf16 ulp of the oracle's (exp's last bits are not pinned by the reference)
    assert np.array_equal(wts.view(np.uint32) & 0xFFFF, np.zeros_like(wts, dtype=np.uint32))
    ulp = np.maximum(np.abs(want_wts), 2.0 ** -126) * 2.0 ** -7
    assert (np.abs(wts - want_wts) <= ulp).all()


def want_plan(picks, e, tile):
    flat = picks.reshape(-1).tolist()
    items, members = [], []
    for ex in range(e):
        pairs = [p for p, v in enumerate(flat) if v == ex]
        for j in range(0, len(pairs), tile):
            items.append([ex, len(members) + j, min(tile, len(pairs) - j)])
        members += pairs
    return items, members, len(set(flat))


@pytest.mark.parametrize("rows,prefill,tile", [(23, False, 64), (23, True, 64), (300, False, 64), (300, True, 64),
                                              (1500, True, 64), (1500, True, 16), (1, False, 64), (4000, True, 64)])
def test_plan_groups_pairs_by_expert(rows, prefill, tile):
    """The reference's plan golden (tests/cuda/test_experts.py:118-134): 7 slots, 50 experts, one expert in every row."""

    from tensorfold_b200 import experts

    slots, e = 7, 50
    g = torch.Generator().manual_seed(9)
    picks = torch.stack([torch.randperm(e, generator=g)[:slots] for _ in range(rows)]).to(torch.int32)
    picks[:, 0] = 3
    plan = experts.Plan(rows, slots, e, DEV, prefill=prefill)
    experts.route(picks.to(DEV), plan, tile)
    assert plan.tile == (tile if prefill else experts.TILE)
    want_items, want_members, distinct = want_plan(picks, e, plan.tile)
    n = int(plan.counts[0])
    assert n == len(want_items) and int(plan.counts[1]) == distinct
    assert plan.items[:n].tolist() == want_items
    assert plan.members.tolist() == want_members


def test_plan_with_many_experts_and_skipped_ids():
    from oracle import cpu
    from tensorfold_b200 import experts

    g = torch.Generator().manual_seed(4)
    e, rows, slots = 1024, 700, 9
    picks = torch.randint(0, e + 3, (rows, slots), generator=g).to(torch.int32)     # ids >= e are left out
    plan = experts.Plan(rows, slots, e, DEV)
    experts.route(picks.to(DEV), plan)
    items, members, counts = cpu.plan(picks.numpy(), e, experts.TILE)
    n = int(plan.counts[0])
    assert n == len(items) and plan.counts.tolist() == counts.tolist()
    assert np.array_equal(plan.items[:n].cpu().numpy(), items)
    assert np.array_equal(plan.members[:len(members)].cpu().numpy(), members)


@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
def test_combine_slot_order_fma_chain(ydtype):
    from tensorfold_b200 import moe

    g = torch.Generator().manual_seed(8)
    t, s, d = 19, 9, 2048
    y = torch.randn((t, s, d), generator=g).to(ydtype)
    w = torch.rand((t, s), generator=g).to(torch.bfloat16).float()
    got = moe.combine(y.to(DEV), w.to(DEV)).cpu()
    acc = np.zeros((t, d), dtype=np.float64)
    yf, wf = y.float().numpy().astype(np.float64), w.numpy().astype(np.float64)
    acc32 = np.zeros((t, d), dtype=np.float32)
    for k in range(s):
        acc32 = (wf[:, k:k + 1] * yf[:, k] + acc32.astype(np.float64)).astype(np.float32)   # fma: one rounding a step
    want = torch.from_numpy(acc32).to(torch.bfloat16)
    assert (got.view(torch.int16) != want.view(torch.int16)).float().mean() < 1e-4          # double-rounding slack only
    assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-6)
    out32 = torch.empty((t, d), dtype=torch.float32, device=DEV)
    moe.combine(y.to(DEV), w.to(DEV), out32)
    assert np.abs(out32.cpu().numpy() - acc32).max() <= 1e-6 * np.abs(acc32).max()


@pytest.mark.parametrize("t,e,k,shared", [(1, 128, 8, False), (64, 128, 8, False), (100, 256, 8, True), (128, 1000, 6, True)])
def test_fused_select_plan_equals_the_two_kernels(t, e, k, shared):
    from tensorfold_b200 import experts, moe

    logits = _logits(t, e + (1 if shared else 0), 200 + t).to(DEV)
    a = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=shared)
    b = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=shared)
    moe.select(logits, a, k, e)                                               # one launch
    moe.select_rows(logits, b, k, e)
    experts.route(b.pick[:t], b.plan)
    assert torch.equal(a.pick, b.pick) and torch.equal(a.wts, b.wts)
    n = int(b.plan.counts[0])
    assert torch.equal(a.plan.counts, b.plan.counts) and torch.equal(a.plan.items[:n], b.plan.items[:n])
    assert torch.equal(a.plan.members, b.plan.members)


@pytest.mark.parametrize("t,d,e,k,shared", [(1, 2048, 128, 8, False), (5, 768, 13, 4, True), (8, 256, 50, 7, False),
                                            (9, 2048, 128, 8, False), (64, 2048, 128, 8, False),
                                            (33, 6144, 256, 8, True), (3, 512, 1000, 6, True)])
def test_one_launch_routing_equals_the_three_kernels(t, d, e, k, shared, pdl):
    """``moe.route`` (router, selection and plan finished by whichever block comes last) against ``router``,
    ``select_rows`` and ``route`` as separate launches: logits, picks, weights and the plan bit for bit, on two calls
    in a row (the arrival counters return to zero) with different rows."""

    from tensorfold_b200 import experts, moe

    ne = e + (1 if shared else 0)
    g = torch.Generator().manual_seed(500 + t)
    rows_w = (torch.randn((ne, d), generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    a = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=shared)
    b = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=shared)
    assert t <= moe.route_rows(rows_w)
    for call in range(2):
        x = torch.randn((t, d), generator=g).to(torch.bfloat16).to(DEV)
        moe.route(x, rows_w, a, k, e)                                           # one launch
        moe.router(x, rows_w, b.logits[:t])
        moe.select_rows(b.logits[:t], b, k, e)
        experts.route(b.pick[:t], b.plan)
        torch.cuda.synchronize()
        assert torch.equal(a.logits[:t], b.logits[:t]), call
        assert torch.equal(a.pick[:t], b.pick[:t]) and torch.equal(a.wts[:t], b.wts[:t]), call
        n = int(b.plan.counts[0])
        assert torch.equal(a.plan.counts, b.plan.counts) and torch.equal(a.plan.items[:n], b.plan.items[:n])
        assert torch.equal(a.plan.members[:t * a.slots], b.plan.members[:t * a.slots])
        assert int(a.arrive_route.abs().sum()) == 0
    with pytest.raises(ValueError):
        moe.route(torch.zeros((moe.route_rows(rows_w) + 1, d), dtype=torch.bfloat16, device=DEV), rows_w,
                  moe.MoEBuffers(moe.route_rows(rows_w) + 1, _Cfg(e, k), DEV, shared=shared), k, e)


def test_windowed_plan_and_combine():
    """The expert-parallel forms: a plan of the ids in [lo, lo + n) renumbered from 0, selection + that plan in one
    launch, and a combine over those slots only."""

    import ctypes

    from oracle import cpu
    from tensorfold_b200 import _lib, experts, moe

    t, e, k, lo, n = 96, 128, 8, 32, 48
    logits = _logits(t, e, 77).to(DEV)
    buf = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=False)
    moe.select_rows(logits, buf, k, e)
    stream = torch.cuda.current_stream().cuda_stream
    plan = experts.Plan(t, k, n, DEV)
    _lib.call("tfb_plan_window", buf.pick.data_ptr(), t * k, lo, n, experts.TILE, plan.members.data_ptr(),
              plan.items.data_ptr(), plan.counts.data_ptr(), stream)
    items, members, counts = cpu.plan(buf.pick.cpu().numpy() - lo, n, experts.TILE)
    cnt = int(plan.counts[0])
    assert plan.counts.tolist() == counts.tolist()
    assert np.array_equal(plan.items[:cnt].cpu().numpy(), items)
    assert np.array_equal(plan.members[:len(members)].cpu().numpy(), members)
    buf2 = moe.MoEBuffers(t, _Cfg(e, k), DEV, shared=False)
    plan2 = experts.Plan(t, k, n, DEV)
    _lib.call("tfb_select_plan_window", logits.data_ptr(), e, buf2.pick.data_ptr(), buf2.wts.data_ptr(), t, e, k, 0,
              experts.TILE, lo, n, plan2.members.data_ptr(), plan2.items.data_ptr(), plan2.counts.data_ptr(), stream)
    assert torch.equal(buf2.pick, buf.pick) and torch.equal(buf2.wts, buf.wts)
    assert torch.equal(plan2.counts, plan.counts) and torch.equal(plan2.items[:cnt], plan.items[:cnt])
    assert torch.equal(plan2.members[:len(members)], plan.members[:len(members)])
    d = 256
    y = torch.randn((t, k, d), device=DEV)
    out = torch.empty((t, d), dtype=torch.float32, device=DEV)
    _lib.call("tfb_combine_window", y.data_ptr(), 0, buf.wts.data_ptr(), buf.pick.data_ptr(), lo, n, out.data_ptr(), 1,
              t, k, d, stream)
    mask = ((buf.pick >= lo) & (buf.pick < lo + n)).float()
    want = moe.combine(y * mask[..., None], buf.wts, torch.empty_like(out))     # zeroed rows add exactly nothing
    assert torch.equal(out, want)


@pytest.mark.parametrize("experts,top_k,shared,norm", [(64, 6, 1, True), (256, 8, 1, True), (160, 6, 2, False), (33, 4, 0, True)])
def test_sigmoid_bias_selection_matches_the_sorted_order(experts, top_k, shared, norm):
    """The GLM / Nemotron routers' selection: picks equal the sort by (-(sigmoid + bias), id), weights the normalised
    scores; rows whose choices are closer than the exp's rounding are left out of the index check."""

    from oracle import routers
    from tensorfold_b200 import moe

    rows = 97
    g = torch.Generator(device="cuda").manual_seed(experts)
    logits = torch.randn((rows, experts + 3), generator=g, device="cuda") * 2.0
    bias = torch.randn((experts,), generator=g, device="cuda") * 0.1
    logits[5, :experts] = 0.25                                   # a row of ties: the lowest ids win
    bias_t = bias.clone()
    slots = top_k + shared
    pick = torch.zeros((rows, slots), dtype=torch.int32, device="cuda")
    wts = torch.zeros((rows, slots), dtype=torch.float32, device="cuda")
    moe.select_sigmoid(logits, bias_t, pick, wts, top_k, experts, 2.5, norm, shared)
    want_pick, want_wts, gap = routers.sigmoid_topk(logits.cpu().numpy(), bias.cpu().numpy(), top_k, 2.5, norm, shared)
    got_pick, got_wts = pick.cpu().numpy(), wts.cpu().numpy()
    clear = gap > 1e-6
    clear[5] = False
    assert clear.sum() > rows * 0.9
    assert (got_pick[clear] == want_pick[clear]).all()
    np.testing.assert_allclose(got_wts[clear], want_wts[clear], rtol=2e-6, atol=1e-7)
    assert (got_pick[:, top_k:] == np.arange(experts, experts + shared)).all() and (got_wts[:, top_k:] == 1).all()
    # the tie row: equal scores, so the order is by bias then id - compare with the sort on the same fp32 values
    score = 1.0 / (1.0 + np.exp(-np.float32(0.25)))
    choice = (np.float32(score) + bias.cpu().numpy()).astype(np.float32)
    order = sorted(range(experts), key=lambda i: (-choice[i], i))[:top_k]
    assert got_pick[5, :top_k].tolist() == order


@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,d,slots,top_k", [(5, 2688, 8, 6), (64, 2048, 9, 8), (3, 8192, 4, 4), (2, 64, 3, 1)])
def test_add_moe_norm_against_float64(rows, d, slots, top_k, ydtype):
    """Combine + residual add + RMSNorm in one launch (the Nemotron family's ``add_moe_norm``): the new hidden state
    within one bf16 ulp of the float64 result, the normed row within 2^-7, the group sums equal to the sums of the
    stored values."""

    from tensorfold_b200 import moe

    g = torch.Generator().manual_seed(rows + d)
    h = torch.randn((rows, d), generator=g).to(torch.bfloat16).to(DEV)
    y = (torch.randn((rows * slots, d), generator=g) * 0.5).to(ydtype).to(DEV)
    wt = torch.rand((rows, slots), generator=g).float().to(DEV)
    w = (torch.rand((d,), generator=g) + 0.5).to(torch.bfloat16).to(DEV)
    eps = 1e-5
    hn, out, xs = moe.add_moe_norm(h, y, wt, w, eps, top_k)
    y64 = y.double().view(rows, slots, d)
    routed = (wt.double()[:, :top_k, None] * y64[:, :top_k]).sum(1)
    delta = (routed + y64[:, top_k:].sum(1)).to(torch.bfloat16).double()
    want_h = (h.double() + delta)
    ulp = torch.maximum(want_h.abs(), torch.tensor(1e-30, device=DEV, dtype=torch.float64)) * 2.0 ** -7
    assert bool(((hn.double() - want_h).abs() <= ulp + 1e-6).all())
    hf = hn.double()
    want_out = hf / torch.sqrt((hf * hf).mean(1, keepdim=True) + eps) * w.double()
    assert float((out.double() - want_out).abs().max()) <= 2.0 ** -7 * float(want_out.abs().max())
    sums = out.float().view(rows, d // 64, 64).sum(2)
    assert torch.allclose(xs, sums, rtol=1e-5, atol=1e-5)
