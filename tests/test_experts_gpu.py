"""Grouped affine 4-bit experts on the GPU: pack round trip, dequantised weights bit for bit, window invariance,
and outputs against float64 and the CPU oracle.  Calls go through the C ABI via the reference-shaped operators."""

import numpy as np
import pytest
import torch

from helpers import bits, rel_l2, triple_np, words_np

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (SwiGLU, limit, experts incl. shared, D, NI, shared slots): small twins of the reference's cases
CASES = [(True, 0.0, 41, 256, 128, 1), (True, 10.0, 19, 512, 128, 1), (False, 0.0, 12, 384, 192, 2)]
DTYPES = [torch.bfloat16, torch.float16]


def mlx(e, n, k, seed, dtype=torch.bfloat16, gs=64):
    g = torch.Generator(device=DEV).manual_seed(seed)
    words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, n, k // 8), generator=g, device=DEV,
                          dtype=torch.int64).to(torch.int32)
    scales = (torch.rand((e, n, k // gs), generator=g, device=DEV) * 0.02 + 0.001).to(dtype)
    biases = (torch.randn((e, n, k // gs), generator=g, device=DEV) * 0.02).to(dtype)
    return words, scales, biases


def dequant64(words, scales, biases, gs=64):
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=words.device, dtype=torch.int64) * 4
    q = ((w[..., None] >> shifts) & 0xF).reshape(*words.shape[:-1], -1).double()
    return q * scales.double().repeat_interleave(gs, -1) + biases.double().repeat_interleave(gs, -1)


def build(case, seed, dtype=torch.bfloat16):
    from tensorfold_b200 import experts

    swiglu, limit, e, d, ni, _ = case
    up = [mlx(e, ni, d, seed + i, dtype) for i in range(2 if swiglu else 1)]
    down = mlx(e, d, ni, seed + 7, dtype)
    return experts.make(up, down, 64, limit=limit), up, down


def picks_for(rows, case, seed, hot=None):
    _, _, e, _, _, shared = case
    routed = e - shared
    k = min(6, routed)
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(rows):
        r = torch.arange(k) if hot is not None else torch.randperm(routed, generator=g)[:k]
        out.append(torch.cat([r, torch.arange(routed, e)]))
    return torch.stack(out).to(torch.int32).to(DEV)


def experts_tile():
    from tensorfold_b200 import experts

    return experts.TILE


def run(ex, x, picks):
    from tensorfold_b200 import experts

    rows, slots = picks.shape
    plan = experts.Plan(rows, slots, ex.count, DEV)
    experts.route(picks.contiguous(), plan)
    act = torch.empty((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
    y = torch.empty((rows * slots, ex.dims), dtype=torch.float32, device=DEV)
    experts.gate_up(x, ex, plan, act, rows)
    experts.down(act, ex, plan, y, rows)
    return act, y, plan


@pytest.mark.parametrize("dtype", DTYPES)
def test_pack_round_trip(dtype):
    from tensorfold_b200 import experts

    w = mlx(3, 96, 256, 61, dtype)
    back = experts.unpack(experts.pack(*w, 64), 64, dtype)
    assert all(torch.equal(a, b) for a, b in zip(back, w))


@pytest.mark.parametrize("dtype", DTYPES)
def test_dequantised_weights_bit_exact(dtype):
    """The kernels' weight values against the CPU oracle's, both forms, bit for bit."""

    from oracle import cpu
    from tensorfold_b200 import experts

    w = mlx(2, 64, 192, 5, dtype)
    blocks = experts.pack(*w, 64)
    fp16 = dtype == torch.float16
    wn = triple_np(w)
    dec = experts.dequantize(blocks, 64, scale_dtype=dtype).cpu().numpy()
    assert np.array_equal(dec.view(np.uint32), cpu.dequant(*wn, 64, fp16, False).view(np.uint32))
    assert np.array_equal(dec, dequant64(*w).float().cpu().numpy())
    pre = experts.dequantize(blocks, 64, prefill=True, scale_dtype=dtype).float().cpu().numpy()
    assert np.array_equal(pre.view(np.uint32), cpu.dequant(*wn, 64, fp16, True).view(np.uint32))


def test_one_hot_rows_read_back_every_nibble():
    """Scale 1, bias 0 and one-hot inputs return each stored code through the decode matmul
    (the probe of the reference's tests/cuda/test_qmm.py:98-111)."""

    from tensorfold_b200 import experts

    e, n, k = 2, 64, 128
    g = torch.Generator(device=DEV).manual_seed(2)
    words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, n, k // 8), generator=g, device=DEV,
                          dtype=torch.int64).to(torch.int32)
    ones = torch.ones((e, n, k // 64), dtype=torch.bfloat16, device=DEV)
    zeros = torch.zeros_like(ones)
    ex = experts.make([(words, ones, zeros)], (torch.zeros((e, k, n // 8), dtype=torch.int32, device=DEV),
                                               torch.ones((e, k, n // 64), dtype=torch.bfloat16, device=DEV),
                                               torch.zeros((e, k, n // 64), dtype=torch.bfloat16, device=DEV)), 64)
    x = torch.eye(k, dtype=torch.bfloat16, device=DEV)                         # row i: input i alone
    q = ((words.to(torch.int64)[..., None] >> (torch.arange(8, device=DEV) * 4)) & 0xF).reshape(e, n, k).float()
    for expert in range(e):
        picks = torch.full((k, 1), expert, dtype=torch.int32, device=DEV)
        plan = experts.Plan(k, 1, e, DEV)
        experts.route(picks, plan)
        out = torch.empty((k, n), dtype=torch.float32, device=DEV)
        experts._run(0, x, 1, ex.up, k // 64, n // 32, plan, out, n, 0.0, experts.max_items(k, e), ex)
        assert torch.equal(out, q[expert].t().contiguous())


@pytest.mark.parametrize("case", CASES)
def test_pairs_do_not_depend_on_the_window(case, pdl):
    ex, _, _ = build(case, 11)
    rows = 40
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    picks = picks_for(rows, case, 3)
    slots = picks.shape[1]
    act, y, _ = run(ex, x, picks)
    alone = [run(ex, x[r:r + 1], picks[r:r + 1]) for r in range(rows)]
    assert torch.equal(act, torch.cat([a[0] for a in alone])) and torch.equal(y, torch.cat([a[1] for a in alone]))
    for m in (2, 3, 8, 9, 16, 17, 33):
        a_m, y_m, _ = run(ex, x[:m], picks[:m])
        assert torch.equal(a_m, act[:m * slots]) and torch.equal(y_m, y[:m * slots]), m
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(5)).to(DEV)
    a_p, y_p, _ = run(ex, x[perm], picks[perm])
    idx = (perm[:, None] * slots + torch.arange(slots, device=DEV)).reshape(-1)
    assert torch.equal(a_p, act[idx]) and torch.equal(y_p, y[idx])


@pytest.mark.parametrize("case", CASES)
def test_an_expert_shared_by_many_rows(case):
    ex, _, _ = build(case, 21)
    rows = 37
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    picks = picks_for(rows, case, 4, hot=0)
    _, y, plan = run(ex, x, picks)
    slots = picks.shape[1]
    alone = torch.cat([run(ex, x[r:r + 1], picks[r:r + 1])[1] for r in range(rows)])
    assert torch.equal(y, alone)
    assert int(plan.counts[1]) == slots
    assert int(plan.counts[0]) == slots * -(-37 // experts_tile())   # 37 pairs an expert: full items, then the rest


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_matches_fp64(case, dtype):
    """Against float64 over the dequantised weights, with the reference's own bars
    (tests/cuda/test_experts.py:159-188): act within 2^-6 of the largest value, down within 1e-5 of it."""

    swiglu, limit = case[0], case[1]
    ex, up, down = build(case, 31, dtype)
    rows = 5
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    picks = picks_for(rows, case, 6)
    act, y, _ = run(ex, x, picks)
    slots = picks.shape[1]
    pe = picks.reshape(-1).long()
    xr = x.double().repeat_interleave(slots, 0)
    projs = [torch.einsum("pk,pnk->pn", xr, dequant64(*m)[pe]) for m in up]
    if swiglu:
        g, u = (t.float().to(torch.bfloat16).double() for t in projs)
        if limit:
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        ref = (g * torch.sigmoid(g)).to(torch.bfloat16).double() * u
    else:
        ref = projs[0].float().to(torch.bfloat16).double().clamp(min=0) ** 2
    assert (act.double() - ref).abs().max() <= 2 ** -6 * ref.abs().max()
    yref = torch.einsum("pk,pnk->pn", act.double(), dequant64(*down)[pe])
    assert (y.double() - yref).abs().max() <= 1e-5 * yref.abs().max()


def test_graph_replay_follows_the_picks(pdl):
    from tensorfold_b200 import experts

    case = CASES[1]
    ex, _, _ = build(case, 41)
    rows = 9
    picks = picks_for(rows, case, 7).contiguous()
    slots = picks.shape[1]
    plan = experts.Plan(rows, slots, ex.count, DEV)
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    act = torch.empty((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
    y = torch.empty((rows * slots, ex.dims), dtype=torch.float32, device=DEV)

    def step():
        experts.route(picks, plan)
        experts.gate_up(x, ex, plan, act, rows)
        experts.down(act, ex, plan, y, rows)

    step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for seed in (8, 9):
        picks.copy_(picks_for(rows, case, seed))
        g.replay()
        _, want, _ = run(ex, x, picks)
        assert torch.equal(y, want)


def test_many_units_keep_the_bits():
    case = (True, 0.0, 257, 2048, 128, 1)
    ex, _, _ = build(case, 81)
    rows = 64
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    g = torch.Generator().manual_seed(12)
    picks = torch.stack([torch.cat([torch.randperm(256, generator=g)[:8], torch.tensor([256])])
                         for _ in range(rows)]).to(torch.int32).to(DEV)
    _, y, plan = run(ex, x, picks)
    for r in (0, 31, 63):
        assert torch.equal(run(ex, x[r:r + 1], picks[r:r + 1])[1], y[9 * r:9 * r + 9]), r


@pytest.mark.parametrize("shared", [False, True])
@pytest.mark.parametrize("rows", [1, 9, 64])
def test_layer_against_the_cpu_oracle(rows, shared, pdl):
    """moe.run end to end on a small layer: picks bit exact, weights within a bf16 ulp, output rel-L2 <= 1e-2 against
    the fp64-accumulated reference and against the CPU restatement."""

    from oracle import affine, cpu
    from tensorfold_b200 import experts, moe, synthetic

    shape = synthetic.SMALL_SHARED if shared else synthetic.SMALL
    gate, up, down = synthetic.affine_layer(shape, DEV)
    x = synthetic.activations(shape, rows, DEV)
    rt = synthetic.router_rows(shape, DEV)
    layer = moe.Routed(rt, experts.make([gate, up], down, 64), shape.top_k, shared=shared)
    buf = moe.MoEBuffers(rows, moe._Shape(layer), DEV, shared=shared)
    moe.moe(x, layer.router, layer.experts, buf, layer.top_k, layer.count)
    out = moe.combine(buf.y[:rows], buf.wts[:rows])
    assert torch.equal(moe.run(x, layer), out)
    o_cpu, pick, wts, act, y = cpu.moe_layer(bits(x), bits(rt), shape.experts, shape.top_k, shared, triple_np(gate),
                                             triple_np(up), triple_np(down), 64, True, want_parts=True)
    assert np.array_equal(buf.pick[:rows].cpu().numpy(), pick)
    assert np.abs(buf.wts[:rows].cpu().numpy() - wts).max() <= 2 ** -8
    _, _, o64 = affine.layer64(bits(x), pick, wts, triple_np(gate), triple_np(up), triple_np(down), 64, True)
    assert rel_l2(out.float().cpu().numpy(), o64) <= 1e-2
    assert rel_l2(out.float().cpu().numpy(), affine.bf16_value(o_cpu)) <= 1e-2


@pytest.mark.parametrize("shared", [False, True])
@pytest.mark.parametrize("rows", [1, 5, 9, 64])
def test_fewer_launches_give_the_same_bits(rows, shared, pdl):
    """The layer with the one-launch routing and with the combine folded into the down projection (three launches)
    against the default six: the same output bits, per-slot rows and plan, eagerly and from a CUDA graph, twice in a
    row (the kernels' arrival counters return to zero)."""

    from tensorfold_b200 import experts, moe, synthetic

    shape = synthetic.SMALL_SHARED if shared else synthetic.SMALL
    gate, up, down = synthetic.affine_layer(shape, DEV)
    layer = moe.Routed(synthetic.router_rows(shape, DEV), experts.make([gate, up], down, 64), shape.top_k, shared=shared)
    xs = [synthetic.activations(shape, rows, DEV, index=30 + i) for i in range(2)]
    want = [moe.run(x, layer).clone() for x in xs]
    was = moe.FUSED_ROUTE_ROWS, moe.FUSED_COMBINE_ROWS
    try:
        moe.FUSED_ROUTE_ROWS, moe.FUSED_COMBINE_ROWS = 256, 256
        buf = moe.MoEBuffers(rows, moe._Shape(layer), DEV, shared=shared)
        out = torch.zeros((rows, shape.dims), dtype=torch.bfloat16, device=DEV)
        for x, w in zip(xs, want):
            assert moe.layer(x, layer, buf, out) == 3
            assert torch.equal(out, w)
            assert torch.equal(moe.combine(buf.y[:rows], buf.wts[:rows]), w)      # every slot's row is still stored
            assert int(buf.arrive_route.abs().sum()) == 0 and int(buf.arrive_combine.abs().sum()) == 0
        runner = moe.Runner(layer, rows)
        assert runner.launches == 3
        for x, w in zip(xs, want):
            assert torch.equal(runner(x), w)
    finally:
        moe.FUSED_ROUTE_ROWS, moe.FUSED_COMBINE_ROWS = was


@pytest.mark.parametrize("reduce", ["rows", "tokens"])
def test_gathered_expert_parallel_on_one_rank_is_the_layer(reduce):
    """World size 1: the expert-parallel step (windowed plan and combine included) gives moe.run's output."""

    from tensorfold_b200 import ep, experts, moe, synthetic

    shape, rows = synthetic.SMALL, 33
    gate, up, down = synthetic.affine_layer(shape, DEV)
    rt = synthetic.router_rows(shape, DEV)
    ex = experts.make([gate, up], down, 64)
    x = synthetic.activations(shape, rows, DEV)
    want = moe.run(x, moe.Routed(rt, ex, shape.top_k, shared=False))
    got = ep.GatheredExpertParallel(rt, ex, shape.experts, shape.top_k, rows, reduce=reduce).forward(x)
    if reduce == "rows":
        assert torch.equal(got, want)
    else:
        assert torch.equal(got, want)          # one rank: the partial sum is the whole slot-order sum


@pytest.mark.parametrize("case", CASES)
def test_items_of_16_pairs_give_the_same_bits(case):
    from tensorfold_b200 import experts

    ex, _, _ = build(case, 51)
    rows = 60
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    picks = picks_for(rows, case, 9, hot=0)                       # every row on the same experts: full items
    act, y, plan8 = run(ex, x, picks)
    slots = picks.shape[1]
    plan = experts.Plan(rows, slots, ex.count, DEV, decode_tile=experts.WIDE_TILE)
    experts.route(picks.contiguous(), plan)
    act16 = torch.empty_like(act)
    y16 = torch.empty_like(y)
    experts.gate_up(x, ex, plan, act16, rows)
    experts.down(act16, ex, plan, y16, rows)
    assert torch.equal(act16, act) and torch.equal(y16, y)
    assert int(plan.counts[0]) < int(plan8.counts[0])


def test_split_plan_sets_hot_experts_apart_and_keeps_the_cold_pairs_bits():
    """``Plan(hot=)`` + ``route_split``: experts with at least ``hot`` pairs (here also under a window offset) get
    prompt-form items, the rest decode items; cold pairs keep their bits, hot pairs stay within the layer tolerance."""

    from tensorfold_b200 import experts

    case = CASES[0]                                      # 41 experts incl. 1 shared
    ex, _, _ = build(case, 51)
    rows, hot = 60, 24
    g = torch.Generator().manual_seed(5)
    # expert 3 in every row, expert 7 in half of them, the rest spread thin; the shared expert (40) in every row
    cols = []
    for r in range(rows):
        rest = (torch.randperm(30, generator=g)[:3] + 9).tolist()
        cols.append([3, 7 if r % 2 == 0 else 8] + rest + [40])
    picks = torch.tensor(cols, dtype=torch.int32, device=DEV)
    slots = picks.shape[1]
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    _, y_plain, _ = run(ex, x, picks)
    plan = experts.Plan(rows, slots, ex.count, DEV, hot=hot)
    experts.route_split(picks, plan)
    counts = np.bincount(picks.cpu().numpy().reshape(-1), minlength=ex.count)
    n_small, n_big = plan.counts.cpu().tolist(), plan.big_counts.cpu().tolist()
    hot_ids = [e for e in range(ex.count) if counts[e] >= hot]
    assert sorted(hot_ids) == [3, 7, 8, 40]
    assert n_big == [len(hot_ids), len(hot_ids)] and n_small[1] == int((counts > 0).sum()) - len(hot_ids)
    big = plan.big_items[:n_big[0]].cpu().numpy()
    small = plan.items[:n_small[0]].cpu().numpy()
    assert big[:, 0].tolist() == hot_ids and big[:, 2].tolist() == [int(counts[e]) for e in hot_ids]
    assert not set(small[:, 0].tolist()) & set(hot_ids) and (small[:, 2] <= plan.tile).all()
    members = plan.members.cpu().numpy()
    pk = picks.cpu().numpy().reshape(-1)
    for e, first, cnt in list(big) + list(small):
        mine = members[first:first + cnt]
        assert (pk[mine] == e).all() and (np.diff(mine) > 0).all()
    act = torch.zeros((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
    y = torch.zeros((rows * slots, ex.dims), dtype=torch.float32, device=DEV)
    experts.gate_up(x, ex, plan, act, rows)
    experts.down(act, ex, plan, y, rows)
    cold = torch.from_numpy(~np.isin(pk, hot_ids)).to(DEV)
    assert torch.equal(y[cold], y_plain[cold])
    err = (y[~cold].double() - y_plain[~cold].double()).norm() / y_plain[~cold].double().norm()
    assert 0 < err < 1e-2
    # a window: only experts 8..39, renumbered from 0
    sub = experts.Plan(rows, slots, 32, DEV, hot=hot)
    experts.route_split(picks, sub, lo=8)
    assert sub.big_items[:sub.big_counts[0].item(), 0].cpu().tolist() == [0]          # expert 8
    assert int(sub.items[:sub.counts[0].item(), 2].sum()) + int(counts[8]) == int(counts[8:40].sum())
