"""The prefill form (tcgen05 grouped GEMM) through the C ABI: weights bit for bit, chunk and item invariance,
outputs against float64 over the bf16-rounded weights and against the CPU oracle."""

import numpy as np
import pytest
import torch

from helpers import bits, rel_l2, triple_np
from test_experts_gpu import CASES, DTYPES, build, dequant64, mlx, picks_for

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run(ex, x, picks, tile=None, y_dtype=torch.float32):
    from tensorfold_b200 import experts

    rows, slots = picks.shape
    plan = experts.Plan(rows, slots, ex.count, DEV, prefill=True)
    experts.route(picks.contiguous(), plan, tile or experts.PREFILL_TILE)
    act = torch.empty((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
    y = torch.empty((rows * slots, ex.dims), dtype=y_dtype, device=DEV)
    experts.gate_up(x, ex, plan, act, rows)
    experts.down(act, ex, plan, y, rows)
    return act, y, plan


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_hot_rows_read_back_the_prefill_weights(dtype):
    """One-hot inputs return each bf16 weight exactly (fp32 out): the operand layout, the swizzle and the prefill
    form's rounding, bit for bit against the CPU oracle."""

    from oracle import cpu
    from tensorfold_b200 import _lib, experts

    e, n, k = 3, 192, 256
    w = mlx(e, n, k, 77, dtype)
    ex = experts.make([w], mlx(e, k, n, 78, dtype), 64)
    want = cpu.dequant(*triple_np(w), 64, dtype == torch.float16, True)          # [e, n, k] bf16 values as fp32
    x = torch.eye(k, dtype=torch.bfloat16, device=DEV)
    for expert in range(e):
        picks = torch.full((k, 1), expert, dtype=torch.int32, device=DEV)
        plan = experts.Plan(k, 1, e, DEV, prefill=True)
        experts.route(picks, plan)
        out = torch.zeros((k, n), dtype=torch.float32, device=DEV)
        experts._run(0, x, 1, ex.up, k // 64, n // 32, plan, out, n, 0.0, experts.max_items(k, e, plan.tile), ex, True)
        torch.cuda.synchronize()
        assert _lib.kernel_status() == 0
        assert np.array_equal(out.cpu().numpy().view(np.uint32), np.ascontiguousarray(want[expert].T).view(np.uint32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_matches_fp64_over_bf16_weights(case, dtype):
    swiglu, limit = case[0], case[1]
    ex, up, down = build(case, 31, dtype)
    rows = 5
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    picks = picks_for(rows, case, 6)
    act, y, _ = run(ex, x, picks)
    slots = picks.shape[1]
    pe = picks.reshape(-1).long()
    xr = x.double().repeat_interleave(slots, 0)

    def weights(m):
        if dtype == torch.bfloat16:
            return dequant64(*m).to(torch.bfloat16).double()      # (double -> bf16 double rounding is vanishingly rare)
        return dequant64(*m).float().to(torch.bfloat16).double()

    projs = [torch.einsum("pk,pnk->pn", xr, weights(m)[pe]) for m in up]
    if swiglu:
        g, u = (t.float().to(torch.bfloat16).double() for t in projs)
        if limit:
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        ref = (g * torch.sigmoid(g)).to(torch.bfloat16).double() * u
    else:
        ref = projs[0].float().to(torch.bfloat16).double().clamp(min=0) ** 2
    assert (act.double() - ref).abs().max() <= 2 ** -6 * ref.abs().max()
    yref = torch.einsum("pk,pnk->pn", act.double(), weights(down)[pe])
    assert (y.double() - yref).abs().max() <= 1e-5 * yref.abs().max()


@pytest.mark.parametrize("case", CASES)
def test_rows_do_not_depend_on_the_chunk_or_the_item(case, pdl):
    ex, _, _ = build(case, 71)
    rows = 200
    x = (torch.randn((rows, ex.dims), device=DEV) * 0.5).to(torch.bfloat16)
    picks = picks_for(rows, case, 13)
    slots = picks.shape[1]
    act, y, plan = run(ex, x, picks)
    for a, b in ((0, 1), (77, 78), (199, 200), (0, 7), (5, 22), (0, 64), (100, 200)):
        a1, y1, _ = run(ex, x[a:b], picks[a:b])
        assert torch.equal(a1, act[a * slots:b * slots]) and torch.equal(y1, y[a * slots:b * slots]), (a, b)
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(5)).to(DEV)
    a_p, y_p, _ = run(ex, x[perm], picks[perm])
    idx = (perm[:, None] * slots + torch.arange(slots, device=DEV)).reshape(-1)
    assert torch.equal(a_p, act[idx]) and torch.equal(y_p, y[idx])
    _, y16, _ = run(ex, x, picks, y_dtype=torch.bfloat16)
    assert torch.equal(y16, y.to(torch.bfloat16))                  # bf16 down is the fp32 result rounded once
    counts = {}
    for tile in (16, 64, 192):                                     # items of any size give every pair the same bits
        a_t, y_t, p_t = run(ex, x, picks, tile=tile)
        assert torch.equal(a_t, act) and torch.equal(y_t, y), tile
        counts[tile] = int(p_t.counts[0])
    assert counts[192] <= counts[64] < counts[16]


@pytest.mark.parametrize("shared", [False, True])
def test_prefill_layer_against_the_oracle(shared, pdl):
    from oracle import affine, cpu
    from tensorfold_b200 import _lib, experts, moe, synthetic

    shape = synthetic.SMALL_SHARED if shared else synthetic.SMALL
    rows = 300
    gate, up, down = synthetic.affine_layer(shape, DEV)
    x = synthetic.activations(shape, rows, DEV)
    rt = synthetic.router_rows(shape, DEV)
    layer = moe.Routed(rt, experts.make([gate, up], down, 64), shape.top_k, shared=shared)
    out = moe.run(x, layer, prefill=True)
    torch.cuda.synchronize()
    assert _lib.kernel_status() == 0
    logits = cpu.router_logits(bits(x), bits(rt))
    pick, wts = cpu.topk_rows(logits, shape.experts, shape.top_k, shared)
    _, _, o64 = affine.layer64(bits(x), pick, wts, triple_np(gate), triple_np(up), triple_np(down), 64, True,
                               prefill=True)
    assert rel_l2(out.float().cpu().numpy(), o64) <= 1e-2
    dec = moe.run(x, layer)                                        # the decode form agrees within the same tolerance
    assert rel_l2(out.float().cpu().numpy(), dec.float().cpu().numpy()) <= 1e-2
