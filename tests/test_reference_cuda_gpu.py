"""This library's kernels against the REFERENCE's own CUDA kernels on the same GPU: the reference's ``experts.cu`` /
``experts_pack.cu`` compiled unmodified for sm_100 by ``oracle/build_ref_cuda.py`` (where the reference tree is
mounted; the built module travels to the GPU box).  The plan tables must be equal; activations and per-pair outputs
agree within the reference's own bars against float64 (``tests/cuda/test_experts.py:159-188``: 2^-6 of the largest
activation, 1e-5 of the largest output), taken twice since both sides carry them.  Skipped when the module was never
built."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref_cuda

    mod = build_ref_cuda.load()
    if mod is None:
        pytest.skip("the reference's CUDA extension was not built (oracle/build_ref_cuda.py needs the reference tree)")
    return mod


def _ref_plan(ref, picks, experts, tile=16):
    rows, slots = picks.shape
    pairs = rows * slots
    members = torch.zeros((pairs,), dtype=torch.int32, device=DEV)
    items = torch.zeros((min(pairs, experts) + pairs // 16, 3), dtype=torch.int32, device=DEV)
    counts = torch.zeros((2,), dtype=torch.int32, device=DEV)
    rank = torch.zeros((max(pairs, 1),), dtype=torch.int32, device=DEV)
    hist = torch.zeros((-(-pairs // 1024) * experts,), dtype=torch.int32, device=DEV)
    ref.plan(picks, pairs, experts, tile, members, items, counts, rank, hist)
    return members, items, counts


@pytest.mark.parametrize("rows,slots,experts", [(23, 7, 50), (300, 7, 50), (1500, 7, 50), (64, 8, 128), (256, 9, 257)])
def test_plan_tables_equal_the_reference_kernels(ref, rows, slots, experts):
    from tensorfold_b200 import experts as grouped

    g = torch.Generator().manual_seed(rows + slots)
    picks = torch.stack([torch.randperm(experts, generator=g)[:slots] for _ in range(rows)]).to(torch.int32)
    picks[:, 0] = 3                                                    # one expert present in every row
    picks = picks.to(DEV).contiguous()
    members, items, counts = _ref_plan(ref, picks, experts)
    plan = grouped.Plan(rows, slots, experts, DEV, decode_tile=grouped.WIDE_TILE)
    grouped.route(picks, plan)
    torch.cuda.synchronize()
    n = int(counts[0])
    assert plan.counts.tolist() == counts.tolist()
    assert torch.equal(plan.items[:n], items[:n])
    assert torch.equal(plan.members, members)


@pytest.mark.parametrize("rows", [1, 9, 64])
def test_gate_up_and_down_against_the_reference_kernels(ref, rows):
    """Both projections of a small layer (bf16 scales, the reference's convention) through both libraries."""

    from tensorfold_b200 import experts as grouped
    from tensorfold_b200 import synthetic

    shape = synthetic.LayerShape("ref_check", 11, 512, 24, 256, 6)
    gate, up, down = synthetic.affine_layer(shape, DEV, torch.bfloat16)
    x = synthetic.activations(shape, rows, DEV)
    g = torch.Generator().manual_seed(rows)
    picks = torch.stack([torch.randperm(shape.experts, generator=g)[:shape.top_k] for _ in range(rows)])
    picks = picks.to(torch.int32).to(DEV).contiguous()
    pairs, nb_up, nb_down = rows * shape.top_k, shape.width // 32, shape.dims // 32

    def ref_pack(m):
        e, n, k8 = m[0].shape
        out = torch.empty((e, n // 32, k8 * 8 // 64, 288), dtype=torch.int32, device=DEV)
        ref.pack(m[0].contiguous(), m[1].contiguous(), m[2].contiguous(), 64, out)
        return out

    w_up = torch.stack([ref_pack(gate), ref_pack(up)], dim=3).contiguous()
    w_down = ref_pack(down).unsqueeze(3).contiguous()
    members, items, counts = _ref_plan(ref, picks, shape.experts)
    max_items = min(pairs, shape.experts) + pairs // 16
    act_r = torch.zeros((pairs, shape.width), dtype=torch.bfloat16, device=DEV)
    y_r = torch.zeros((pairs, shape.dims), dtype=torch.float32, device=DEV)
    ref.run(64, 2, x, shape.top_k, w_up, shape.dims // 64, nb_up, items, counts, members, act_r, shape.width, 0.0,
            max_items * nb_up)
    ref.run(64, 0, act_r, 0, w_down, shape.width // 64, nb_down, items, counts, members, y_r, shape.dims, 0.0,
            max_items * nb_down)
    ex = grouped.make([gate, up], down, 64)
    plan = grouped.Plan(rows, shape.top_k, shape.experts, DEV)
    grouped.route(picks, plan)
    act = torch.zeros_like(act_r)
    y = torch.zeros_like(y_r)
    grouped.gate_up(x, ex, plan, act, rows)
    grouped.down(act_r, ex, plan, y, rows)                            # the same inputs as the reference's down
    torch.cuda.synchronize()
    a, b = act.float().cpu().numpy(), act_r.float().cpu().numpy()
    assert np.abs(a - b).max() <= 2 * 2.0 ** -6 * np.abs(b).max()
    assert np.abs(y.cpu().numpy() - y_r.cpu().numpy()).max() <= 2e-5 * np.abs(y_r.cpu().numpy()).max()
    assert np.isfinite(a).all() and np.abs(b).max() > 0


@pytest.fixture(scope="module")
def ref_exl3():
    from oracle import build_ref_cuda

    mod = build_ref_cuda.load("exl3")
    if mod is None:
        pytest.skip("the reference's EXL3 extension was not built (oracle/build_ref_cuda.py needs the reference tree)")
    return mod


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_trellis_decode_equals_the_reference_kernels(ref_exl3, cb):
    """W_q of every width through this library's lane decode and through the reference's kernel: the same fp16 bits."""

    from tensorfold_b200.exl3 import experts as x3

    g = torch.Generator().manual_seed(40 + cb)
    for k2 in range(2, 17):
        t = torch.randint(-32768, 32768, (8, 16, 8 * k2), dtype=torch.int32, generator=g).to(torch.int16).to(DEV)
        want = torch.empty((128, 256), dtype=torch.float16, device=DEV)
        ref_exl3.dequant(t.contiguous(), want, k2, cb)
        got = x3.dequant(t, cb)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), k2


@pytest.mark.parametrize("rows,weighted", [(1, True), (9, False), (64, True)])
def test_routed_exl3_layer_against_the_reference_kernels(ref_exl3, rows, weighted):
    """A mixed-width layer through both libraries' launches: per-slot rows (or the weighted sum) agree to 2e-3 of the
    largest output (each side is within the reference's 1e-2 bar of float64; the roundings differ only in the order of
    fp32 sums)."""

    from oracle import ref_exl3 as drive
    from tensorfold_b200 import synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape = synthetic.LayerShape("ref_x3", 12, 512, 16, 256, 4)
    bits = lambda e, m: (2, 3, 4, 5, 6, 8)[(e + m) % 6]                             # noqa: E731
    gate, up, down = synthetic.exl3_layer(shape, DEV, bits)
    ex = x3.prepare(gate, up, down, x3.CB_3INST, device=DEV)
    x = synthetic.activations(shape, rows, DEV)
    g = torch.Generator().manual_seed(rows)
    pick = torch.stack([torch.randperm(shape.experts + 1, generator=g)[:shape.top_k] for _ in range(rows)])
    pick = pick.to(torch.int32).to(DEV).contiguous()                               # id 16 is not a routed expert
    wts = (torch.rand((rows, shape.top_k), generator=g) * 0.3 + 0.05).to(DEV) if weighted else None
    s_ref = drive.Scratch(ex, rows, shape.top_k)
    out_ref = torch.zeros((rows, shape.dims), dtype=torch.float32, device=DEV)
    want = drive.routed(ref_exl3, x, pick, wts, ex, s_ref, out_ref).clone()
    s = x3.Scratch(ex, rows, shape.top_k)
    got = x3.routed(x, pick, wts, ex, s, None, rows)
    torch.cuda.synchronize()
    if not weighted:                                                               # skipped slots keep what they held: 0
        want, got = want.view(rows, shape.top_k, -1), got.view(rows, shape.top_k, -1)
    assert torch.isfinite(got).all() and float(want.abs().max()) > 0
    assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())
    assert int(s.count[0]) == int(s_ref.count[0])
