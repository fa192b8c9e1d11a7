"""EXL3 routed experts on the GPU through the C ABI: lane decode bit for bit against the oracle and the reference's
fixtures, grouping order, window invariance, and the layer against float64."""

import math
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLDEN = np.load(Path(__file__).parent / "golden" / "exl3_golden.npz")


def _trellis(k, n, k2, gen):
    v = torch.randint(-32768, 32768, (k // 16, n // 16, 8 * k2), dtype=torch.int32, generator=gen)
    return v.to(torch.int16).to(DEV).contiguous()


def _scale(n, mag, gen):
    sign = torch.randint(0, 2, (n,), generator=gen).float() * 2 - 1
    return (sign * (torch.rand((n,), generator=gen) + 0.5) * mag).half().to(DEV)


@pytest.mark.parametrize("cb", [0, 1, 2])
@pytest.mark.parametrize("k2", list(range(2, 17)))
def test_decode_matches_the_bitstream(cb, k2):
    """Every codebook and width (half-integer rates included) against the numpy restatement, bit for bit."""

    from oracle import exl3 as ref
    from tensorfold_b200.exl3 import experts

    g = torch.Generator().manual_seed(100 * cb + k2)
    t = _trellis(48, 32, k2, g)
    got = experts.dequant(t, cb).cpu().numpy()
    want = ref.unpack(t.cpu().numpy(), cb)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_decode_matches_the_reference_fixtures():
    from tensorfold_b200.exl3 import experts

    for key in GOLDEN.files:
        if key.startswith("t_cb"):
            cb = int(key[4])
            got = experts.dequant(torch.from_numpy(GOLDEN[key]).to(DEV), cb).cpu().numpy()
            assert np.array_equal(got.view(np.uint16), GOLDEN["w" + key[1:]]), key


def _layer(E, D, I, k2s, cb, seed):
    from tensorfold_b200.exl3 import experts

    g = torch.Generator().manual_seed(seed)
    gate, up, down = [], [], []
    for e in range(E):
        kg, ku, kd = k2s[e]
        gate.append((_trellis(D, I, kg, g), _scale(D, 1 / math.sqrt(D), g), _scale(I, 1.0, g)))
        up.append((_trellis(D, I, ku, g), _scale(D, 1 / math.sqrt(D), g), _scale(I, 1.0, g)))
        down.append((_trellis(I, D, kd, g), _scale(I, 1 / math.sqrt(I), g), _scale(D, 0.25, g)))
    return experts.prepare(gate, up, down, cb), (gate, up, down)


def _picks(E, R, k, gen, shared=False):
    sel = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(R)]).to(torch.int32)
    w = torch.rand((R, k), generator=gen) * 0.2 + 0.05
    if shared:
        sel = torch.cat([sel, torch.full((R, 1), E, dtype=torch.int32)], 1)
        w = torch.cat([w, torch.ones((R, 1))], 1)
    return sel.to(DEV).contiguous(), w.float().to(DEV).contiguous()


def test_grouping_order():
    from oracle import exl3 as ref
    from tensorfold_b200.exl3 import experts

    E, R, k = 24, 40, 6
    ex, _ = _layer(E, 128, 128, [(4, 4, 4)] * E, 0, 3)
    g = torch.Generator().manual_seed(5)
    sel, _ = _picks(E, R, k, g, shared=True)
    s = experts.Scratch(ex, R, k + 1)
    experts.group(sel, s, R, E)
    uids, members = ref.group(sel.cpu().numpy(), E)
    n = int(s.count[0])
    ids, mem = s.window(R)
    assert n == len(uids) and ids[:n].tolist() == uids.tolist()
    assert np.array_equal(mem[:n].cpu().numpy(), members)


MIXED = [
    (2, lambda e: (4 + 2 * (e % 3), 4 + 2 * (e % 3), 4 + 2 * ((e + 1) % 3))),
    (2, lambda e: ((2, 3, 5, 6, 7, 8, 10, 12, 14, 16)[e % 10],) * 2 + ((3, 5, 7, 8, 16)[e % 5],)),
    (1, lambda e: ((2, 4, 6, 8, 10, 12, 14, 16)[e % 8],) * 2 + ((4, 6, 8)[e % 3],)),
    (0, lambda e: ((2, 4, 6, 8, 10, 12, 14, 16)[(e + 3) % 8],) * 2 + ((8, 6, 16)[e % 3],)),
]


@pytest.mark.parametrize("cb,kfun", MIXED, ids=[f"cb{m[0]}_{i}" for i, m in enumerate(MIXED)])
def test_mixed_width_rows_are_independent_and_match_float64(cb, kfun, pdl):
    """A width per expert matrix: each row gives identical bits alone and inside windows of 1..128 rows, and the
    layer agrees with the float64 reference (the bar of tests/cuda/test_exl3_experts.py:181-205: 1e-2 of the max)."""

    from oracle import exl3 as ref
    from tensorfold_b200 import _lib
    from tensorfold_b200.exl3 import experts

    E, D, I, TOPK = 24, 512, 256, 6
    ex, mats = _layer(E, D, I, [kfun(e) for e in range(E)], cb, seed=11 + cb)
    g = torch.Generator().manual_seed(3)
    ROWS = 128
    x = torch.randn((ROWS, D), generator=g).to(torch.bfloat16).to(DEV)
    sel, w = _picks(E, ROWS, TOPK, g, shared=True)
    scratch = experts.Scratch(ex, ROWS, TOPK + 1)

    def run(rows):
        out = experts.routed(x[rows], sel[rows].contiguous(), w[rows].contiguous(), ex, scratch, None, len(rows))
        return out.clone()

    full = run(list(range(ROWS)))
    torch.cuda.synchronize()
    assert _lib.kernel_status() == 0
    assert torch.isfinite(full).all()
    for n in (1, 2, 3, 16, 17, 64, 128):
        for start in (0, ROWS - n):
            rows = list(range(start, start + n))
            assert torch.equal(run(rows), full[rows]), (n, start)
    mats_np = [[(t.cpu().numpy(), a.cpu().numpy(), b.cpu().numpy()) for t, a, b in m] for m in mats]
    want = ref.routed(x[:4].float().cpu().numpy(), sel[:4].cpu().numpy(), w[:4].cpu().numpy(), *mats_np, cb)
    err = np.abs(full[:4].double().cpu().numpy() - want).max() / np.abs(want).max()
    assert err < 1e-2, err


def test_per_slot_output_and_fused_combine_agree():
    from tensorfold_b200.exl3 import experts

    E, D, I, TOPK, R = 12, 256, 128, 4, 9
    ex, _ = _layer(E, D, I, [(8, 8, 8)] * E, 0, 21)
    g = torch.Generator().manual_seed(8)
    x = torch.randn((R, D), generator=g).to(torch.bfloat16).to(DEV)
    sel, w = _picks(E, R, TOPK, g)
    s = experts.Scratch(ex, R, TOPK)
    y = experts.routed(x, sel, None, ex, s, None, R).clone().view(R, TOPK, D)
    out = experts.routed(x, sel, w, ex, s, None, R)
    acc = torch.zeros((R, D), dtype=torch.float32, device=DEV)
    for k in range(TOPK):
        acc = torch.addcmul(acc, w[:, k:k + 1], y[:, k])          # not fused: compare with a tolerance
    assert torch.allclose(out, acc, rtol=1e-5, atol=1e-6)
    assert torch.equal(s.y[:R * TOPK].view(R, TOPK, D), y)         # the fused launch stores the same per-slot y


@pytest.mark.parametrize("widths", [lambda e: (8, 8, 4), lambda e: ((4, 16, 7)[e % 3], (5, 8)[e % 2], (2, 9, 12, 6)[e % 4])],
                         ids=["one_width", "mixed_widths"])
def test_grouping_ahead_of_the_call_gives_the_same_rows(widths):
    """``group`` then ``routed(group_first=False)`` (the caller grouped already) equals the call that groups itself.
    With mixed widths the self-grouping call also runs its items width by width (the other does not): same bits, and
    the three width-ordered tables are the items, each once, widest first."""

    from tensorfold_b200.exl3 import experts

    E, D, I, TOPK, R = 10, 256, 128, 3, 37
    ex, _ = _layer(E, D, I, [widths(e) for e in range(E)], 0, 27)
    assert ex.mixed == (widths(0) != widths(1))
    g = torch.Generator().manual_seed(12)
    x = torch.randn((R, D), generator=g).to(torch.bfloat16).to(DEV)
    sel, w = _picks(E, R, TOPK, g, shared=True)
    s = experts.Scratch(ex, R, TOPK + 1)
    want = experts.routed(x, sel, w, ex, s, None, R).clone()
    s2 = experts.Scratch(ex, R, TOPK + 1)
    experts.group(sel, s2, R, E)
    got = experts.routed(x, sel, w, ex, s2, None, R, group_first=False)
    assert torch.equal(got, want)
    assert int(s2.count[0]) == int(s.count[0]) == len(set(sel[:, :TOPK].reshape(-1).tolist()))
    if ex.mixed:
        n = int(s.sort_counts[0])
        items = s.sort_items[:n].cpu()
        for m, k2 in enumerate((ex.gate_k2, ex.up_k2, ex.down_k2)):
            table = s.by_width[m, :n].cpu()
            assert sorted(table[:, 3].tolist()) == list(range(n))                  # every item once
            assert torch.equal(table[:, :3], items[table[:, 3].long()])             # with its own three fields
            seen = k2.cpu()[table[:, 0].long()].tolist()
            assert seen == sorted(seen, reverse=True)                               # widest first


def test_graph_replay_equals_eager(pdl):
    from tensorfold_b200.exl3 import experts

    E, D, I, TOPK = 16, 256, 128, 4
    ex, _ = _layer(E, D, I, [(4 + 2 * (e % 3), 6, 8) for e in range(E)], 1, 33)
    g = torch.Generator().manual_seed(9)
    for R in (1, 4):
        x = torch.randn((R, D), generator=g).to(torch.bfloat16).to(DEV)
        sel, w = _picks(E, R, TOPK, g)
        s = experts.Scratch(ex, R, TOPK)
        out = torch.empty((R, D), dtype=torch.float32, device=DEV)
        experts.routed(x, sel, w, ex, s, out, R)
        eager = out.clone()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            experts.routed(x, sel, w, ex, s, out, R)
        out.zero_()
        graph.replay()
        assert torch.equal(out, eager)
        sel2, w2 = _picks(E, R, TOPK, g)
        sel.copy_(sel2)
        w.copy_(w2)
        graph.replay()
        want = experts.routed(x, sel, w, ex, experts.Scratch(ex, R, TOPK), None, R)
        assert torch.equal(out, want)


@pytest.mark.parametrize("bits,cb", [(4, "3inst"), (2, "mcg"), (6, "3inst"), (3.5, "mul1")])
@pytest.mark.parametrize("m", [1, 9, 128])
def test_dense_linear_against_float64_and_rows_alone(bits, cb, m):
    """``exl3.linear.Exl3Linear`` (the experts' kernels on a one-matrix layer): output against the float64 restatement
    of the reference's forward, W_q bit for bit, a row alone gives the same bits."""

    from oracle import exl3 as ref
    from tensorfold_b200.exl3 import linear

    k, n = 256, 384
    g = torch.Generator(device="cuda").manual_seed(int(bits * 10) + m)
    trellis = torch.randint(-32768, 32768, (k // 16, n // 16, int(16 * bits)), generator=g, device="cuda",
                            dtype=torch.int32).to(torch.int16)
    sign = lambda c: (torch.randint(0, 2, (c,), generator=g, device="cuda").float() * 2 - 1)          # noqa: E731
    suh = (sign(k) * (torch.randn((k,), generator=g, device="cuda") * 0.02).abs()).half()
    svh = (sign(n) * (torch.randn((n,), generator=g, device="cuda") * 0.02).abs()).half()
    bias = (torch.randn((n,), generator=g, device="cuda") * 0.01).half()
    layer = linear.Exl3Linear.from_tensors(trellis, suh, svh, cb, bias)
    assert layer.k == k and layer.n == n and layer.k2 == int(2 * bits)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    got = layer(x, out_dtype=torch.float32)
    cbid = linear.CODEBOOK_IDS[cb]
    want = ref.linear(x.double().cpu().numpy(), trellis.cpu().numpy(), suh.cpu().numpy(), svh.cpu().numpy(), cbid)
    want = want + bias.double().cpu().numpy()
    err = np.abs(got.double().cpu().numpy() - want).max() / np.abs(want).max()
    assert err < 2e-3, err
    assert np.array_equal(layer.unpack().cpu().numpy().view(np.uint16),
                          ref.unpack(trellis.cpu().numpy(), cbid).astype(np.float16).view(np.uint16))
    r = m // 2
    assert torch.equal(layer(x[r:r + 1], out_dtype=torch.float32), got[r:r + 1])
    with pytest.raises(ValueError):
        layer(torch.zeros((129, k), dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("bits,cb,bias", [(4, "3inst", True), (2.5, "mul1", False), (5, "mcg", True)])
@pytest.mark.parametrize("m,odt", [(129, torch.float32), (700, torch.bfloat16)])
def test_prompt_matmul_against_float64_and_the_decode_form(bits, cb, bias, m, odt):
    """``exl3.prefill.matmul`` (W_q decoded once, dense GEMM, this library's rotations): against the float64
    restatement of the reference's forward (the bar of its prompt path, tests/cuda/test_exl3_prefill.py: 2e-3 of the
    max), rows in a strided output, a row's value independent of the rows beside it up to the GEMM's tiling (1e-3),
    and agreement with the decode form on the rows that one takes."""

    from oracle import exl3 as ref
    from tensorfold_b200.exl3 import linear, prefill

    k, n = 384, 256
    g = torch.Generator(device="cuda").manual_seed(int(bits * 10) + m)
    trellis = torch.randint(-32768, 32768, (k // 16, n // 16, int(16 * bits)), generator=g, device="cuda",
                            dtype=torch.int32).to(torch.int16)
    sign = lambda c: (torch.randint(0, 2, (c,), generator=g, device="cuda").float() * 2 - 1)          # noqa: E731
    suh = (sign(k) * (torch.randn((k,), generator=g, device="cuda") * 0.02).abs()).half()
    svh = (sign(n) * (torch.randn((n,), generator=g, device="cuda") * 0.02).abs()).half()
    b = (torch.randn((n,), generator=g, device="cuda") * 0.01).half() if bias else None
    layer = linear.Exl3Linear.from_tensors(trellis, suh, svh, cb, b)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    ws = prefill.Workspace()
    wide = torch.full((m, n + 64), 7.0, dtype=odt, device="cuda")
    out = prefill.matmul(layer, x, wide[:, :n], ws)
    assert out.data_ptr() == wide.data_ptr() and bool((wide[:, n:] == 7.0).all())
    want = ref.linear(x[:40].double().cpu().numpy(), trellis.cpu().numpy(), suh.cpu().numpy(), svh.cpu().numpy(),
                      linear.CODEBOOK_IDS[cb])
    if bias:
        want = want + b.double().cpu().numpy()
    tol = 2e-3 if odt == torch.float32 else 1e-2
    err = np.abs(out[:40].double().cpu().numpy() - want).max() / np.abs(want).max()
    assert err < tol, err
    small = torch.empty((40, n), dtype=odt, device="cuda")
    prefill.matmul(layer, x[:40], small, ws)                       # the workspace is reused, fewer rows
    scale = float(out[:40].float().abs().max())
    assert float((small.float() - out[:40].float()).abs().max()) <= (1e-3 if odt == torch.float32 else 1e-2) * scale
    dec = layer(x[:40], out_dtype=torch.float32)
    assert float((dec - out[:40].float()).abs().max()) <= tol * scale
    assert ws.nbytes() >= k * n * 2 + m * k * 2 + m * n * 4
    with pytest.raises(ValueError):
        prefill.matmul(layer, x, torch.empty((m, n + 1), device="cuda"), ws)


@pytest.mark.parametrize("R", [1, 37])
def test_blocks_of_two_or_four_column_tiles_give_the_same_bits(R, monkeypatch):
    """The trellis kernel's thread blocks take four 16-column tiles, or two where a launch of 4.00-bit tensors would
    leave SMs idle: the choice is the host's (a function of the call's shape) and no bit depends on it."""

    from tensorfold_b200.exl3 import experts

    E, D, I, TOPK = 10, 256, 384, 3
    ex, _ = _layer(E, D, I, [(8, 8, 8)] * E, 0, 31)
    g = torch.Generator().manual_seed(14)
    x = torch.randn((R, D), generator=g).to(torch.bfloat16).to(DEV)
    sel, w = _picks(E, R, TOPK, g)
    outs = []
    for tiles in (4, 2):
        monkeypatch.setattr(experts, "col_tiles", lambda *a, tiles=tiles, **k: tiles)
        s = experts.Scratch(ex, R, TOPK)
        outs.append((experts.routed(x, sel, w, ex, s, None, R).clone(), s.y[:R * TOPK].clone()))
    torch.cuda.synchronize()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert bool(torch.isfinite(outs[0][0]).all()) and float(outs[0][0].abs().max()) > 0


@pytest.mark.parametrize("R", [1, 37, 200])
def test_the_short_loop_build_for_mixed_widths_gives_the_same_bits(R, monkeypatch):
    """A projection whose tensors differ in width runs the kernel's build with short loops (blocks of different widths
    then share an SM's instruction cache); the all-widths build with unrolled loops gives the same bits."""

    from tensorfold_b200.exl3 import experts

    E, D, I, TOPK = 12, 256, 384, 3
    ex, _ = _layer(E, D, I, [((2, 16, 7)[e % 3], (5, 3, 8)[e % 3], (4, 9, 12, 6)[e % 4]) for e in range(E)], 0, 33)
    assert ex.mixed
    g = torch.Generator().manual_seed(15)
    x = torch.randn((R, D), generator=g).to(torch.bfloat16).to(DEV)
    sel, w = _picks(E, R, TOPK, g)
    outs = []
    for compact in (True, False):
        monkeypatch.setattr(experts, "COMPACT_MIXED", compact)
        s = experts.Scratch(ex, R, TOPK)
        outs.append((experts.routed(x, sel, w, ex, s, None, R).clone(), s.y[:R * TOPK].clone()))
    torch.cuda.synchronize()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert bool(torch.isfinite(outs[0][0]).all()) and float(outs[0][0].abs().max()) > 0
