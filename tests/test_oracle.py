"""The CPU oracle against the reference's own golden vectors and known-answer checks (no GPU)."""

import ctypes
from pathlib import Path

import numpy as np
import pytest

from oracle import affine, cpu

ROOT = Path(__file__).resolve().parent.parent


def test_code_extraction_known_answer():
    """The packed-code pattern of the reference's test (tests/test_affine_rows.py:104-111): values
    (29 i + i // 7) mod 16 packed little-endian read back, across word and group boundaries."""

    for group in (32, 64, 128):
        values = [(i * 29 + i // 7) % 16 for i in range(group * 3)]
        packed = sum(v << (4 * i) for i, v in enumerate(values))
        words = np.array([(packed >> (32 * i)) & 0xFFFFFFFF for i in range(len(values) // 8)], dtype=np.uint32)
        assert affine.codes(words).tolist() == values
        assert [cpu.lib().tfo_code_at(words.ctypes.data, i, 4) for i in range(len(values))] == values
        assert affine.pack_codes(np.array(values)).tolist() == words.tolist()


def test_code_extraction_matches_the_reference_header():
    """Against the reference's own header compiled as C++ (oracle/build_ref.py), when it has been built."""

    ref_path = ROOT / "oracle" / "_ref" / "libaffine_header.so"
    if not ref_path.exists():
        from oracle import build_ref

        if build_ref.build() is None:
            pytest.skip("the reference tree is not mounted and no prebuilt header library exists")
    ref = ctypes.CDLL(str(ref_path))
    ref.decode.restype = ctypes.c_uint32
    ref.decode.argtypes = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int)
    rng = np.random.default_rng(7)
    words = rng.integers(0, 2 ** 32, size=64, dtype=np.uint64).astype(np.uint32)
    q = affine.codes(words)
    for i in range(words.size * 8):
        assert ref.decode(words.ctypes.data, i, 4) == q[i] == cpu.lib().tfo_code_at(words.ctypes.data, i, 4)


def want_plan(picks, e, tile):
    """The pure-Python plan of the reference's test (semantics of tests/cuda/test_experts.py:107-115)."""

    flat = picks.reshape(-1).tolist()
    items, members = [], []
    for ex in range(e):
        pairs = [p for p, v in enumerate(flat) if v == ex]
        for j in range(0, len(pairs), tile):
            items.append([ex, len(members) + j, min(tile, len(pairs) - j)])
        members += pairs
    return items, members, len(set(flat))


@pytest.mark.parametrize("rows,tile", [(23, 16), (23, 64), (300, 16), (300, 64), (1500, 64), (1500, 16)])
def test_plan_golden(rows, tile):
    slots, e = 7, 50
    rng = np.random.default_rng(9)
    picks = np.stack([rng.permutation(e)[:slots] for _ in range(rows)]).astype(np.int32)
    picks[:, 0] = 3
    items, members, counts = cpu.plan(picks, e, tile)
    wi, wm, distinct = want_plan(picks, e, tile)
    assert items.tolist() == wi and members.tolist() == wm and counts.tolist() == [len(wi), distinct]


def test_many_rows_on_one_expert_make_items_of_16_16_5():
    picks = np.full((37, 1), 2, dtype=np.int32)
    items, members, counts = cpu.plan(picks, 4, 16)
    assert items.tolist() == [[2, 0, 16], [2, 16, 16], [2, 32, 5]] and members.tolist() == list(range(37))


def test_topk_indices_are_the_sorted_order_and_weights_renormalise():
    rng = np.random.default_rng(3)
    t, e, k = 40, 64, 10
    logits = rng.standard_normal((t, e + 1)).astype(np.float32)
    logits[5, :] = 0.0                                              # ties: the lower ids win
    logits[6, 10:20] = 1.5
    pick, wts = cpu.topk_rows(logits, e, k, True)
    for r in range(t):
        want = sorted(range(e), key=lambda i: (-logits[r, i], i))[:k]
        assert pick[r, :k].tolist() == want
        ex = np.exp((logits[r, want] - logits[r, want[0]]).astype(np.float64))
        assert np.abs(wts[r, :k] - ex / ex.sum()).max() < 2 ** -8
        assert pick[r, k] == e
        assert abs(wts[r, k] - 1 / (1 + np.exp(-float(affine.round_bf16(logits[r, e:e + 1])[0])))) < 2 ** -8
    assert pick[5, :k].tolist() == list(range(k))
    assert np.array_equal(affine.round_bf16(wts), wts)
    pick2, wts2 = cpu.topk_rows(logits, e, k, False)
    assert np.array_equal(pick2, pick[:, :k]) and np.array_equal(wts2, wts[:, :k])


def test_router_logits_follow_the_stated_order():
    """The C restatement against a numpy one of the same order, bit for bit, and against float64 within rounding."""

    rng = np.random.default_rng(5)
    t, d, ne = 7, 768, 13
    x = affine.bf16_bits(rng.standard_normal((t, d)).astype(np.float32))
    w = affine.bf16_bits((rng.standard_normal((ne, d)) * 0.02).astype(np.float32))
    got = cpu.router_logits(x, w)
    xv, wv = affine.bf16_value(x), affine.bf16_value(w)
    pad = (-d) % 256
    xp = np.pad(xv, ((0, 0), (0, pad))).reshape(t, -1, 32, 8)
    wp = np.pad(wv, ((0, 0), (0, pad))).reshape(ne, -1, 32, 8)
    acc = np.zeros((t, ne, 32), dtype=np.float32)
    for c in range(xp.shape[1]):
        for j in range(8):
            acc = acc + xp[:, None, c, :, j] * wp[None, :, c, :, j]       # the product is exact in fp32
    lanes = np.arange(32)
    for m in (16, 8, 4, 2, 1):
        acc = acc + acc[..., lanes ^ m]
    assert np.array_equal(got, acc[..., 0])
    assert np.abs(got - xv.astype(np.float64) @ wv.astype(np.float64).T).max() < 1e-5


def _matrix(rng, e, n, k, fp16):
    words = rng.integers(0, 2 ** 32, size=(e, n, k // 8), dtype=np.uint64).astype(np.uint32)
    s = np.abs(rng.standard_normal((e, n, k // 64)) * 0.01).astype(np.float32)
    b = (rng.standard_normal((e, n, k // 64)) * 0.01).astype(np.float32)
    if fp16:
        return words, s.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16)
    return words, affine.bf16_bits(s), affine.bf16_bits(b)


@pytest.mark.parametrize("fp16", [False, True])
def test_dequantised_weights(fp16):
    rng = np.random.default_rng(11)
    words, s, b = _matrix(rng, 2, 32, 192, fp16)
    exact = affine.dequant64(words, s, b, 64, fp16)
    dec = cpu.dequant(words, s, b, 64, fp16, False)
    assert np.array_equal(dec, exact.astype(np.float32))                       # one rounding of the exact value
    pre = cpu.dequant(words, s, b, 64, fp16, True)
    assert np.array_equal(affine.round_bf16(pre), pre)
    if fp16:
        assert np.array_equal(pre, affine.round_bf16(dec))
    else:
        import torch

        # a bf16 fma: torch computes q * s + b in double here, and double -> bf16 needs care, so check neighbours
        assert np.abs(pre.astype(np.float64) - exact).max() <= np.abs(exact).max() * 2 ** -8
        lo = torch.from_numpy(exact).to(torch.float32).to(torch.bfloat16).float().numpy()
        assert (pre != lo).mean() < 1e-3                                       # they differ only at double roundings


def test_affine_rows_track_float64_and_share_one_row_arithmetic():
    rng = np.random.default_rng(13)
    n, k = 64, 768
    words, s, b = _matrix(rng, 1, n, k, True)
    x = affine.bf16_bits(rng.standard_normal((5, k)).astype(np.float32))
    got = cpu.affine_rows(x, words[0], s[0], b[0], 64, True, out_bf16=False)
    want = affine.bf16_value(x).astype(np.float64) @ affine.dequant64(words[0], s[0], b[0], 64, True).T
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    alone = np.concatenate([cpu.affine_rows(x[r:r + 1], words[0], s[0], b[0], 64, True, out_bf16=False)
                            for r in range(5)])
    assert np.array_equal(alone, got)                                          # a row's bits ignore the other rows


@pytest.mark.parametrize("shared", [False, True])
def test_cpu_layer_tracks_the_float64_layer(shared):
    rng = np.random.default_rng(17)
    t, d, e, ni, k = 9, 256, 12, 128, 4
    ne = e + (1 if shared else 0)
    gate, up, down = _matrix(rng, ne, ni, d, True), _matrix(rng, ne, ni, d, True), _matrix(rng, ne, d, ni, True)
    x = affine.bf16_bits(rng.standard_normal((t, d)).astype(np.float32))
    rt = affine.bf16_bits((rng.standard_normal((ne, d)) * 0.02).astype(np.float32))
    out, pick, wts, act, y = cpu.moe_layer(x, rt, e, k, shared, gate, up, down, 64, True, want_parts=True)
    a64, y64, o64 = affine.layer64(x, pick, wts, gate, up, down, 64, True)
    assert np.abs(affine.bf16_value(act) - a64).max() <= 2 ** -6 * np.abs(a64).max()
    assert np.abs(y - y64).max() <= 2e-2 * np.abs(y64).max()
    err = np.linalg.norm(affine.bf16_value(out) - o64) / np.linalg.norm(o64)
    assert err < 1e-2


def test_sigmoid_router_restatement_orders_by_choice_then_id():
    from oracle import routers

    rng = np.random.default_rng(3)
    logits = rng.standard_normal((6, 20)).astype(np.float32)
    logits[2, :] = 0.5
    bias = np.zeros((20,), dtype=np.float32)
    pick, wts, gap = routers.sigmoid_topk(logits, bias, 4, 1.0, True, 1)
    assert pick[2, :4].tolist() == [0, 1, 2, 3] and pick[:, 4].tolist() == [20] * 6
    np.testing.assert_allclose(wts[:, :4].sum(-1), 1.0, rtol=1e-6)
    for r in (0, 1, 3):
        assert pick[r, :4].tolist() == np.argsort(-logits[r], kind="stable")[:4].tolist()   # sigmoid is monotone
    assert gap[2] == 0.0 and (wts[:, 4] == 1.0).all()


def test_item_bound_holds_for_every_split_of_the_pairs():
    """``max_items`` (what sizes the plan tables and the grids): never below the items a plan makes, for any way the
    pairs fall on the experts, and exact for one expert."""

    import random

    from tensorfold_b200 import experts
    from tensorfold_b200.exl3 import experts as x3

    rnd = random.Random(7)
    for _ in range(4000):
        e, p, tile = rnd.randint(1, 12), rnd.randint(0, 70), rnd.choice([8, 16, 192])
        counts = [0] * e
        for _ in range(p):
            counts[rnd.randrange(e) if rnd.random() < 0.7 else 0] += 1
        made = sum((c + tile - 1) // tile for c in counts)
        assert made <= experts.max_items(p, e, tile) <= min(p, e) + p // tile
        assert sum((c + 15) // 16 for c in counts) <= x3.max_items(p, e)
    assert experts.max_items(17, 1, 8) == 3 and experts.max_items(16, 1, 8) == 2 and experts.max_items(0, 5, 8) == 0
