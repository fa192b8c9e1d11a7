"""The EXL3 oracle restatement against fixtures made by the reference's own decoder (no GPU)."""

from pathlib import Path

import numpy as np
import pytest

from oracle import exl3
from oracle import exl3 as ref

GOLDEN = np.load(Path(__file__).parent / "golden" / "exl3_golden.npz")


def test_every_codebook_and_width_decodes_like_the_reference():
    seen = 0
    for key in GOLDEN.files:
        if key.startswith("t_cb"):
            cb = int(key[4])
            got = exl3.unpack(GOLDEN[key], cb)
            assert np.array_equal(got.view(np.uint16), GOLDEN["w" + key[1:]]), key
            seen += 1
    assert seen == 27                                    # 3inst and mcg at 8 widths, mul1 at 11


def test_codebook_spot_values():
    for cb in range(3):
        states = GOLDEN[f"cb{cb}_states"].astype(np.int64)
        assert np.array_equal(exl3.codebook(cb)[states].view(np.uint16), GOLDEN[f"cb{cb}_values"])


def test_rotated_forward():
    y = exl3.linear(GOLDEN["fwd_x"], GOLDEN["fwd_t"], GOLDEN["fwd_suh"].view(np.float16),
                    GOLDEN["fwd_svh"].view(np.float16), exl3.CB_MCG)
    assert np.allclose(y, GOLDEN["fwd_y"], rtol=1e-12, atol=1e-12)
    h = exl3.hadamard()
    assert np.allclose(h @ h, np.eye(128), atol=1e-12)


def test_window_ends_and_positions():
    for k2 in range(2, 17):
        e = exl3.window_end(np.arange(256), k2)
        assert e[-1] == 128 * k2 and np.all(np.diff(e) >= 1)
    rows, cols = exl3.tile_positions()
    assert sorted(zip(rows.tolist(), cols.tolist())) == [(r, c) for r in range(16) for c in range(16)]


def test_grouping_semantics():
    pick = np.array([[3, 1, 7], [1, 9, 3], [7, 7, 2]], dtype=np.int32)           # 9 is not a routed expert (E = 8)
    uids, members = exl3.group(pick, 8)
    assert uids.tolist() == [1, 2, 3, 7]
    assert members.tolist() == [[1, 32, -1], [66, -1, -1], [0, 34, -1], [2, 64, 65]]


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_c_restatement_decodes_like_the_numpy_one(cb):
    """``oracle/cpu_exl3.c`` (the timed CPU baseline of the EXL3 path) against the pinned numpy decoder, bit for bit,
    at every width."""

    from oracle import cpu

    rng = np.random.default_rng(17 + cb)
    for k2 in range(2, 17):
        t = rng.integers(-32768, 32768, (3, 2, 8 * k2)).astype(np.int16)
        assert np.array_equal(cpu.exl3_unpack(t, cb).view(np.uint16), ref.unpack(t, cb).view(np.uint16)), k2


def test_c_restatement_of_the_routed_layer():
    from oracle import cpu

    rng = np.random.default_rng(3)
    e_count, d, ni, rows, k = 6, 256, 128, 5, 3

    def mat(kk, nn, bits):
        return (rng.integers(-32768, 32768, (kk // 16, nn // 16, 16 * bits)).astype(np.int16),
                (rng.standard_normal(kk) * 0.05).astype(np.float16), rng.standard_normal(nn).astype(np.float16))

    gate = [mat(d, ni, 2 + e % 4) for e in range(e_count)]
    up = [mat(d, ni, 3 + e % 3) for e in range(e_count)]
    down = [mat(ni, d, 4) for e in range(e_count)]
    x = rng.standard_normal((rows, d)).astype(np.float32)
    pick = np.stack([rng.permutation(e_count + 1)[:k] for _ in range(rows)]).astype(np.int32)   # id 6 is skipped
    wts = rng.random((rows, k)).astype(np.float32)
    got = cpu.exl3_routed(x, pick, wts, gate, up, down, 0, d, ni)
    want = ref.routed(x, pick, wts, gate, up, down, 0)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
