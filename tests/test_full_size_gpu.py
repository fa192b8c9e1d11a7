"""BASELINE-size cases on the GPU: config 2 (affine, 64 tokens and a 2048-token prompt) against the CPU oracle, and
config 3 (EXL3 4.00 bpw) against float64 for a few rows plus the size-independent properties (a row's bits do not
depend on its window; routing equals the sorted order)."""

import numpy as np
import pytest
import torch

from helpers import bits, rel_l2, triple_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def c2():
    from tensorfold_b200 import experts, moe, synthetic

    shape = synthetic.C2
    gate, up, down = synthetic.affine_layer(shape, DEV)
    rt = synthetic.router_rows(shape, DEV)
    layer = moe.Routed(rt, experts.make([gate, up], down, 64), shape.top_k, shared=False)
    return shape, layer, (gate, up, down), rt


def test_config2_decode_64_tokens_against_the_cpu_oracle(c2):
    from oracle import affine, cpu
    from tensorfold_b200 import moe, synthetic

    shape, layer, (gate, up, down), rt = c2
    x = synthetic.activations(shape, 64, DEV)
    buf = moe.MoEBuffers(64, moe._Shape(layer), DEV, shared=False)
    moe.moe(x, layer.router, layer.experts, buf, layer.top_k, layer.count)
    out = moe.combine(buf.y, buf.wts)
    o_cpu, pick, wts, act, y = cpu.moe_layer(bits(x), bits(rt), shape.experts, shape.top_k, False, triple_np(gate),
                                             triple_np(up), triple_np(down), 64, True, want_parts=True)
    assert np.array_equal(buf.pick.cpu().numpy(), pick)                          # routing indices: bit exact
    logits = buf.logits.cpu().numpy()
    for r in range(64):
        assert pick[r].tolist() == sorted(range(shape.experts), key=lambda i: (-logits[r, i], i))[:shape.top_k]
    margin = np.sort(logits, axis=1)[:, -shape.top_k] - np.sort(logits, axis=1)[:, -shape.top_k - 1]
    assert margin.min() > 0                                                      # no tie decided the selection
    assert np.abs(buf.wts.cpu().numpy() - wts).max() <= 2 ** -8
    assert rel_l2(out.float().cpu().numpy(), affine.bf16_value(o_cpu)) <= 1e-2
    assert rel_l2(buf.y.view(-1, shape.dims).cpu().numpy(), y) <= 1e-3
    one = moe.run(x[17:18], layer)                                               # a row alone gives the same bits
    assert torch.equal(one, out[17:18])


def test_config2_prompt_2048_tokens_properties(c2):
    from oracle import cpu
    from tensorfold_b200 import moe, synthetic

    shape, layer, (gate, up, down), rt = c2
    x = synthetic.activations(shape, 2048, DEV, index=5)
    out = moe.run(x, layer, prefill=True)
    dec = moe.run(x[:96], layer)                                                  # decode form: same tolerance class
    assert rel_l2(out[:96].float().cpu().numpy(), dec.float().cpu().numpy()) <= 1e-2
    part = moe.run(x[100:400], layer, prefill=True)                               # chunk invariance at full size
    assert torch.equal(part, out[100:400])
    o_cpu = cpu.moe_layer(bits(x[:32]), bits(rt), shape.experts, shape.top_k, False, triple_np(gate), triple_np(up),
                          triple_np(down), 64, True)
    from oracle import affine

    assert rel_l2(out[:32].float().cpu().numpy(), affine.bf16_value(o_cpu)) <= 1e-2


def test_config3_exl3_layer_rows_and_float64():
    from oracle import exl3 as ref
    from tensorfold_b200 import moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape = synthetic.C3
    gate, up, down = synthetic.exl3_layer(shape, DEV, 4)
    ex = x3.prepare(gate, up, down, x3.CB_3INST, device=DEV)
    rt = synthetic.router_rows(shape, DEV)
    rows = 64
    x = synthetic.activations(shape, rows, DEV)

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    buf = moe.MoEBuffers(rows, _Cfg, DEV, shared=False)
    moe.router(x, rt, buf.logits)
    moe.select_rows(buf.logits, buf, shape.top_k, shape.experts)
    s = x3.Scratch(ex, rows, shape.top_k)
    full = x3.routed(x, buf.pick, buf.wts, ex, s, None, rows).clone()
    assert torch.isfinite(full).all()
    for a, b in ((0, 1), (63, 64), (5, 22)):
        got = x3.routed(x[a:b], buf.pick[a:b].contiguous(), buf.wts[a:b].contiguous(), ex, s, None, b - a)
        assert torch.equal(got, full[a:b])
    pick, wts = buf.pick[:2].cpu().numpy(), buf.wts[:2].cpu().numpy()
    used = sorted(set(pick.reshape(-1).tolist()))
    mats = [[None] * shape.experts for _ in range(3)]
    for e in used:
        for m, src in enumerate((gate, up, down)):
            mats[m][e] = tuple(t.cpu().numpy() for t in src[e])
    want = ref.routed(x[:2].float().cpu().numpy(), pick, wts, *mats, ref.CB_3INST)
    err = np.abs(full[:2].double().cpu().numpy() - want).max() / np.abs(want).max()
    assert err < 1e-2, err
