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


def test_config2_decode_64_tokens_against_the_cpu_oracle(c2, pdl):
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


def test_config1_one_token_against_the_cpu_oracle(pdl):
    """Config 1: the full-size layer on ONE token, its own seeded weights, against the CPU restatement of the
    reference's affine-row arithmetic and the float64 layer; the same token inside a 64-token call gives the same bits."""

    from oracle import affine, cpu
    from tensorfold_b200 import experts, moe, synthetic

    shape = synthetic.C1
    gate, up, down = synthetic.affine_layer(shape, DEV)
    rt = synthetic.router_rows(shape, DEV)
    layer = moe.Routed(rt, experts.make([gate, up], down, 64), shape.top_k, shared=False)
    x = synthetic.activations(shape, 64, DEV)
    buf = moe.MoEBuffers(1, moe._Shape(layer), DEV, shared=False)
    moe.moe(x[:1], layer.router, layer.experts, buf, layer.top_k, layer.count)
    out = moe.combine(buf.y, buf.wts)
    o_cpu, pick, wts, act, y = cpu.moe_layer(bits(x[:1]), bits(rt), shape.experts, shape.top_k, False, triple_np(gate),
                                             triple_np(up), triple_np(down), 64, True, want_parts=True)
    assert np.array_equal(buf.pick.cpu().numpy(), pick)
    logits = buf.logits.cpu().numpy()[0]
    assert pick[0].tolist() == sorted(range(shape.experts), key=lambda i: (-logits[i], i))[:shape.top_k]
    assert np.abs(buf.wts.cpu().numpy() - wts).max() <= 2 ** -8
    assert rel_l2(out.float().cpu().numpy(), affine.bf16_value(o_cpu)) <= 1e-2
    assert rel_l2(buf.y.view(-1, shape.dims).cpu().numpy(), y) <= 1e-3
    used = sorted(set(pick.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    sub = lambda m: tuple(t[used].contiguous() for t in m)                         # noqa: E731
    pk = np.vectorize(remap.get)(pick).astype(np.int32)
    _, _, o64 = affine.layer64(bits(x[:1]), pk, wts, triple_np(sub(gate)), triple_np(sub(up)), triple_np(sub(down)),
                               64, True)
    assert rel_l2(out.float().cpu().numpy(), o64) <= 1e-2
    assert torch.equal(moe.run(x, layer)[:1], out)                               # the batch does not change its bits


def test_config2_prompt_2048_tokens_properties(c2, pdl):
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


def test_config3_exl3_layer_rows_and_float64(pdl):
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
    sel = [0, 21, 42, 63]
    pick, wts = buf.pick[sel].cpu().numpy(), buf.wts[sel].cpu().numpy()
    used = sorted(set(pick.reshape(-1).tolist()))
    mats = [[None] * shape.experts for _ in range(3)]
    for e in used:
        for m, src in enumerate((gate, up, down)):
            mats[m][e] = tuple(t.cpu().numpy() for t in src[e])
    want = ref.routed(x[sel].float().cpu().numpy(), pick, wts, *mats, ref.CB_3INST)
    err = np.abs(full[sel].double().cpu().numpy() - want).max() / np.abs(want).max()
    assert err < 1e-2, err


def test_config4_large_experts_with_shared_expert_and_skewed_routing():
    """Config 4's layer (hidden 6144, 256 experts x FFN 2048, top-8 + a shared expert, 256 tokens, Zipf-skewed router)
    on one GPU: routing against the sorted order, a few rows against the CPU oracle, and row invariance."""

    from oracle import affine, cpu
    from tensorfold_b200 import experts, moe, synthetic

    shape = synthetic.C4
    gate, up, down = synthetic.affine_layer(shape, DEV)
    rt = synthetic.router_rows(shape, DEV)
    layer = moe.Routed(rt, experts.make([gate, up], down, 64), shape.top_k, shared=True)
    rows = 256
    x = synthetic.activations(shape, rows, DEV)
    buf = moe.MoEBuffers(rows, moe._Shape(layer), DEV, shared=True)
    moe.router(x, rt, buf.logits)
    buf.logits[:, :shape.experts] += synthetic.zipf_bias(shape, 1.1, DEV)          # uneven expert loads
    moe.select(buf.logits, buf, shape.top_k, shape.experts)
    ex = layer.experts
    experts.gate_up(x, ex, buf.plan, buf.act.view(-1, ex.width), rows)
    experts.down(buf.act.view(-1, ex.width), ex, buf.plan, buf.y.view(-1, ex.dims), rows)
    out = moe.combine(buf.y, buf.wts)
    logits = buf.logits.cpu().numpy()
    pick = buf.pick.cpu().numpy()
    for r in range(0, rows, 17):
        want = sorted(range(shape.experts), key=lambda i: (-logits[r, i], i))[:shape.top_k]
        assert pick[r, :shape.top_k].tolist() == want and pick[r, shape.top_k] == shape.experts
    counts = np.bincount(pick[:, :shape.top_k].reshape(-1), minlength=shape.experts)
    assert counts.max() > 8 * max(1, int(np.median(counts)))                       # the skew is real
    # three rows against the float64 reference over the experts they use
    sel = [0, 100, 255]
    used = sorted(set(pick[sel].reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    sub = lambda m: tuple(t[used].contiguous() for t in m)                         # noqa: E731
    pk = np.vectorize(remap.get)(pick[sel]).astype(np.int32)
    _, _, o64 = affine.layer64(bits(x[sel]), pk, buf.wts[sel].cpu().numpy(), triple_np(sub(gate)), triple_np(sub(up)),
                               triple_np(sub(down)), 64, True)
    assert rel_l2(out[sel].float().cpu().numpy(), o64) <= 1e-2
    # a row alone: same bits
    buf1 = moe.MoEBuffers(1, moe._Shape(layer), DEV, shared=True)
    buf1.logits.copy_(buf.logits[100:101])
    moe.select(buf1.logits, buf1, shape.top_k, shape.experts)
    experts.gate_up(x[100:101], ex, buf1.plan, buf1.act.view(-1, ex.width), 1)
    experts.down(buf1.act.view(-1, ex.width), ex, buf1.plan, buf1.y.view(-1, ex.dims), 1)
    assert torch.equal(moe.combine(buf1.y, buf1.wts), out[100:101])


def test_config5_mixed_width_exl3_stack():
    """Config 5 at full size: all eight layers (hidden 4096, 160 experts x FFN 1536, top-8, a seeded width of 2..8 bits
    per tensor) with a bf16 residual add between them, at every batch size of the sweep - 1, 8, 32, 128 and 512
    tokens: finite, a row's bits after eight layers do not depend on the batch it ran in, routing equals the sorted
    order, and layer one is within 1e-2 of float64 for two rows."""

    import random

    from oracle import exl3 as ref
    from tensorfold_b200 import _lib, moe, synthetic
    from tensorfold_b200.exl3 import experts as x3

    shape, depth = synthetic.C5, 8
    rng = random.Random(5005)
    widths = {}

    def bits_of(layer):
        return lambda e, m: widths.setdefault((layer, e, m), rng.choice((2, 3, 4, 5, 6, 7, 8)))

    layers, mats0 = [], None
    for li in range(depth):
        gate, up, down = synthetic.exl3_layer(shape, DEV, bits_of(li), copy=li)
        if li == 0:
            mats0 = (gate, up, down)
        layers.append((x3.prepare(gate, up, down, x3.CB_3INST, device=DEV),
                       synthetic.router_rows(shape, DEV)))
        del gate, up, down
    assert len({v for v in widths.values()}) == 7 and len(widths) == depth * shape.experts * 3

    class _Cfg:
        num_experts_per_tok, num_experts = shape.top_k, shape.experts
        moe_intermediate_size, hidden_size = shape.width, shape.dims

    def stack(h):
        rows = h.shape[0]
        first = None
        for ex, rt in layers:
            buf = moe.MoEBuffers(rows, _Cfg, DEV, shared=False)
            moe.router(h, rt, buf.logits)
            moe.select_rows(buf.logits, buf, shape.top_k, shape.experts)
            y = x3.routed(h, buf.pick, buf.wts, ex, x3.Scratch(ex, rows, shape.top_k), None, rows)
            if first is None:
                first = (y.clone(), buf.pick.clone(), buf.wts.clone(), buf.logits.clone())
            h = (h.float() + y).to(torch.bfloat16)                                 # residual add in bf16
        return h, first

    x = synthetic.activations(shape, 512, DEV)
    full, (y0, pick0, wts0, logits0) = stack(x)
    torch.cuda.synchronize()
    assert _lib.kernel_status() == 0
    assert torch.isfinite(full.float()).all()
    for rows in (1, 8, 32, 128):                                                   # the other batch sizes of the sweep
        part, _ = stack(x[:rows])
        assert torch.equal(part, full[:rows]), rows
    for a, b in ((3, 11), (511, 512)):                                             # and windows that do not start at 0
        part, _ = stack(x[a:b])
        assert torch.equal(part, full[a:b])
    lg = logits0.cpu().numpy()
    for r in range(0, 512, 37):
        want = sorted(range(shape.experts), key=lambda i: (-lg[r, i], i))[:shape.top_k]
        assert pick0[r].tolist() == want
    gate, up, down = mats0
    used = sorted(set(pick0[:2].reshape(-1).tolist()))
    mats = [[None] * shape.experts for _ in range(3)]
    for e in used:
        for m, src in enumerate((gate, up, down)):
            mats[m][e] = tuple(t.cpu().numpy() for t in src[e])
    want = ref.routed(x[:2].float().cpu().numpy(), pick0[:2].cpu().numpy(), wts0[:2].cpu().numpy(), *mats,
                      ref.CB_3INST)
    err = np.abs(y0[:2].double().cpu().numpy() - want).max() / np.abs(want).max()
    assert err < 1e-2, err
