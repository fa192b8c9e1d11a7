"""The checkpoint reader (``tensorfold_b200.load``): container parsing on CPU, and on the GPU layers built from a
written checkpoint equal layers built from the tensors directly."""

import numpy as np
import pytest
import torch


def _save(path, tensors):
    from safetensors.torch import save_file

    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path))


def test_container_round_trip_and_helpers(tmp_path):
    from tensorfold_b200 import load

    g = torch.Generator().manual_seed(1)
    tensors = {
        "a.weight": torch.randint(-2 ** 31, 2 ** 31 - 1, (6, 40), generator=g, dtype=torch.int64).to(torch.int32),
        "a.scales": torch.randn((6, 5), generator=g).to(torch.bfloat16),
        "b.trellis": torch.randint(-32768, 32767, (8, 8, 64), generator=g, dtype=torch.int32).to(torch.int16),
        "b.suh": torch.randn((128,), generator=g).half(),
        "b.mcg": torch.zeros((1,), dtype=torch.int32),
        "c": torch.randn((3, 7), generator=g),
    }
    _save(tmp_path / "model-00001.safetensors", {k: v for k, v in tensors.items() if not k.startswith("c")})
    _save(tmp_path / "model-00002.safetensors", {"c": tensors["c"]})
    ck = load.Checkpoint(tmp_path)
    assert ck.names() == sorted(tensors) and ck.has("c") and not ck.has("d")
    for name, t in tensors.items():
        got = ck.get(name)
        assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape)
        assert torch.equal(got.view(torch.uint8), t.contiguous().view(torch.uint8))
    f, b, e, dtype, shape = ck.entry("b.trellis")
    assert f.name == "model-00001.safetensors" and e - b == 8 * 8 * 64 * 2 and dtype == "I16" and shape == [8, 8, 64]
    assert ck.codebook("b") == "mcg" and ck.codebook("a") == "3inst"
    with pytest.raises(KeyError):
        ck.get("nope")
    one = load.Checkpoint(tmp_path / "model-00002.safetensors")
    assert one.names() == ["c"]
    # sign words: bit b of word w set -> element 16 w + b is -1
    packed = torch.tensor([0b101, -32768], dtype=torch.int16)
    signs = load.unpack_signs(packed)
    want = np.ones(32, dtype=np.float16)
    want[[0, 2, 31]] = -1
    assert signs.dtype == torch.float16 and np.array_equal(signs.numpy(), want)
    # affine dequantisation against the nibble definition
    words = tensors["a.weight"][:, :8]
    scales = torch.rand((6, 1), generator=g).to(torch.bfloat16)
    biases = torch.randn((6, 1), generator=g).to(torch.bfloat16)
    w = load.dequantize(words, scales, biases, 64)
    u = words.numpy().view(np.uint32)
    q = np.stack([(u >> (4 * i)) & 15 for i in range(8)], -1).reshape(6, 64).astype(np.float32)
    assert np.array_equal(w.numpy(), q * scales.float().numpy() + biases.float().numpy())


@pytest.mark.gpu
def test_affine_layer_from_a_checkpoint_equals_the_layer_from_tensors(tmp_path):
    from tensorfold_b200 import experts, load, moe, synthetic

    dev = torch.device("cuda", 0)
    shape = synthetic.SMALL_SHARED
    gate, up, down = synthetic.affine_layer(shape, dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(7)
    e1 = shape.experts + 1

    def q4(rows, k):
        words = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, k // 8), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
        return words, (torch.rand((rows, k // 64), generator=g, device=dev) * 0.01).to(torch.bfloat16), \
            (torch.randn((rows, k // 64), generator=g, device=dev) * 0.05).to(torch.bfloat16)

    rg, rs = q4(shape.experts, shape.dims), q4(1, shape.dims)
    tensors = {}
    for name, t in (("gate", rg), ("shared_expert_gate", rs)):
        for part, v in zip(("weight", "scales", "biases"), t):
            tensors[f"l.mlp.{name}.{part}"] = v.cpu()
    for proj, m in (("gate_proj", gate), ("up_proj", up), ("down_proj", down)):
        for part, v in zip(("weight", "scales", "biases"), m):
            tensors[f"l.mlp.switch_mlp.{proj}.{part}"] = v[:shape.experts].cpu()
            tensors[f"l.mlp.shared_expert.{proj}.{part}"] = v[shape.experts].cpu()
    _save(tmp_path / "model.safetensors", tensors)
    layer = load.affine_routed(load.Checkpoint(tmp_path), "l.mlp.", shape.top_k, dev)
    router = torch.cat([load.dequantize(*rg), load.dequantize(*rs)]).to(torch.bfloat16)
    want_layer = moe.Routed(router, experts.make([gate, up], down, 64), shape.top_k, shared=True)
    assert layer.count == shape.experts and layer.experts.count == e1 and torch.equal(layer.router, router)
    assert torch.equal(layer.experts.up, want_layer.experts.up) and torch.equal(layer.experts.down, want_layer.experts.down)
    x = synthetic.activations(shape, 9, dev)
    assert torch.equal(moe.run(x, layer), moe.run(x, want_layer))


@pytest.mark.gpu
def test_exl3_groups_from_a_checkpoint(tmp_path):
    from tensorfold_b200 import load, synthetic
    from tensorfold_b200.exl3 import experts as x3
    from tensorfold_b200.exl3 import linear

    dev = torch.device("cuda", 0)
    shape = synthetic.SMALL
    count = 4
    gate, up, down = synthetic.exl3_layer(shape, dev, lambda e, m: (2, 4, 6)[(e + m) % 3])
    tensors = {}
    for e in range(count):
        for proj, m in (("gate_proj", gate), ("up_proj", up), ("down_proj", down)):
            t, suh, svh = m[e]
            tensors[f"x.experts.{e}.{proj}.trellis"] = t.cpu()
            tensors[f"x.experts.{e}.{proj}.suh"] = suh.cpu()
            tensors[f"x.experts.{e}.{proj}.svh"] = svh.cpu()
    t, _, svh = gate[0]
    tensors["x.q_proj.trellis"], tensors["x.q_proj.svh"] = t.cpu(), svh.cpu()
    tensors["x.q_proj.su"] = torch.randint(-32768, 32767, (shape.dims // 16,), dtype=torch.int32).to(torch.int16)
    tensors["x.q_proj.mcg"] = torch.zeros((1,), dtype=torch.int32)
    _save(tmp_path / "model.safetensors", tensors)
    ck = load.Checkpoint(tmp_path)
    ex = load.exl3_routed(ck, "x.experts", count, dev)
    want = x3.prepare(gate[:count], up[:count], down[:count], x3.CB_3INST, device=dev)
    assert ex.count == count and torch.equal(ex.gate_k2, want.gate_k2) and torch.equal(ex.down_k2, want.down_k2)
    assert torch.equal(ex.suh_g, want.suh_g) and torch.equal(ex.svh_d, want.svh_d)
    rows = 5
    x = synthetic.activations(shape, rows, dev)
    pick = torch.tensor([[0, 1, 2, 3]] * rows, dtype=torch.int32, device=dev)
    wts = torch.full((rows, 4), 0.25, dtype=torch.float32, device=dev)
    s = x3.Scratch(ex, rows, 4, device=dev)
    got = x3.routed(x, pick, wts, ex, s, None, rows).clone()
    assert torch.equal(got, x3.routed(x, pick, wts, want, x3.Scratch(want, rows, 4, device=dev), None, rows))
    lin = load.exl3_linear(ck, "x.q_proj", dev)
    assert lin.codebook == "mcg" and lin.k == shape.dims and lin.n == shape.width
    signs = load.unpack_signs(tensors["x.q_proj.su"]).to(dev)
    direct = linear.Exl3Linear.from_tensors(t, signs, svh, "mcg")
    assert torch.equal(lin(x), direct(x))


def test_exl3_groups_the_kernels_cannot_take_are_refused_by_name(tmp_path):
    """The header checks of ``src/tensorfold/cuda/exl3/format.py:226-267``, one bad group each; a good group parses to
    its width, codebook and sizes."""

    from tensorfold_b200 import load

    def group(k=128, n=256, words=40, **extra):
        g = {"trellis": torch.zeros((k // 16, n // 16, words), dtype=torch.int16),
             "suh": torch.ones((k,), dtype=torch.float16), "svh": torch.ones((n,), dtype=torch.float16)}
        g.update(extra)
        return {name: t for name, t in g.items() if t is not None}

    mark = torch.zeros((1,), dtype=torch.int32)
    cases = {
        "good": (group(mul1=mark), None),
        "signs": (group(words=48, suh=None, svh=None, su=torch.zeros((8,), dtype=torch.int16),
                        sv=torch.zeros((16,), dtype=torch.int16), bias=torch.zeros((256,), dtype=torch.float16)), None),
        "notrellis": ({"suh": torch.ones((128,), dtype=torch.float16)}, "no .trellis"),
        "dtype": (group(trellis=torch.zeros((8, 16, 40), dtype=torch.int32), mul1=mark), "trellis must be int16"),
        "rank": (group(trellis=torch.zeros((8, 640), dtype=torch.int16)), "trellis must be int16"),
        "width": (group(words=36, mul1=mark), "EXL3 widths"),
        "wide": (group(words=144), "EXL3 widths"),
        "both": (group(mul1=mark, mcg=mark), "both mcg and mul1"),
        "half": (group(mcg=mark), "need the mul1 codebook"),
        "half3": (group(), "need the mul1 codebook"),
        "noin": (group(words=32, suh=None), "no input scales"),
        "noout": (group(words=32, svh=None), "no output scales"),
        "inshape": (group(words=32, suh=torch.ones((64,), dtype=torch.float16)), ".suh must be F16 [128]"),
        "outtype": (group(words=32, svh=torch.ones((256,), dtype=torch.float32)), ".svh must be F16 [256]"),
        "sushape": (group(words=32, suh=None, su=torch.zeros((128,), dtype=torch.int16)), ".su must be I16 [8]"),
        "k64": (group(k=64, words=32), "multiples of 128"),
        "n192": (group(n=192, words=32), "multiples of 128"),
    }
    tensors = {f"{name}.{part}": t.clone() for name, (g, _) in cases.items() for part, t in g.items()}
    _save(tmp_path / "model.safetensors", tensors)
    ck = load.Checkpoint(tmp_path)
    assert load.parse_group(ck, "good") == (2.5, "mul1", 128, 256, "suh", "svh", False)
    assert load.parse_group(ck, "signs") == (3.0, "3inst", 128, 256, "su", "sv", True)
    for name, (_, why) in cases.items():
        if why is None:
            continue
        with pytest.raises(ValueError) as err:
            load.parse_group(ck, name)
        assert why in str(err.value) and str(err.value).startswith(name + ":"), (name, str(err.value))
        with pytest.raises(ValueError):
            load.exl3_group(ck, name, "cpu")
