"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

One generator per tensor, seed = 1000 * config + tensor index, so every tensor can be regenerated alone.  Router rows
bf16 ~ N(0, 0.02); activations bf16 ~ N(0, 1); affine experts: uint32 words of uniform nibbles, scale |N(0, 0.01)|,
bias N(0, 0.01) per 64 inputs (fp16, or bf16 for the reference's CUDA convention).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class LayerShape:
    name: str
    config: int            # seed family
    dims: int              # D
    experts: int           # E routed experts
    width: int             # NI
    top_k: int
    shared: bool = False   # one always-on shared expert of the same width behind a sigmoid gate


C1 = LayerShape("c1", 1, 2048, 128, 768, 8)
C2 = LayerShape("c2", 2, 2048, 128, 768, 8)
C4 = LayerShape("c4", 4, 6144, 256, 2048, 8, shared=True)
SMALL = LayerShape("small", 9, 256, 12, 128, 4)
SMALL_SHARED = LayerShape("small_shared", 10, 256, 12, 128, 4, shared=True)


def _gen(seed: int, device) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def activations(shape: LayerShape, rows: int, device="cuda", index: int = 0) -> torch.Tensor:
    g = _gen(1000 * shape.config + index, device)
    return torch.randn((rows, shape.dims), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)


def router_rows(shape: LayerShape, device="cuda", zipf: float = 0.0) -> torch.Tensor:
    """[E (+1), D] bf16 ~ N(0, 0.02); the shared expert's gate row last."""

    g = _gen(1000 * shape.config + 1, device)
    n = shape.experts + (1 if shape.shared else 0)
    return (torch.randn((n, shape.dims), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)


def zipf_bias(shape: LayerShape, s: float = 1.1, device="cuda") -> torch.Tensor:
    """Additive logit skew log(rank^-s) under a seeded permutation of the experts, [E] fp32."""

    g = torch.Generator().manual_seed(1000 * shape.config + 2)
    perm = torch.randperm(shape.experts, generator=g)
    rank = torch.empty(shape.experts, dtype=torch.float32)
    rank[perm] = torch.arange(1, shape.experts + 1, dtype=torch.float32)
    return (-s * torch.log(rank)).to(device)


def affine_matrix(seed: int, e: int, n: int, k: int, device="cuda", scale_dtype=torch.float16, gs: int = 64):
    """(words int32 [e, n, k/8], scales, biases [e, n, k/gs])."""

    g = _gen(seed, device)
    words = torch.randint(-(2 ** 31), 2 ** 31, (e, n, k // 8), generator=g, device=device, dtype=torch.int64)
    words = words.to(torch.int32)
    scales = (torch.randn((e, n, k // gs), generator=g, device=device, dtype=torch.float32) * 0.01).abs()
    biases = torch.randn((e, n, k // gs), generator=g, device=device, dtype=torch.float32) * 0.01
    return words, scales.to(scale_dtype), biases.to(scale_dtype)


def affine_layer(shape: LayerShape, device="cuda", scale_dtype=torch.float16, copy: int = 0):
    """(gate, up, down) MLX triples for the layer's E (+1 shared) experts; ``copy`` selects an independent weight set."""

    e = shape.experts + (1 if shape.shared else 0)
    base = 1000 * shape.config + 10 + 3 * copy
    gate = affine_matrix(base, e, shape.width, shape.dims, device, scale_dtype)
    up = affine_matrix(base + 1, e, shape.width, shape.dims, device, scale_dtype)
    down = affine_matrix(base + 2, e, shape.dims, shape.width, device, scale_dtype)
    return gate, up, down


C3 = LayerShape("c3", 3, 2048, 128, 768, 8)
C5 = LayerShape("c5", 5, 4096, 160, 1536, 8)


def exl3_matrix(seed: int, k: int, n: int, bits: int, device="cuda"):
    """(trellis int16 [k/16, n/16, 16 * bits] of uniform 16-bit words, suh fp16 [k], svh fp16 [n] = +-1 x |N(0, 0.02)|)."""

    g = _gen(seed, device)
    t = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * bits), generator=g, device=device, dtype=torch.int32)

    def scale(m):
        sign = torch.randint(0, 2, (m,), generator=g, device=device).float() * 2 - 1
        return (sign * (torch.randn((m,), generator=g, device=device) * 0.02).abs()).half()

    return t.to(torch.int16), scale(k), scale(n)


def exl3_layer(shape: LayerShape, device="cuda", bits=4, copy: int = 0):
    """Per-expert (gate, up, down) triples at ``bits`` per weight; ``bits`` may be a callable (expert, matrix) -> bits
    for mixed-width stacks (config 5 draws 2..8 per tensor from a seeded generator)."""

    base = 1000 * shape.config + 10 + 1000003 * copy
    gate, up, down = [], [], []
    for e in range(shape.experts):
        b = [bits(e, m) if callable(bits) else bits for m in range(3)]
        gate.append(exl3_matrix(base + 3 * e, shape.dims, shape.width, b[0], device))
        up.append(exl3_matrix(base + 3 * e + 1, shape.dims, shape.width, b[1], device))
        down.append(exl3_matrix(base + 3 * e + 2, shape.width, shape.dims, b[2], device))
    return gate, up, down
