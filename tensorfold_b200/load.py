"""Load-time path: safetensors checkpoints straight into this library's layouts.

A small reader of the safetensors container (8-byte little-endian header length, JSON header, raw tensor bytes) that
hands tensors to ``experts.make`` / ``exl3.experts.prepare`` / ``qmm.pack`` without a dequantised copy ever existing:
* MLX affine 4-bit checkpoints - a layer's router rows and experts as ``moe.Routed`` (names as in
  ``src/tensorfold/families/qwen3_5_moe/cuda/weights.py:32-46``);
* EXL3 checkpoints - a group's ``trellis`` / ``suh`` | ``su`` / ``svh`` | ``sv`` / ``mcg`` | ``mul1`` parts
  (``src/tensorfold/cuda/exl3/format.py:226-267``) as ``Exl3Linear`` or as a layer's ``Exl3RoutedExperts``
  (``src/tensorfold/families/qwen4_exp/cuda/exl3.py:22-83``).
Bytes are read with plain buffered reads into pinned memory and copied to the device; the packing itself runs on the
GPU (``tfb_pack``).  The reference's O_DIRECT span reader (``src/tensorfold/cuda/direct_read.py``) is not rebuilt.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

DTYPES = {"BOOL": torch.bool, "U8": torch.uint8, "I8": torch.int8, "I16": torch.int16, "U16": torch.uint16,
          "I32": torch.int32, "U32": torch.uint32, "I64": torch.int64, "F16": torch.float16, "BF16": torch.bfloat16,
          "F32": torch.float32, "F64": torch.float64}
PROJS = ("gate_proj", "up_proj", "down_proj")


class Checkpoint:
    """The tensors of one ``.safetensors`` file or of a folder of them: every file's header is read (an index file
    beside them is not needed and not looked at)."""

    def __init__(self, path: str | Path) -> None:
        root = Path(path)
        files = [root] if root.is_file() else sorted(root.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no .safetensors under {root}")
        self.headers: dict[Path, tuple[int, dict]] = {}
        self.where: dict[str, Path] = {}
        for f in files:
            with open(f, "rb") as fh:
                size = struct.unpack("<Q", fh.read(8))[0]
                header = json.loads(fh.read(size))
            header.pop("__metadata__", None)
            self.headers[f] = (8 + size, header)
            for name in header:
                self.where[name] = f

    def names(self) -> list[str]:
        return sorted(self.where)

    def has(self, name: str) -> bool:
        return name in self.where

    def entry(self, name: str) -> tuple[Path, int, int, str, list[int]]:
        """(file, absolute begin, absolute end, dtype name, shape)."""

        if name not in self.where:
            raise KeyError(f"{name} is in no file of this checkpoint")
        f = self.where[name]
        base, header = self.headers[f]
        e = header[name]
        begin, end = e["data_offsets"]
        return f, base + begin, base + end, e["dtype"], list(e["shape"])

    def get(self, name: str, device: str | torch.device = "cpu") -> torch.Tensor:
        f, begin, end, dtype, shape = self.entry(name)
        if dtype not in DTYPES:
            raise ValueError(f"{name}: dtype {dtype} is not handled")
        cuda = torch.device(device).type == "cuda"
        raw = torch.empty((end - begin,), dtype=torch.uint8, pin_memory=cuda and torch.cuda.is_available())
        view, at = memoryview(raw.numpy()), 0
        with open(f, "rb", buffering=0) as fh:
            fh.seek(begin)
            while at < end - begin:
                got = fh.readinto(view[at:])
                if not got:
                    raise IOError(f"short read of {f} at {begin + at}")
                at += got
        t = raw.view(DTYPES[dtype]).reshape(shape)
        return t.to(device) if cuda else t

    def codebook(self, prefix: str) -> str:
        return "mul1" if self.has(prefix + ".mul1") else "mcg" if self.has(prefix + ".mcg") else "3inst"


def dequantize(words: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, gs: int = 64) -> torch.Tensor:
    """MLX affine words [..., K * bits / 32] with scales and biases [..., K / gs] -> fp32 [..., K] (s * q + b); for the
    router rows, which the layer keeps in bf16 (``src/tensorfold/families/qwen3_5_moe/cuda/weights.py:20-29``)."""

    k = scales.shape[-1] * gs
    bits = 32 * words.shape[-1] // k
    per = 32 // bits
    w = words.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, device=words.device, dtype=torch.int64) * bits
    q = ((w[..., None] >> shifts) & ((1 << bits) - 1)).reshape(*words.shape[:-1], k).to(torch.float32)
    return q * scales.float().repeat_interleave(gs, -1) + biases.float().repeat_interleave(gs, -1)


def unpack_signs(packed: torch.Tensor) -> torch.Tensor:
    """su / sv int16 [n/16] -> fp16 [n] of +1 and -1: bit b of word w set means element 16 w + b is -1
    (``src/tensorfold/cuda/exl3/format.py:135-140``)."""

    p = packed.cpu().numpy().view(np.uint16).astype(np.uint32).reshape(-1)
    bits = (p[:, None] >> np.arange(16, dtype=np.uint32)) & 1
    return torch.from_numpy((1.0 - 2.0 * bits.reshape(-1)).astype(np.float16))


def affine_routed(ck: Checkpoint, prefix: str, top_k: int, device="cuda", gs: int = 64):
    """Layer ``prefix`` (ending in "mlp.") of an MLX affine 4-bit checkpoint as ``moe.Routed``: router rows dequantised
    once to bf16 (the shared expert's gate row last), experts packed on the GPU (the shared expert last)."""

    from . import experts as grouped
    from . import moe

    def triple(name: str):
        w = ck.get(name + ".weight", device)
        return (w.view(torch.int32) if w.dtype != torch.int32 else w), ck.get(name + ".scales", device), \
            ck.get(name + ".biases", device)

    shared = ck.has(prefix + "shared_expert_gate.weight")
    rows = [dequantize(*triple(prefix + "gate"), gs)]
    if shared:
        rows.append(dequantize(*triple(prefix + "shared_expert_gate"), gs))
    router = torch.cat(rows).to(torch.bfloat16).contiguous()

    def table(proj: str):
        mine = triple(prefix + f"switch_mlp.{proj}")
        if not shared:
            return tuple(t.contiguous() for t in mine)
        extra = triple(prefix + f"shared_expert.{proj}")
        return tuple(torch.cat([a, b[None]]).contiguous() for a, b in zip(mine, extra))

    ex = grouped.make([table("gate_proj"), table("up_proj")], table("down_proj"), gs)
    return moe.Routed(router, ex, int(top_k), shared=shared)


EXL3_BITS = (1.0, 1.5, 2.0, 2.5, 3.0, 3.5, 4.0, 4.5, 5.0, 5.5, 6.0, 6.5, 7.0, 7.5, 8.0)
EXL3_PARTS = ("trellis", "suh", "su", "svh", "sv", "mcg", "mul1", "bias")
HADAMARD = 128


def parse_group(ck: Checkpoint, prefix: str) -> tuple[float, str, int, int, str, str, bool]:
    """(bits, codebook, K, N, input-scale part, output-scale part, has bias) of the EXL3 group ``prefix`` from the
    header entries alone; ValueError, saying why, for a group the kernels cannot take.  The refusals are those of
    ``src/tensorfold/cuda/exl3/format.py:226-267``: no trellis, a trellis that is not int16 [K/16, N/16, 16 * bits]
    at a width of 1..8 bits in half steps, both codebook markers, a fractional width without the mul1 codebook,
    missing or mis-shaped scales (fp16 [K] / [N], or packed signs int16 [K/16] / [N/16]), K or N not a multiple of
    the 128-point rotation."""

    def fail(why: str) -> ValueError:
        return ValueError(f"{prefix}: {why}")

    parts = {}
    for part in EXL3_PARTS:
        if ck.has(f"{prefix}.{part}"):
            _, _, _, dtype, shape = ck.entry(f"{prefix}.{part}")
            parts[part] = (dtype, shape)
    if "trellis" not in parts:
        raise fail("no .trellis")
    dtype, shape = parts["trellis"]
    if dtype != "I16" or len(shape) != 3:
        raise fail(f"trellis must be int16 [K/16, N/16, 16 * bits], got {dtype} {shape}")
    bits = shape[2] / 16
    if shape[2] % 8 or bits not in EXL3_BITS:
        raise fail(f"a trellis row of {shape[2]} words is {bits} bits; EXL3 widths are 1..8 in half steps")
    marks = [m for m in ("mcg", "mul1") if m in parts]
    if len(marks) > 1:
        raise fail("both mcg and mul1 markers")
    cb = marks[0] if marks else "3inst"
    if not float(bits).is_integer() and cb != "mul1":
        raise fail(f"{bits}-bit tiles need the mul1 codebook, found {cb}")
    k, n = 16 * shape[0], 16 * shape[1]
    chosen = []
    for full, packed, size, what in (("suh", "su", k, "input"), ("svh", "sv", n, "output")):
        if full in parts:
            name, want = full, ("F16", [size])
        elif packed in parts:
            name, want = packed, ("I16", [size // 16])
        else:
            raise fail(f"no {what} scales (.{full} or .{packed})")
        if (parts[name][0], list(parts[name][1])) != want:
            raise fail(f".{name} must be {want[0]} {want[1]}, got {parts[name][0]} {parts[name][1]}")
        chosen.append(name)
    if k % HADAMARD or n % HADAMARD:
        raise fail(f"K={k} and N={n} must be multiples of {HADAMARD} (the rotation's blocks)")
    return float(bits), cb, k, n, chosen[0], chosen[1], "bias" in parts


def exl3_group(ck: Checkpoint, prefix: str, device="cuda"):
    """(trellis int16, suh fp16 [K], svh fp16 [N], codebook name, bias or None) of the EXL3 group ``prefix``; the
    group's header entries are checked (``parse_group``) before any bytes are read."""

    parse_group(ck, prefix)
    trellis = ck.get(prefix + ".trellis", device)

    def scales(full: str, packed: str, size: int) -> torch.Tensor:
        if ck.has(f"{prefix}.{full}"):
            t = ck.get(f"{prefix}.{full}")
        elif ck.has(f"{prefix}.{packed}"):
            t = unpack_signs(ck.get(f"{prefix}.{packed}"))
        else:
            raise KeyError(f"{prefix}: no .{full} or .{packed}")
        if t.dtype != torch.float16 or t.numel() != size:
            raise ValueError(f"{prefix}.{full}: fp16 [{size}] expected")
        return t.reshape(size).to(device)

    k, n = 16 * trellis.shape[0], 16 * trellis.shape[1]
    bias = ck.get(prefix + ".bias", device) if ck.has(prefix + ".bias") else None
    return trellis, scales("suh", "su", k), scales("svh", "sv", n), ck.codebook(prefix), bias


def exl3_linear(ck: Checkpoint, prefix: str, device="cuda"):
    """The EXL3 group ``prefix`` (e.g. "model.layers.0.self_attn.q_proj") as an ``Exl3Linear``."""

    from .exl3 import linear

    trellis, suh, svh, cb, bias = exl3_group(ck, prefix, device)
    return linear.Exl3Linear.from_tensors(trellis, suh, svh, cb, bias, device)


def exl3_routed(ck: Checkpoint, prefix: str, count: int, device="cuda"):
    """Experts ``prefix.{0..count-1}.{gate,up,down}_proj`` as ``Exl3RoutedExperts``, each matrix at its own width."""

    from .exl3 import experts as x3

    names = [f"{prefix}.{e}" for e in range(count)]
    books = {ck.codebook(f"{nm}.{p}") for nm in names for p in PROJS}
    if len(books) > 1:
        raise ValueError(f"{prefix}: the experts mix EXL3 codebooks ({', '.join(sorted(books))}); the grouped kernel "
                         "takes one codebook a layer")
    lists = {p: [exl3_group(ck, f"{nm}.{p}", device)[:3] for nm in names] for p in PROJS}
    return x3.prepare(lists["gate_proj"], lists["up_proj"], lists["down_proj"], books.pop(), device=device)
