"""EXL3 prompt matmuls: for more rows than the decode form takes (128), W_q is decoded once into fp16 and a dense GEMM
does the product; this library's kernels do the rotations either side of it.

Mirrors ``tensorfold.cuda.exl3.prefill`` (``src/tensorfold/cuda/exl3/prefill.py:15-95``): ``Workspace``, ``tiles``,
``matmul(layer, x, out, ws)``.  The steps are the reference's: the input rotation (the experts' prologue), the decode
of the whole trellis through the kernels' own lane decoder (``tfb_exl3_dequant``: the bit-exact W_q), a plain fp16
GEMM with fp32 accumulation and fp32 output (cuBLAS through ``torch.mm``: a library GEMM, as the reference uses
Triton's), and the output rotation, svh and bias in fp32 (``tfb_exl3_rot_out``; the reference rotates by two bf16
products with the Hadamard matrix, this one by the exact butterfly).  No CPU path.
"""

from __future__ import annotations

import torch

from .. import _lib
from .linear import CODEBOOK_IDS, Exl3Linear

_OUT_TYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def tiles(k: int, n: int) -> tuple[int, int]:
    """(rows, columns) the output rotation handles at once: a row's 128-column block - the shape's alone, so a row
    never depends on its chunk.  The GEMM's own tiling is the library's."""

    return 1, 128


class Workspace:
    """One decoded W_q, one rotated input and one product, grown to the largest call and reused (calls run in order on
    one stream)."""

    def __init__(self) -> None:
        self.w: torch.Tensor | None = None
        self.xh: torch.Tensor | None = None
        self.z: torch.Tensor | None = None
        self.pick: torch.Tensor | None = None

    def _grow(self, name: str, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        t = getattr(self, name)
        if t is None or t.numel() < numel or t.device != torch.device(device):
            t = torch.empty((numel,), dtype=dtype, device=device)
            setattr(self, name, t)
        return t

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w, self.xh, self.z) if t is not None)


def matmul(layer: Exl3Linear, x: torch.Tensor, out: torch.Tensor, ws: Workspace) -> torch.Tensor:
    """out [M, N] (row stride free; fp32, fp16 or bf16) = x [M, K] @ W + bias for any M, the prompt path's arithmetic."""

    m, k, n = x.shape[0], layer.k, layer.n
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or x.dim() != 2:
        raise ValueError("prefill matmul: x must be CUDA bf16 or fp16 [M, K]")
    if x.shape[1] != k or out.shape != (m, n) or out.stride(1) != 1:
        raise ValueError(f"prefill matmul: x {tuple(x.shape)} and out {tuple(out.shape)} do not match K={k}, N={n}")
    if out.dtype not in _OUT_TYPES or out.device != x.device:
        raise ValueError("prefill matmul: out must be fp32, fp16 or bf16 on x's device")
    if m == 0:
        return out
    x = x.contiguous()
    dev = x.device
    st = torch.cuda.current_stream(dev).cuda_stream
    xh = ws._grow("xh", m * k, torch.float16, dev)[:m * k].view(m, k)
    wq = ws._grow("w", k * n, torch.float16, dev)[:k * n].view(k, n)
    z = ws._grow("z", m * n, torch.float32, dev)[:m * n].view(m, n)
    pick = ws._grow("pick", m, torch.int32, dev)[:m]                # every row is a pair of the one "expert"
    with torch.cuda.device(dev):
        pick.zero_()
        _lib.call("tfb_exl3_prologue", x.data_ptr(), x.stride(0), int(x.dtype == torch.float16), pick.data_ptr(),
                  layer.suh.data_ptr(), 0, xh.data_ptr(), 0, m, k, 1, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, st)
        _lib.call("tfb_exl3_dequant", layer.trellis.data_ptr(), wq.data_ptr(), k, n, layer.k2,
                  CODEBOOK_IDS[layer.codebook], st)
        torch.mm(xh, wq, out_dtype=torch.float32, out=z)
        _lib.call("tfb_exl3_rot_out", z.data_ptr(), layer.svh.data_ptr(),
                  layer.bias.data_ptr() if layer.bias is not None else 0, out.data_ptr(), out.stride(0),
                  _OUT_TYPES[out.dtype], m, n, st)
    return out
