"""EXL3 linear layers (attention and head projections) on the routed experts' kernels: the layer is one "expert" and
every input row one member, so the trellis decoder, the K split by shape and the row invariance are the experts'.

Mirrors ``tensorfold.cuda.exl3.linear`` (``src/tensorfold/cuda/exl3/linear.py:58-203``): ``Exl3Linear.from_tensors``,
``__call__`` (y = x @ W + bias for 1..128 rows, any codebook and width), ``unpack``, ``unpack_cuda``, ``k2_of``.
The input rotation is the experts' prologue with one matrix, the product and the output rotation their down
projection.
The trellis is read where the caller keeps it (the reference's "stored" layout; no strip copy is made).  No CPU path.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import _lib
from . import experts as routed

CODEBOOK_IDS = {"3inst": routed.CB_3INST, "mcg": routed.CB_MCG, "mul1": routed.CB_MUL1}
MAX_ROWS = 128


def k2_of(bits: float) -> int:
    k2 = int(round(2 * bits))
    if k2 not in routed.K2_SUPPORTED or abs(2 * bits - k2) > 1e-9:
        raise ValueError(f"unsupported EXL3 bit width {bits}")
    return k2


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


@dataclass
class Exl3Linear:
    """One EXL3 layer on the GPU: trellis int16 [K/16, N/16, 16 * bits] in place, fp16 scales, optional fp16 bias."""

    trellis: torch.Tensor
    suh: torch.Tensor             # fp16 [K]
    svh: torch.Tensor             # fp16 [N]
    bias: torch.Tensor | None     # fp16 [N]
    bits: float
    codebook: str
    k: int
    n: int
    _state: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_tensors(cls, trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor, codebook: str,
                     bias: torch.Tensor | None = None, device: str | torch.device = "cuda") -> "Exl3Linear":
        if codebook not in CODEBOOK_IDS:
            raise ValueError(f"unknown EXL3 codebook {codebook!r}")
        if trellis.dim() != 3 or trellis.dtype != torch.int16:
            raise ValueError("trellis must be int16 [K/16, N/16, 16 * bits]")
        bits = trellis.shape[2] / 16
        if not float(bits).is_integer() and codebook != "mul1":
            raise ValueError(f"{bits}-bit EXL3 tiles need the mul1 codebook")
        k2_of(bits)
        k, n = 16 * trellis.shape[0], 16 * trellis.shape[1]
        if k % 128 or n % 128:
            raise ValueError(f"K={k} and N={n} must be multiples of 128")

        def scales(t: torch.Tensor, size: int) -> torch.Tensor:
            if t.dtype != torch.float16 or t.numel() != size:
                raise ValueError(f"scales must be fp16 [{size}]")
            return t.reshape(size).to(device).contiguous()

        b = None if bias is None else bias.to(device=device, dtype=torch.float16).contiguous()
        return cls(trellis.to(device).contiguous(), scales(suh, k), scales(svh, n), b, bits, codebook, k, n)

    @property
    def k2(self) -> int:
        return k2_of(self.bits)

    def nbytes(self) -> int:
        return self.trellis.numel() * 2

    def _tables(self, m: int) -> dict:
        """What the experts' kernels need to see the layer as one "expert" whose members are the m input rows: the
        pointer and width of the one matrix, all-zero picks, and the sort of those picks (rows in order, items of 16)."""

        st = self._state
        if "ptr" not in st:
            dev = self.trellis.device
            if self.trellis.data_ptr() % 16:
                raise ValueError("the trellis must start on a 16-byte boundary")
            st["ptr"] = torch.tensor([self.trellis.data_ptr()], dtype=torch.int64, device=dev)
            st["k2"] = torch.tensor([self.k2], dtype=torch.int32, device=dev)
            st["rows"] = {}
        rows = st["rows"].get(m)
        if rows is None:
            dev = self.trellis.device
            n_items = -(-m // routed.ITEM_PAIRS)
            first = torch.arange(n_items, dtype=torch.int32) * routed.ITEM_PAIRS
            items = torch.stack([torch.zeros_like(first), first, (m - first).clamp(max=routed.ITEM_PAIRS)], dim=1)
            rows = st["rows"][m] = {
                "pick": torch.zeros((m,), dtype=torch.int32, device=dev),
                "members": torch.arange(m, dtype=torch.int32, device=dev),
                "items": items.contiguous().to(dev),
                "counts": torch.tensor([n_items, 1], dtype=torch.int32, device=dev),
                "arrive": torch.zeros((n_items * (self.n // 128),), dtype=torch.int32, device=dev),
                "n_items": n_items,
            }
        return {**st, **rows}

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                 xh: torch.Tensor | None = None, z: torch.Tensor | None = None) -> torch.Tensor:
        """y [M, N] = x [M, K] @ W + bias for M = 1 .. MAX_ROWS; scratch ``xh`` fp16 [M, K] and ``z`` fp32 [M, N] are
        allocated when not given.  Every 16 rows decode the trellis once (the decode form of the experts)."""

        if not x.is_cuda or x.dim() != 2 or x.shape[1] != self.k or not 1 <= x.shape[0] <= MAX_ROWS:
            raise ValueError(f"x must be CUDA [1..{MAX_ROWS}, {self.k}], got {tuple(x.shape)}")
        if x.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("x must be bf16 or fp16")
        x = x.contiguous()
        m, dev = x.shape[0], x.device
        t = self._tables(m)
        if xh is None:
            xh = torch.empty((m, self.k), dtype=torch.float16, device=dev)
        if z is None:
            z = torch.empty((m, self.n), dtype=torch.float32, device=dev)
        y = torch.empty((m, self.n), dtype=torch.float32, device=dev)
        s = _stream(x)
        with torch.cuda.device(dev):
            _lib.call("tfb_exl3_prologue", x.data_ptr(), x.stride(0), int(x.dtype == torch.float16),
                      t["pick"].data_ptr(), self.suh.data_ptr(), 0, xh.data_ptr(), 0, m, self.k, 1, 1, 0, 0, 0, 0, 0,
                      0, 0, 0, 0, 0, s)
            _lib.call("tfb_exl3_down", xh.data_ptr(), t["ptr"].data_ptr(), t["k2"].data_ptr(), t["items"].data_ptr(),
                      t["counts"].data_ptr(), t["members"].data_ptr(), z.data_ptr(), t["arrive"].data_ptr(),
                      self.svh.data_ptr(), y.data_ptr(), self.k, self.n, m, CODEBOOK_IDS[self.codebook], t["n_items"],
                      0, routed.ITEM_PAIRS, self.k2, routed.col_tiles(t["n_items"], t["n_items"], self.n, 1, self.k2), s)
        if self.bias is not None:
            y += self.bias.float()
        want = out_dtype or (out.dtype if out is not None else x.dtype)
        if out is None:
            return y.to(want)
        out.copy_(y)
        return out

    def unpack(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """W_q [K, N] fp16 decoded on the GPU, into ``out`` when given."""

        w = routed.dequant(self.trellis, self.codebook)
        if out is None:
            return w
        out.copy_(w)
        return out


def unpack_cuda(trellis: torch.Tensor, codebook: str) -> torch.Tensor:
    """W_q [K, N] fp16 from trellis int16 [K/16, N/16, 16 * bits] on the GPU."""

    return routed.dequant(trellis.cuda().contiguous(), codebook)
