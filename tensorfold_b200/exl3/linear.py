"""EXL3 linear layers (attention and head projections) on the routed experts' kernels: the layer is one "expert" and
every input row one member, so the trellis decoder, the K split by shape and the row invariance are the experts'.

Mirrors ``tensorfold.cuda.exl3.linear`` (``src/tensorfold/cuda/exl3/linear.py:58-203``): ``Exl3Linear.from_tensors``,
``__call__`` (y = x @ W + bias for 1..128 rows, any codebook and width), ``unpack``, ``unpack_cuda``, ``k2_of``.
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

    def _tables(self):
        """Pointer / width tables of the one matrix, and per row count the members of "expert" 0 (never changes)."""

        st = self._state
        if "ptr" not in st:
            dev = self.trellis.device
            st["ptr"] = torch.tensor([self.trellis.data_ptr()], dtype=torch.int64, device=dev)
            st["k2"] = torch.tensor([self.k2], dtype=torch.int32, device=dev)
            st["ids"] = torch.zeros((1,), dtype=torch.int32, device=dev)
            st["count"] = torch.ones((1,), dtype=torch.int32, device=dev)
            st["pick"] = torch.zeros((MAX_ROWS,), dtype=torch.int32, device=dev)
            st["members"] = {}
        return st

    def _members(self, m: int) -> torch.Tensor:
        st = self._tables()
        mem = st["members"].get(m)
        if mem is None:
            # row * 32 + slot for slot 0 of every row, the table the grouping kernel would make for all-zero picks
            mem = (torch.arange(m, dtype=torch.int32, device=self.trellis.device) * 32).contiguous()
            st["members"][m] = mem
        return mem

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                 xh: torch.Tensor | None = None, z: torch.Tensor | None = None) -> torch.Tensor:
        """y [M, N] = x [M, K] @ W + bias for M = 1..128; scratch ``xh`` fp16 [M, K] and ``z`` fp32 [M, N] are
        allocated when not given."""

        if not x.is_cuda or x.dim() != 2 or x.shape[1] != self.k or not 1 <= x.shape[0] <= MAX_ROWS:
            raise ValueError(f"x must be CUDA [1..{MAX_ROWS}, {self.k}], got {tuple(x.shape)}")
        if x.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("x must be bf16 or fp16")
        x = x.contiguous()
        m, dev = x.shape[0], x.device
        st = self._tables()
        if xh is None:
            xh = torch.empty((m, self.k), dtype=torch.float16, device=dev)
        if z is None:
            z = torch.empty((m, self.n), dtype=torch.float32, device=dev)
        y = torch.empty((m, self.n), dtype=torch.float32, device=dev)
        pick, mem, s = st["pick"], self._members(m), _stream(x)
        cb = CODEBOOK_IDS[self.codebook]
        with torch.cuda.device(dev):
            _lib.call("tfb_exl3_rot_in", x.data_ptr(), x.stride(0), 1 if x.dtype == torch.float16 else 0,
                      pick.data_ptr(), self.suh.data_ptr(), self.suh.data_ptr(), xh.data_ptr(), xh.data_ptr(), m,
                      self.k, 1, 1, s)
            _lib.call("tfb_exl3_grouped", xh.data_ptr(), xh.data_ptr(), st["ptr"].data_ptr(), st["ptr"].data_ptr(),
                      st["k2"].data_ptr(), st["k2"].data_ptr(), st["ids"].data_ptr(), st["count"].data_ptr(),
                      mem.data_ptr(), z.data_ptr(), 1, self.k, self.n, m, 1, cb, m, 1, s)
            _lib.call("tfb_exl3_down_epilogue", z.data_ptr(), pick.data_ptr(), self.svh.data_ptr(), y.data_ptr(), 0, 0,
                      m, self.n, 1, 1, s)
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
