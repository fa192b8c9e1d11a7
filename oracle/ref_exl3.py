"""TEST INFRASTRUCTURE: drives the REFERENCE's own EXL3 expert kernels (its extension compiled unmodified by
``oracle/build_ref_cuda.py``) through the call sequence of its ``routed`` operator, so that this library's EXL3 path can
be checked against, and timed beside, the reference's kernels on the same GPU.

The sequence and the tile settings are the reference's (``src/tensorfold/cuda/exl3/experts.py:136-143`` the settings,
``:146-170`` the scratch, ``:173-202`` the launches); the layer object is this library's ``Exl3RoutedExperts``, whose
fields carry the same tables.  Nothing here is used by the product."""

from __future__ import annotations

import torch

GATEUP, DOWN = (8, 4, 4, 1), (8, 4, 1, 1)            # (n tiles a block, warps, K splits, tiles in flight)
FALLBACKS = ((8, 4, 2, 1), (8, 4, 1, 1), (4, 4, 2, 2), (4, 4, 1, 2))


def config(k: int, n: int, gateup: bool):
    for nt, w, sk, pf in ((GATEUP if gateup else DOWN), *FALLBACKS):
        if k % (16 * sk * w) == 0 and n % (16 * nt) == 0:
            return nt, w, sk, pf
    raise ValueError(f"no tile setting divides K={k}, N={n}")


class Scratch:
    def __init__(self, ex, rows: int, slots: int, device="cuda") -> None:
        d, i, p = ex.dims, ex.width, rows * slots
        self.cfg_gu, self.cfg_d = config(d, i, True), config(i, d, False)
        self.xg = torch.zeros((p, d), dtype=torch.float16, device=device)
        self.xu = torch.zeros((p, d), dtype=torch.float16, device=device)
        self.xd = torch.zeros((p, i), dtype=torch.float16, device=device)
        self.z = torch.zeros((max(2 * self.cfg_gu[2] * i, self.cfg_d[2] * d) * p,), dtype=torch.float32, device=device)
        self.y = torch.zeros((p, d), dtype=torch.float32, device=device)
        maxu = min(p, ex.count)
        self.ids = torch.zeros((maxu,), dtype=torch.int32, device=device)
        self.count = torch.zeros((1,), dtype=torch.int32, device=device)
        self.members = torch.full((maxu, rows), -1, dtype=torch.int32, device=device)
        self.rows, self.slots = rows, slots


def routed(ext, x, pick, wts, ex, s: Scratch, out, limit: float = 3.0e38, act_mode: int = 1):
    """The reference's launches for R = s.rows rows: y per slot [R * slots, D] fp32, or ``out`` [R, D] when ``wts``."""

    r, slots, d, i, e = s.rows, s.slots, ex.dims, ex.width, ex.count
    p = r * slots
    ext.group(pick, s.ids, s.count, s.members, r, slots, e)
    ext.rot_in(x, x.stride(0), pick, ex.suh_g, ex.suh_u, s.xg, s.xu, r, d, slots, e)
    nt, w, sk, pf = s.cfg_gu
    ext.grouped(s.xg, s.xu, ex.gate_ptr, ex.up_ptr, ex.gate_k2, ex.up_k2, s.ids, s.count, s.members, s.z, 2, d, i, p,
                sk, slots, ex.cb, nt, w, pf, ex.k2_gu[0], ex.k2_gu[1])
    ext.gateup_epilogue(s.z, pick, ex.svh_g, ex.svh_u, ex.suh_d, s.xd, r, p, i, sk, slots, e, float(limit), act_mode)
    nt, w, sk, pf = s.cfg_d
    ext.grouped(s.xd, s.xd, ex.down_ptr, ex.down_ptr, ex.down_k2, ex.down_k2, s.ids, s.count, s.members, s.z, 1, i, d,
                p, sk, slots, ex.cb, nt, w, pf, ex.k2_d[0], ex.k2_d[1])
    if wts is None:
        ext.down_epilogue(s.z, pick, ex.svh_d, s.y, r, p, d, sk, slots, e)
        return s.y
    ext.down_combine(s.z, pick, ex.svh_d, s.y, wts, out, r, p, d, sk, slots, e)
    return out
