"""Makes ``exl3_golden.npz`` from the REFERENCE's own decoder (run where the reference tree is mounted; its root is
taken from ``TENSORFOLD_REFERENCE``, the same variable ``oracle/build_ref.py`` reads):

    python tests/golden/make_exl3_golden.py

For every codebook and every width the reference's format module accepts it stores a small random trellis and the
W_q bits ``tensorfold.cuda.exl3.format.unpack`` returns for it, plus codebook spot values and one rotated forward.
The tests compare the oracle restatement (and, on the GPU, the kernels) with these arrays.
"""

import os
import sys
from pathlib import Path

import numpy as np

# the reference checkout: $TENSORFOLD_REFERENCE, else a folder named "reference" beside this repository
sys.path.insert(0, str(Path(os.environ.get("TENSORFOLD_REFERENCE") or Path(__file__).resolve().parents[3] / "reference") / "src"))
from tensorfold.cuda.exl3 import format as fmt  # noqa: E402

out = {}
rng = np.random.default_rng(2026)
for ci, cb in enumerate(fmt.CODEBOOKS):
    table = fmt.codebook(cb)
    spots = np.array([0, 1, 0xFFFF, *rng.integers(0, 65536, size=61).tolist()], dtype=np.int64)
    out[f"cb{ci}_states"] = spots.astype(np.uint16)
    out[f"cb{ci}_values"] = table[spots].view(np.uint16)
    for bits in fmt.BITS:
        if not (float(bits).is_integer() or cb == "mul1"):
            continue
        k2 = int(2 * bits)
        t = rng.integers(-2 ** 15, 2 ** 15, size=(2, 3, fmt.tile_words(bits)), dtype=np.int64).astype(np.int16)
        out[f"t_cb{ci}_k{k2}"] = t
        out[f"w_cb{ci}_k{k2}"] = fmt.unpack(t, bits, cb).view(np.uint16)
# one layer forward: K = 256, N = 128, 3 bits, mcg
t = rng.integers(-2 ** 15, 2 ** 15, size=(16, 8, fmt.tile_words(3)), dtype=np.int64).astype(np.int16)
suh = (rng.standard_normal(256) * 0.05).astype(np.float16)
svh = (rng.standard_normal(128) * 0.5).astype(np.float16)
x = rng.standard_normal((3, 256))
out.update(fwd_t=t, fwd_suh=suh.view(np.uint16), fwd_svh=svh.view(np.uint16), fwd_x=x,
           fwd_y=fmt.forward(x, t, suh, svh, 3, "mcg"))
np.savez_compressed(Path(__file__).with_name("exl3_golden.npz"), **out)
print(len(out), "arrays")
