"""Dense 4-bit lane matmul (``tensorfold_b200.qmm``): pack round trip, outputs against float64 in both arithmetic forms,
row invariance, group sums.  Follows the reference's checks for its ``kernels/qmm`` (tests/cuda/test_qmm.py)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def mlx(n, k, seed, dtype=torch.bfloat16, gs=64):
    g = torch.Generator(device=DEV).manual_seed(seed)
    words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (n, k // 8), generator=g, device=DEV, dtype=torch.int64).to(torch.int32)
    scales = (torch.rand((n, k // gs), generator=g, device=DEV) * 0.02 + 0.001).to(dtype)
    biases = (torch.randn((n, k // gs), generator=g, device=DEV) * 0.02).to(dtype)
    return words, scales, biases


def dequant64(words, scales, biases, gs=64):
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=words.device, dtype=torch.int64) * 4
    q = ((w[..., None] >> shifts) & 0xF).reshape(words.shape[0], -1).double()
    return q * scales.double().repeat_interleave(gs, -1) + biases.double().repeat_interleave(gs, -1)


def rows(m, k, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn((m, k), generator=g, device=DEV).to(torch.bfloat16)


@pytest.mark.parametrize("n,k", [(96, 512), (200, 2048), (1024, 768)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pack_round_trip(n, k, dtype):
    from tensorfold_b200 import qmm

    w, s, b = mlx(n, k, 5, dtype)
    q = qmm.pack(w, s, b, 64)
    assert q.n == n and q.k == k and q.n_pad % 32 == 0
    w2, s2, b2 = qmm.unpack(q)
    assert torch.equal(w2, w) and torch.equal(s2.view(torch.int16), s.view(torch.int16))
    assert torch.equal(b2.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("n,k", [(96, 512), (200, 2048), (2048, 768)])
@pytest.mark.parametrize("m", [1, 7, 16, 45])
def test_matmul_against_float64_and_rows_alone(n, k, m):
    from tensorfold_b200 import qmm

    w, s, b = mlx(n, k, 11)
    q = qmm.pack(w, s, b, 64)
    x = rows(m, k, 3)
    want = x.double() @ dequant64(w, s, b).t()
    got = qmm.matmul(x, q, f32=True)
    assert got.shape == (m, n) and got.dtype == torch.float32
    assert (got.double() - want).abs().max() <= 1e-5 * want.abs().max() * (k / 64) ** 0.5 + 1e-6
    got16 = qmm.matmul(x, q)
    assert torch.equal(got16, got.to(torch.bfloat16))
    r = m // 2
    assert torch.equal(qmm.matmul(x[r:r + 1], q, f32=True), got[r:r + 1])          # a row alone: the same bits
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    assert qmm.matmul(x, q, f32=True, out=out) is out and torch.equal(out, got)


@pytest.mark.parametrize("n,k,m", [(256, 512, 40), (1024, 2048, 300)])
def test_prefill_matmul_uses_weights_rounded_once_to_bf16(n, k, m):
    from tensorfold_b200 import qmm

    w, s, b = mlx(n, k, 13)
    q = qmm.pack(w, s, b, 64)
    x = rows(m, k, 4)
    wq = dequant64(w, s, b)
    # bf16 scales: the kernel's weight is the bf16 fma of (q, s, b): exact product and sum, one rounding
    w16 = wq.to(torch.bfloat16).double()
    want = x.double() @ w16.t()
    got = qmm.prefill_matmul(x, q, f32=True)
    assert (got.double() - want).abs().max() <= 2e-5 * want.abs().max() + 1e-6
    part = qmm.prefill_matmul(x[17:30], q, f32=True)
    assert torch.equal(part, got[17:30])
    assert torch.equal(qmm.prefill_matmul(x, q), got.to(torch.bfloat16))


def test_group_sums_and_argument_errors():
    from tensorfold_b200 import qmm

    x = rows(9, 640, 8)
    xs = qmm.group_sums(x)
    want = x.double().reshape(9, 10, 64).sum(-1)
    assert xs.shape == (9, 10) and (xs.double() - want).abs().max() < 1e-4
    wide = rows(9, 1280, 9)[:, :640]                                    # strided rows
    assert torch.equal(qmm.group_sums(wide), qmm.group_sums(wide.contiguous()))
    w, s, b = mlx(64, 640, 2)
    q = qmm.pack(w, s, b, 64)
    with pytest.raises(ValueError):
        qmm.matmul(x.float(), q)
    with pytest.raises(ValueError):
        qmm.matmul(x, q, sk=1)                                         # 10 groups are two slices: not the caller's choice
    with pytest.raises(ValueError):
        qmm.matmul(x, q, reduce=False, part=torch.empty(10, device=DEV))
    assert qmm.split_k(64, 2048) == 4 and qmm.split_k(64, 768) == 2 and qmm.bucket(3) == 8 and qmm.bucket(300) == 16


@pytest.mark.parametrize("n,k,m", [(96, 512, 1), (200, 2048, 5), (1024, 768, 19), (64, 256, 3)])
def test_k_slices_apart_add_up_to_the_reduced_bits(n, k, m):
    """``matmul(reduce=False)``: fp32 (split_k, M, n) slices whose sum in slice order is ``matmul(f32=True)`` bit for
    bit; ``part=`` is filled in place; one slice returns the product itself (the reference's contract,
    src/tensorfold/cuda/kernels/qmm.py:156-177)."""

    from tensorfold_b200 import qmm

    w, s, b = mlx(n, k, n + k)
    q = qmm.pack(w, s, b, 64)
    x = rows(m, k, m)
    whole = qmm.matmul(x, q, f32=True)
    sk = qmm.split_k(n, k)
    got = qmm.matmul(x, q, reduce=False)
    if sk == 1:
        assert got.shape == (m, n) and torch.equal(got.float(), qmm.matmul(x, q).float())
        return
    assert got.shape == (sk, m, n) and got.dtype == torch.float32 and got.is_contiguous()
    total = got[0].clone()
    for i in range(1, sk):
        total += got[i]
    assert torch.equal(total, whole)
    assert float(got[sk - 1].abs().max()) > 0
    part = torch.full((sk * m * n + 7,), 3.0, device=DEV)
    again = qmm.matmul(x, q, reduce=False, part=part)
    assert again.data_ptr() == part.data_ptr() and torch.equal(again, got) and bool((part[sk * m * n:] == 3.0).all())
