"""A barrier between expert-parallel ranks whose peer never arrives: the wait runs out after the set limit, the status
word names the barrier and the missing rank, nothing is pulled from or stored into a peer, and the context stays usable.

One GPU: a two-rank window table whose entries both point at this GPU's own buffer, so the flag of the other rank is
simply never written.  No kernel is left waiting: the limit is 20 ms.  (The reference's counterpart is the rank named
by ``NCCL.ready``, src/tensorfold/cuda/comm.py:78-101.)"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def short_limit():
    from tensorfold_b200 import _lib

    was = _lib.set_wait_limit_ms(20)
    assert _lib.kernel_status() == 0
    yield
    _lib.set_wait_limit_ms(was)
    _lib.kernel_status()                                   # leave the word clear for the tests that follow


def _window(world, rows, dims):
    """A window laid out as ``ep.PeerWindow`` does: flags, tokens, result buffer; both table entries are this buffer."""

    x_off, x_bytes = 256, rows * dims * 2
    p_off = x_off + (x_bytes + 255) // 256 * 256
    win = torch.zeros(p_off + world * rows * dims * 4, dtype=torch.uint8, device=DEV)
    table = torch.tensor([win.data_ptr()] * world, dtype=torch.int64, device=DEV)
    return win, table, x_off, x_bytes, p_off


@pytest.mark.parametrize("rank,missing", [(0, 1), (1, 0)])
def test_tokens_barrier_names_the_rank_that_never_arrived(short_limit, rank, missing):
    from tensorfold_b200 import _lib

    world, rows, dims = 2, 4, 64
    win, table, x_off, x_bytes, p_off = _window(world, rows, dims)
    win[x_off:x_off + x_bytes] = 7                          # what a pull would bring
    dst = torch.zeros(world * x_bytes, dtype=torch.uint8, device=DEV)
    step = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    seg = ((ctypes.c_int64 * 1)(x_off), (ctypes.c_int64 * 1)(x_bytes), (ctypes.c_void_p * 1)(dst.data_ptr()))
    _lib.call("tfb_peer_gather", table.data_ptr(), rank, world, 1, seg[0], seg[1], seg[2], step.data_ptr(), st)
    # a later kernel of the same step must leave the peers alone while the failure is unread
    y = torch.ones((world * rows, 1, dims), dtype=torch.float32, device=DEV)
    wts = torch.ones((world * rows, 1), dtype=torch.float32, device=DEV)
    pick = torch.zeros((world * rows, 1), dtype=torch.int32, device=DEV)
    _lib.call("tfb_combine_push", y.data_ptr(), wts.data_ptr(), pick.data_ptr(), 0, 1, table.data_ptr(), p_off, rank,
              rows, world * rows, 1, dims, step.data_ptr(), st)
    out = torch.full((rows, dims), 3.0, dtype=torch.float32, device=DEV)
    _lib.call("tfb_peer_sum", table.data_ptr(), rank, p_off, world, rows, dims, out.data_ptr(), 1, 0, 0, 1,
              0, step.data_ptr(), st)
    torch.cuda.synchronize()
    status = _lib.kernel_status()
    assert status & 0xFF == _lib.ST_WAIT_TIMEOUT
    assert (status >> 8) & 0xFF == 1 and (status >> 16) & 0xFF == missing       # tokens barrier, the absent rank
    assert f"rank {missing}" in _lib.describe_status(status) and "tokens barrier" in _lib.describe_status(status)
    assert int(dst.sum()) == 0                                                   # nothing was pulled
    assert float(win[p_off:].view(torch.float32).abs().sum()) == 0.0             # nothing was pushed
    assert float((out - 3.0).abs().sum()) == 0.0                                 # nothing was summed
    assert _lib.kernel_status() == 0                                             # reading cleared the word
    # the context is intact: an ordinary kernel still runs
    assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0


def test_results_barrier_is_told_apart(short_limit):
    from tensorfold_b200 import _lib

    world, rows, dims = 2, 4, 64
    win, table, _, _, p_off = _window(world, rows, dims)
    step = torch.ones(1, dtype=torch.int32, device=DEV)     # one step counted: the barrier waits for flag >= 1
    out = torch.full((rows, dims), 3.0, dtype=torch.float32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    _lib.call("tfb_peer_sum", table.data_ptr(), 0, p_off, world, rows, dims, out.data_ptr(), 1, 0, 0, 1,
              0, step.data_ptr(), st)
    torch.cuda.synchronize()
    with pytest.raises(_lib.StepFailed) as err:
        _lib.check_status()
    assert (err.value.status >> 8) & 0xFF == 2 and (err.value.status >> 16) & 0xFF == 1
    assert "results barrier" in str(err.value) and "rank 1" in str(err.value)
    assert float((out - 3.0).abs().sum()) == 0.0


def test_a_complete_table_passes_and_the_limit_is_checked(short_limit):
    """With one rank the barrier is its own flag: the same calls complete and move the data."""

    from tensorfold_b200 import _lib

    world, rows, dims = 1, 4, 64
    win, table, x_off, x_bytes, p_off = _window(world, rows, dims)
    win[x_off:x_off + x_bytes] = 7
    dst = torch.zeros(x_bytes, dtype=torch.uint8, device=DEV)
    step = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    seg = ((ctypes.c_int64 * 1)(x_off), (ctypes.c_int64 * 1)(x_bytes), (ctypes.c_void_p * 1)(dst.data_ptr()))
    _lib.call("tfb_peer_gather", table.data_ptr(), 0, world, 1, seg[0], seg[1], seg[2], step.data_ptr(), st)
    torch.cuda.synchronize()
    assert _lib.kernel_status() == 0 and int(dst.min()) == 7
    with pytest.raises(ValueError):
        _lib.set_wait_limit_ms(0)
