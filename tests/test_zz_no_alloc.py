"""The grouping entry point that brings its own scratch (``tfb_exl3_group_static``), for hosts that cannot allocate
device memory at call time: same tables as ``tfb_exl3_group`` and as the CPU grouping oracle, on two calls in a row, at
its exact capacity, with the device's memory in use unchanged across a call, and a clear refusal past its built-in size.

This file sorts last so that pytest collects it last: the built-in array is shared by every call in the process, and a
run that stops at the first failure (``-x``) has then already run every other test before this one can fail."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_PAIRS = 32768


def _static(pick, E, R, slots, maxm=None, check_alloc=True):
    from tensorfold_b200 import _lib

    maxu, maxm = min(R * slots, E), R if maxm is None else maxm
    uids = torch.full((maxu,), -7, dtype=torch.int32, device=DEV)
    count = torch.zeros((1,), dtype=torch.int32, device=DEV)
    members = torch.full((maxu, maxm), -7, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    held_before = torch.cuda.memory_allocated()
    _lib.call("tfb_exl3_group_static", pick.data_ptr(), uids.data_ptr(), count.data_ptr(), members.data_ptr(), R,
              slots, E, maxu, maxm, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    if check_alloc:                                    # the call allocates nothing: not through torch, not behind its back
        assert torch.cuda.memory_allocated() == held_before
        assert torch.cuda.mem_get_info()[0] == free_before
    n = int(count[0])
    return n, uids[:n].clone(), members[:n].clone()


def _caller_scratch(pick, E, R, slots, maxm=None):
    from tensorfold_b200 import _lib

    P = R * slots
    maxu, maxm = min(P, E), R if maxm is None else maxm
    uids = torch.full((maxu,), -7, dtype=torch.int32, device=DEV)
    count = torch.zeros((1,), dtype=torch.int32, device=DEV)
    members = torch.full((maxu, maxm), -7, dtype=torch.int32, device=DEV)
    tmp_m = torch.zeros((P,), dtype=torch.int32, device=DEV)
    tmp_i = torch.zeros((max(1, maxu), 3), dtype=torch.int32, device=DEV)
    tmp_c = torch.zeros((2,), dtype=torch.int32, device=DEV)
    _lib.call("tfb_exl3_group", pick.data_ptr(), uids.data_ptr(), count.data_ptr(), members.data_ptr(),
              tmp_m.data_ptr(), tmp_i.data_ptr(), tmp_c.data_ptr(), R, slots, E, maxu, maxm,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    n = int(count[0])
    return n, uids[:n].clone(), members[:n].clone()


def test_built_in_scratch_gives_the_same_tables_twice_in_a_row():
    from oracle import exl3 as ref

    g = torch.Generator().manual_seed(41)
    # the first call on a device sets up (the driver may load the kernel's code then): not measured
    _static(torch.zeros((1, 1), dtype=torch.int32, device=DEV), 4, 1, 1, check_alloc=False)
    # the second call is smaller and routes differently: it must not see anything the first left in the shared array
    for E, R, slots in ((160, 300, 9), (24, 17, 5)):
        pick = torch.randint(0, E + 2, (R, slots), generator=g).to(torch.int32).to(DEV)      # ids >= E are skipped
        n0, u0, m0 = _caller_scratch(pick, E, R, slots)
        n1, u1, m1 = _static(pick, E, R, slots)
        assert n0 == n1 and n0 > 0
        assert torch.equal(u0, u1) and torch.equal(m0, m1)
        uids, members = ref.group(pick.cpu().numpy(), E)                                      # and the CPU oracle's
        assert u1.cpu().tolist() == uids.tolist() and np.array_equal(m1.cpu().numpy(), members)


def test_exact_capacity_with_the_most_experts():
    """32768 pairs over 1024 experts: the last word of the built-in array and the largest shared-memory opt-in."""

    E, slots = 1024, 32
    R = MAX_PAIRS // slots
    g = torch.Generator().manual_seed(43)
    pick = torch.stack([torch.randperm(E, generator=g)[:slots] for _ in range(R)]).to(torch.int32).to(DEV)
    cap = 96                                           # members a row of the table keeps (rows a expert sees: ~32)
    _static(torch.zeros((1, 1), dtype=torch.int32, device=DEV), 4, 1, 1, check_alloc=False)
    n0, u0, m0 = _caller_scratch(pick, E, R, slots, cap)
    n1, u1, m1 = _static(pick, E, R, slots, cap)
    assert n0 == n1 == E and torch.equal(u0, u1) and torch.equal(m0, m1)
    # every pair appears exactly once, under its own expert, in row order
    codes = m1.cpu().numpy()
    pk = pick.cpu().numpy()
    seen = 0
    for u in range(E):
        row = codes[u][codes[u] >= 0]
        assert np.all(np.diff(row) > 0)
        assert np.all(pk[row >> 5, row & 31] == u)
        seen += row.size
    assert seen == MAX_PAIRS


def test_calls_past_the_built_in_size_are_refused():
    from tensorfold_b200 import _lib

    t = torch.zeros((8,), dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="exceed the built-in scratch"):
        _lib.call("tfb_exl3_group_static", t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 4097, 8, 128, 128,
                  4097, 0)
    with pytest.raises(ValueError, match="at most 1024 experts"):
        _lib.call("tfb_exl3_group_static", t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 4, 8, 1025, 32, 4, 0)
