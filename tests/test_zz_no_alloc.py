"""The grouping entry point that brings its own scratch (``tfb_exl3_group_static``), for hosts that cannot allocate
device memory at call time: same tables as ``tfb_exl3_group`` on two calls in a row, and a clear refusal past its
built-in size.  Collected last on purpose."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _both(pick, E, R, slots):
    """(uids, count, members) from the caller-scratch entry point and from the built-in-scratch one."""

    from tensorfold_b200 import _lib

    P = R * slots
    maxu = min(P, E)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        uids = torch.full((maxu,), -7, dtype=torch.int32, device=DEV)
        count = torch.zeros((1,), dtype=torch.int32, device=DEV)
        members = torch.full((maxu, R), -7, dtype=torch.int32, device=DEV)
        if static:
            _lib.call("tfb_exl3_group_static", pick.data_ptr(), uids.data_ptr(), count.data_ptr(), members.data_ptr(),
                      R, slots, E, maxu, R, stream)
        else:
            tmp_m = torch.zeros((P,), dtype=torch.int32, device=DEV)
            tmp_i = torch.zeros((max(1, maxu), 3), dtype=torch.int32, device=DEV)
            tmp_c = torch.zeros((2,), dtype=torch.int32, device=DEV)
            _lib.call("tfb_exl3_group", pick.data_ptr(), uids.data_ptr(), count.data_ptr(), members.data_ptr(),
                      tmp_m.data_ptr(), tmp_i.data_ptr(), tmp_c.data_ptr(), R, slots, E, maxu, R, stream)
        torch.cuda.synchronize()
        n = int(count[0])
        outs.append((n, uids[:n].clone(), members[:n].clone()))
    return outs


def test_built_in_scratch_gives_the_same_tables_twice_in_a_row():
    g = torch.Generator().manual_seed(41)
    # the second call is smaller and routes differently: it must not see anything the first left in the shared array
    for E, R, slots in ((160, 300, 9), (24, 17, 5)):
        pick = torch.randint(0, E + 2, (R, slots), generator=g).to(torch.int32).to(DEV)      # ids >= E are skipped
        (n0, u0, m0), (n1, u1, m1) = _both(pick, E, R, slots)
        assert n0 == n1 and n0 > 0
        assert torch.equal(u0, u1) and torch.equal(m0, m1)


def test_calls_past_the_built_in_size_are_refused():
    from tensorfold_b200 import _lib

    t = torch.zeros((8,), dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="exceed the built-in scratch"):
        _lib.call("tfb_exl3_group_static", t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 4097, 8, 128, 128,
                  4097, 0)
