"""The allocation-free plan entry point against the regular one.

`ffai_op_moe_plan_static` exists for hosts that own every byte of device memory and do not let a
plug-in call the CUDA allocator once they are serving (a server with a pre-sized arena, for
instance).  It keeps its scratch in a fixed array inside the library instead of taking a workspace.
Its results must be identical to the CPU oracle's plan and to `ffai_op_moe_plan` (integers: exact), on the
first call and on later calls that find the previous call's contents in the array.  The file name sorts last so a
run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

from ffai_b200 import capi
from helpers import from_dev, to_dev

pytestmark = pytest.mark.gpu

MAX_ROWS = 131072


def _plan(lib, fn_static, idx, T, k, E):
    import torch
    di = to_dev(idx)
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    perm = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    inv = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    if fn_static:
        rc = lib.ffai_op_moe_plan_static(di.data_ptr(), T, k, E, counts.data_ptr(), offsets.data_ptr(),
                                         perm.data_ptr(), inv.data_ptr(), None)
    else:
        ws = torch.zeros(max(1, lib.ffai_op_moe_plan_workspace_bytes(T * k, E) // 4), dtype=torch.int32, device="cuda")
        rc = lib.ffai_op_moe_plan(di.data_ptr(), T, k, E, counts.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                                  inv.data_ptr(), ws.data_ptr(), None)
    assert rc == capi.FFAI_OK
    torch.cuda.synchronize()
    return [from_dev(t, np.uint32) for t in (counts, offsets, perm, inv)]


def test_static_plan_matches_oracle_and_workspace_plan_twice_in_a_row(ffai_lib, oracle_mod):
    """Both problems hold more than 32768 routed rows, so the count / scan / scatter form runs: the only
    reader of the library-resident array.  The second problem has another shape, and each is planned twice,
    so every call after the first finds the previous call's counters in the array."""
    rng = np.random.default_rng(11)
    for T, k, E in ((8192, 8, 256), (5000, 8, 64)):
        assert T * k > 32768
        idx = np.stack([rng.choice(E, size=k, replace=False) for _ in range(T)]).astype(np.uint32)
        want = oracle_mod.plan(idx, T, k, E)
        regular = _plan(ffai_lib, False, idx, T, k, E)
        for a, b in zip(regular, want):
            assert np.array_equal(a, b)
        for _ in range(2):
            got = _plan(ffai_lib, True, idx, T, k, E)
            for a, b in zip(got, want):
                assert np.array_equal(a, b)


def test_static_plan_rejects_sizes_beyond_its_array(ffai_lib):
    one = 16  # non-null, never dereferenced: validation fails first
    assert ffai_lib.ffai_op_moe_plan_static(one, MAX_ROWS // 8 + 1, 8, 128, one, one, one, one, None) == capi.FFAI_ERR_INVALID_ARG
    assert ffai_lib.ffai_op_moe_plan_static(one, 16, 2, 1025, one, one, one, one, None) == capi.FFAI_ERR_INVALID_ARG
