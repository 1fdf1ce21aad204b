"""The allocation-free self-check entry point against the allocating one.

fo_selftest_static exists for hosts that cannot allocate device memory when they call the
library (a framework that owns the GPU's memory, a server that bans cudaMalloc after
start-up, a sandbox without the allocation calls): its counters sit in a static device array.
Both entry points run the same sweeps, so their reports must be equal, also on a second call
in a row, which only holds if the shared array is cleared every time.  Collected last on
purpose: a failure here cannot hide a failure of any other test in a run that stops early.
"""

import ctypes

import pytest

pytestmark = pytest.mark.gpu


def _alloc(which, arg=0):
    from flashoptim_jax_b200 import _lib

    out = ctypes.c_uint64(0xDEAD)
    _lib.check(_lib.lib().fo_selftest(which, arg, ctypes.byref(out), 0))
    return out.value


def _static(which, arg=0, n=1):
    from flashoptim_jax_b200 import _lib

    out = (ctypes.c_uint64 * n)(*([0xDEAD] * n))
    _lib.check(_lib.lib().fo_selftest_static(which, arg, out, n, 0))
    return list(out)


def test_static_scratch_entry_point_matches_allocating_one_twice_in_a_row():
    from flashoptim_jax_b200 import _lib

    cases = [
        (_lib.FO_SELFTEST_CODE_TABLES, 0), (_lib.FO_SELFTEST_SOFTSIGN, 0), (_lib.FO_SELFTEST_SQRT, 0),
        (_lib.FO_SELFTEST_RECONSTRUCT, 116), (_lib.FO_SELFTEST_SPLIT, 108), (_lib.FO_SELFTEST_GROUP_DIV, 50),
    ]
    for which, arg in cases:
        want = _alloc(which, arg)
        assert _static(which, arg) == [want], (which, arg)
        assert _static(which, arg) == [want], (which, arg, "second call")
    # sweeps with several counters: each one against the allocating entry point's per-counter report
    for which, n in ((_lib.FO_SELFTEST_RCP, 3), (_lib.FO_SELFTEST_PACKED, 2)):
        want = [_alloc(which, k) for k in range(n)]
        assert _static(which, 0, n) == want
        assert _static(which, 0, n) == want


def test_static_scratch_entry_point_refuses_more_counters_than_it_holds():
    from flashoptim_jax_b200 import _lib

    lib = _lib.lib()
    n = _lib.FO_SELFTEST_STATIC_MAX_COUNTERS + 1
    out = (ctypes.c_uint64 * n)()
    rc = lib.fo_selftest_static(_lib.FO_SELFTEST_CODE_TABLES, 0, out, n, 0)
    assert rc == 4  # FO_ERR_TOO_LARGE
    assert b"static scratch holds" in lib.fo_last_error()
    assert lib.fo_selftest_static(_lib.FO_SELFTEST_CODE_TABLES, 0, out, 0, 0) == 1
    assert lib.fo_selftest_static(99, 0, out, 1, 0) == 1
    # and it still works afterwards
    assert _static(_lib.FO_SELFTEST_CODE_TABLES) == [_alloc(_lib.FO_SELFTEST_CODE_TABLES)]
