"""The kernels' exact-arithmetic shortcuts against the plain IEEE formulation, on the device.

fo_selftest sweeps the whole input space where that is feasible (every fp32 for sqrt and
split, every (param bits, ecc) pair for reconstruct, every fp32 in [-1, 1] for the soft-sign
code) and a large random sample for the two-operand divisions.  The bar is zero mismatches.
"""

import ctypes

import pytest

pytestmark = pytest.mark.gpu


def _run(which, arg=0):
    from flashoptim_jax_b200 import _lib

    out = ctypes.c_uint64(12345)
    _lib.check(_lib.lib().fo_selftest(which, arg, ctypes.byref(out), 0))
    return out.value


def test_sqrt_shortcut_matches_ieee_for_every_float():
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_SQRT) == 0


def test_softsign_code_matches_ieee_for_every_float_in_unit_interval():
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_SOFTSIGN) == 0


def test_ecc_fraction_tables():
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_CODE_TABLES) == 0


@pytest.mark.parametrize("pdt", [1, 2], ids=["bf16", "fp16"])
@pytest.mark.parametrize("ecc_bits", [8, 16])
def test_reconstruct_shortcut_exhaustive(pdt, ecc_bits):
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_RECONSTRUCT, pdt * 100 + ecc_bits) == 0


@pytest.mark.parametrize("pdt", [1, 2], ids=["bf16", "fp16"])
@pytest.mark.parametrize("ecc_bits", [8, 16])
def test_split_shortcut_exhaustive(pdt, ecc_bits):
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_SPLIT, pdt * 100 + ecc_bits) == 0


def test_group_scale_division_shortcut_on_random_pairs():
    from flashoptim_jax_b200 import _lib

    # 4e9 random (value, scale) pairs: codes through the reciprocal shortcut vs IEEE divisions
    assert _run(_lib.FO_SELFTEST_GROUP_DIV, 4000) == 0


def test_selftest_rejects_unknown_ids():
    from flashoptim_jax_b200 import _lib

    out = ctypes.c_uint64(0)
    assert _lib.lib().fo_selftest(99, 0, ctypes.byref(out), 0) != 0
    assert _lib.lib().fo_selftest(_lib.FO_SELFTEST_SPLIT, 7, ctypes.byref(out), 0) != 0


def test_reciprocal_shortcut_matches_ieee_for_every_float_in_range():
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_RCP, 0) == 0


def test_packed_product_sum_keeps_two_roundings():
    from flashoptim_jax_b200 import _lib

    assert _run(_lib.FO_SELFTEST_PACKED, 0) == 0
