"""Stand-alone codecs and the fp32 <-> (param, ECC) helpers against the NumPy oracle (bit-exact),
and the reference's own codec tests re-expressed (tests/test_quantization.py, tests/test_compression.py)."""

import numpy as np
import pytest

from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("group_size", [32, 1, 8, 40, 256, 1024])
def test_quantize_dequantize_match_oracle(group_size):
    import flashoptim_jax_b200 as fo

    rng = np.random.default_rng(group_size)
    for shape in ((1,), (31,), (65,), (7, 33), (4097,), (300, 70)):
        x = (rng.normal(0, 1, shape) * np.exp2(rng.integers(-25, 5, shape))).astype(np.float32)
        x.reshape(-1)[::7] = 0
        q = fo.quantize_momentum(H.to_torch(x), group_size)
        want = O.quantize_momentum(x, group_size)
        assert q.values.shape == x.shape and tuple(q.scales.shape) == want.scales.shape
        np.testing.assert_array_equal(H.to_numpy(q.values), want.values)
        np.testing.assert_array_equal(H.bits(H.to_numpy(q.scales)), H.bits(want.scales))
        np.testing.assert_array_equal(H.bits(H.to_numpy(fo.dequantize_momentum(q, group_size))),
                                      H.bits(O.dequantize_momentum(want, group_size)))
        q = fo.quantize_variance(H.to_torch(x * x), group_size)
        want = O.quantize_variance(x * x, group_size)
        np.testing.assert_array_equal(H.to_numpy(q.values), want.values)
        np.testing.assert_array_equal(H.bits(H.to_numpy(q.scales)), H.bits(want.scales))
        np.testing.assert_array_equal(H.bits(H.to_numpy(fo.dequantize_variance(q, group_size))),
                                      H.bits(O.dequantize_variance(want, group_size)))


def test_quantization_reference_tests():
    import torch

    import flashoptim_jax_b200 as fo

    x = torch.linspace(-3.0, 3.0, 65, device="cuda")  # tests/test_quantization.py:13-28
    q = fo.quantize_momentum(x)
    xr = fo.dequantize_momentum(q)
    assert q.values.dtype == torch.int8 and q.scales.dtype == torch.float16
    assert (xr - x).abs().mean() < 0.05
    assert torch.dot(x, xr) / (x.norm() * xr.norm()) > 0.999
    x = torch.linspace(0.0, 10.0, 65, device="cuda")  # tests/test_quantization.py:31-39
    q = fo.quantize_variance(x)
    assert q.values.dtype == torch.uint8
    assert np.isclose(float(q.scales[-1]), float(x[64:].sqrt().max()), rtol=1e-3)
    assert (fo.dequantize_variance(q) - x).abs().mean() < 0.1


@pytest.mark.parametrize("dt,mwb", [("bf16", 24), ("bf16", 32), ("f16", 24), ("f16", 32), ("bf16", None)])
def test_split_reconstruct_match_oracle(dt, mwb):
    import torch

    import flashoptim_jax_b200 as fo

    tdt, ndt = (torch.bfloat16, H.BF16) if dt == "bf16" else (torch.float16, np.dtype(np.float16))
    rng = np.random.default_rng(3)
    lo, hi = (-140, 30) if dt == "bf16" else (-30, 10)
    x = (rng.normal(0, 1, 200000) * np.exp2(rng.integers(lo, hi, 200000))).astype(np.float32)
    x[::11] = 0
    lp, ecc = fo.split_leaf(H.to_torch(x), narrow_dtype=tdt, master_weight_bits=mwb)
    wlp, wecc = O.split_leaf(x, ndt, mwb)
    np.testing.assert_array_equal(H.bits(H.to_numpy(lp)), H.bits(wlp))
    if wecc is None:
        assert ecc.dtype == torch.int32 and ecc.dim() == 0
    else:
        np.testing.assert_array_equal(H.to_numpy(ecc), wecc)
    np.testing.assert_array_equal(H.bits(H.to_numpy(fo.reconstruct_leaf(lp, ecc))), H.bits(O.reconstruct_leaf(wlp, wecc)))


def test_compression_reference_tests():
    import torch

    import flashoptim_jax_b200 as fo

    x = torch.tensor([-3.25, -1.125, -0.2, 0.0, 0.3, 1.75, 7.125, 1000.125], device="cuda")  # test_compression.py:7-22
    lp, ecc = fo.split_leaf(x)
    rec = fo.reconstruct_leaf(lp, ecc)
    plain, fixed = (x - lp.float()).abs(), (x - rec).abs()
    assert lp.dtype == torch.bfloat16 and ecc.dtype == torch.int8
    assert torch.all(fixed <= plain + 1e-12) and torch.any(fixed < plain)
    x = torch.tensor([0.0, 1.0, -2.0, 3.5], device="cuda")  # test_compression.py:25-32
    lp, ecc = fo.split_leaf(x)
    assert torch.all(ecc == 0) and torch.equal(fo.reconstruct_leaf(lp, ecc), x)
    x = torch.tensor([-3.25, -1.125, 0.3, 7.125], device="cuda")  # test_compression.py:35-43
    lp, ecc = fo.split_leaf(x, narrow_dtype=torch.float16, master_weight_bits=32)
    assert lp.dtype == torch.float16 and ecc.dtype == torch.int16
    assert torch.allclose(fo.reconstruct_leaf(lp, ecc), x, atol=1e-4, rtol=1e-4)
    params = {"w": torch.tensor([1.0, -2.0], dtype=torch.bfloat16, device="cuda"), "bn": torch.tensor([0.25, -0.5], device="cuda")}
    errs = {"w": torch.zeros(2, dtype=torch.int8, device="cuda"), "bn": torch.zeros((), dtype=torch.int32)}
    rec = fo.reconstruct_weights(params, errs)  # test_compression.py:46-60
    assert rec["w"].dtype == torch.float32 and torch.equal(rec["bn"], params["bn"])


def test_set_fp32_params_round_trip():
    # tests/test_checkpointing.py:107-141
    import torch

    import flashoptim_jax_b200 as fo

    params = {"w": torch.linspace(-2, 2, 64, device="cuda").to(torch.bfloat16), "norm": torch.tensor([1.0, 0.5, -0.25], device="cuda")}
    grads = {"w": torch.linspace(-0.3, 0.4, 64, device="cuda"), "norm": torch.tensor([0.1, -0.2, 0.3], device="cuda")}
    tx = fo.flash_adamw(learning_rate=1e-3, fused=False)
    state = tx.init(params)
    params, state = tx.step(params, state, grads)
    fp32 = fo.reconstruct_weights(params, state.ecc)
    rp, recc = fo.set_fp32_params(fp32, param_template=params, master_weight_bits=24)
    rec = fo.reconstruct_weights(rp, recc)
    assert torch.allclose(rec["w"], fp32["w"], atol=1e-4, rtol=1e-4) and torch.allclose(rec["norm"], fp32["norm"], atol=1e-7, rtol=1e-7)
    assert rp["w"].dtype == torch.bfloat16 and rp["norm"].dtype == torch.float32
    with pytest.raises(ValueError, match="matching tree structure"):
        fo.set_fp32_params({"w": fp32["w"]}, param_template=params)
    assert fo.cast_tree_bf16({"a": torch.ones(2)})["a"].dtype == torch.bfloat16
