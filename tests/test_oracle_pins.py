"""The NumPy oracle against every exact known-answer the reference's own tests hold for this path.

Each test names the reference test it re-expresses (paths inside the reference project).
JAX/optax are not available, so textbook float64 trajectories stand in for optax with the
same loose tolerances the reference uses.
"""

import ml_dtypes
import numpy as np
import pytest

from oracle import flashoptim_oracle as O

BF16 = ml_dtypes.bfloat16


def test_round_to_nearest_ties_go_up():
    # tests/test_quantization.py:42-44
    r = O._round_to_nearest(np.array([-63.5, -62.5, 62.5, 63.5], dtype=np.float32))
    np.testing.assert_array_equal(r, np.array([-63.0, -62.0, 63.0, 64.0], dtype=np.float32))


def test_momentum_roundtrip_quality():
    # tests/test_quantization.py:13-28
    x = np.linspace(-3.0, 3.0, 65, dtype=np.float32)
    q = O.quantize_momentum(x)
    xr = O.dequantize_momentum(q)
    assert q.values.dtype == np.int8 and q.scales.dtype == np.float16
    assert q.values.shape == x.shape and q.scales.shape == (3,)
    assert np.abs(xr - x).mean() < 0.05
    assert np.dot(x, xr) / (np.linalg.norm(x) * np.linalg.norm(xr)) > 0.999


def test_variance_tail_scale_matches_tail_absmax():
    # tests/test_quantization.py:31-39
    x = np.linspace(0.0, 10.0, 65, dtype=np.float32)
    q = O.quantize_variance(x)
    xr = O.dequantize_variance(q)
    assert q.values.dtype == np.uint8
    assert np.isclose(np.float32(q.scales[-1]), np.sqrt(x[64:]).max(), rtol=1e-3)
    assert np.abs(xr - x).mean() < 0.1


def test_split_reconstruct_improves_on_plain_bf16():
    # tests/test_compression.py:7-22
    x = np.array([-3.25, -1.125, -0.2, 0.0, 0.3, 1.75, 7.125, 1000.125], dtype=np.float32)
    lp, ecc = O.split_leaf(x)
    xr = O.reconstruct_leaf(lp, ecc)
    plain = np.abs(x - lp.astype(np.float32))
    fixed = np.abs(x - xr)
    assert lp.dtype == O.BF16 and ecc.dtype == np.int8
    assert np.all(fixed <= plain + 1e-12) and np.any(fixed < plain)


def test_exact_bf16_values_give_zero_ecc():
    # tests/test_compression.py:25-32
    x = np.array([0.0, 1.0, -2.0, 3.5], dtype=BF16).astype(np.float32)
    lp, ecc = O.split_leaf(x)
    np.testing.assert_array_equal(ecc, np.zeros_like(ecc))
    np.testing.assert_array_equal(O.reconstruct_leaf(lp, ecc), x)


def test_fp16_with_int16_ecc():
    # tests/test_compression.py:35-43
    x = np.array([-3.25, -1.125, 0.3, 7.125], dtype=np.float32)
    lp, ecc = O.split_leaf(x, narrow_dtype=np.float16, master_weight_bits=32)
    assert lp.dtype == np.float16 and ecc.dtype == np.int16
    np.testing.assert_allclose(O.reconstruct_leaf(lp, ecc), x, atol=1e-4, rtol=1e-4)


def test_fp32_leaf_has_no_ecc():
    # tests/test_compression.py:46-60 (the 0-d int32 sentinel is None here)
    bn = np.array([0.25, -0.5], dtype=np.float32)
    lp, ecc = O.split_leaf(bn, narrow_dtype=np.float32, master_weight_bits=24)
    assert ecc is None
    np.testing.assert_array_equal(O.reconstruct_leaf(bn, None), bn)


# ---- closed-form single steps (tests/test_optimizer_surface.py:12-161) -----

P = np.array([1.0, -2.0, 3.0], dtype=np.float32)
G = np.array([0.2, -0.1, 0.05], dtype=np.float32)


def _adam_f64(p, g, *, lr, b1, b2, eps, wd, decoupled, step):
    p, g = p.astype(np.float64), g.astype(np.float64)
    lr = float(np.float32(lr))
    if not decoupled and wd:
        g = g + wd * p
    mu = (1 - b1) * g
    nu = (1 - b2) * g * g
    if decoupled and wd:
        p = p * (1 - lr * wd)
    return p - (lr / (1 - b1**step)) * mu / (np.sqrt(nu) / np.sqrt(1 - b2**step) + eps)


@pytest.mark.parametrize("conv", [O.UNFUSED, O.FUSED], ids=["unfused", "fused"])
def test_adam_coupled_closed_form(conv):
    # tests/test_optimizer_surface.py:56-80 (flash_adam, quantize=False, no ECC)
    bc1, bc2 = O.bias_corrections(0.9, 0.999, 1)
    z = np.zeros(3, dtype=np.float32)
    r = O.adam_leaf(G, P, None, z, z, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2,
                    decoupled_weight_decay=False, bias_correction1=bc1, bias_correction2=bc2,
                    quantize=False, master_weight_bits=None, conv=conv)
    exp = _adam_f64(P, G, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=1e-2, decoupled=False, step=1)
    np.testing.assert_allclose(r.param, exp, atol=1e-6, rtol=1e-6)
    assert r.param.dtype == np.float32 and r.ecc is None


@pytest.mark.parametrize("conv", [O.UNFUSED, O.FUSED], ids=["unfused", "fused"])
def test_lion_closed_form(conv):
    # tests/test_optimizer_surface.py:83-104
    r = O.lion_leaf(G, P, None, np.zeros(3, dtype=np.float32), lr=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2,
                    quantize=False, master_weight_bits=None, conv=conv)
    lr = float(np.float32(1e-4))
    exp = P.astype(np.float64) * (1 - lr * 1e-2) - lr * np.sign(0.1 * G)
    np.testing.assert_allclose(r.param, exp, atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(r.mu, 0.01 * G, atol=1e-7, rtol=1e-5)


@pytest.mark.parametrize("conv", [O.UNFUSED, O.FUSED], ids=["unfused", "fused"])
def test_sgd_nesterov_closed_form(conv):
    # tests/test_optimizer_surface.py:107-133; state starts as zeros, so mu1 = (1-damp)*g
    r = O.sgd_leaf(G, P, None, np.zeros(3, dtype=np.float32), lr=1e-3, momentum=0.9, dampening=0.0,
                   weight_decay=1e-2, nesterov=True, decoupled_weight_decay=False,
                   quantize=False, master_weight_bits=None, conv=conv)
    lr = float(np.float32(1e-3))
    g = G.astype(np.float64) + 1e-2 * P
    exp = P - lr * (g + 0.9 * g)
    np.testing.assert_allclose(r.param, exp, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("conv", [O.UNFUSED, O.FUSED], ids=["unfused", "fused"])
def test_sgdw_closed_form(conv):
    # tests/test_optimizer_surface.py:136-161
    r = O.sgd_leaf(G, P, None, np.zeros(3, dtype=np.float32), lr=1e-3, momentum=0.9, dampening=0.0,
                   weight_decay=1e-2, nesterov=False, decoupled_weight_decay=True,
                   quantize=False, master_weight_bits=None, conv=conv)
    lr = float(np.float32(1e-3))
    exp = P.astype(np.float64) * (1 - lr * 1e-2) - lr * G
    np.testing.assert_allclose(r.param, exp, atol=1e-6, rtol=1e-6)


def test_sgd_without_momentum_keeps_no_buffer():
    # tests/test_sgd.py:93-100
    p = np.array([1.0, -2.0, 3.0], dtype=BF16)
    r = O.sgd_leaf(G, p, np.zeros(3, dtype=np.int8), None, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0,
                   nesterov=False, decoupled_weight_decay=False)
    assert r.mu is None and r.param.dtype == O.BF16


# ---- trajectories (tests/test_adamw.py:24-54, test_lion.py:24-51, test_sgd.py:32-59) ----


def _l2(*diffs):
    return np.sqrt(sum(float(np.vdot(d, d)) for d in diffs))


def test_adamw_tracks_float64_adamw_over_10_steps():
    w = np.array([[0.5, -1.0], [1.5, -0.25]], dtype=np.float32)
    b = np.array([0.1, -0.2], dtype=np.float32)
    gw = np.array([[0.3, -0.1], [0.2, -0.4]], dtype=np.float32)
    gb = np.array([0.05, -0.02], dtype=np.float32)
    out = []
    for p32, g in ((w, gw), (b, gb)):
        p = p32.astype(BF16)
        mu, nu, ecc = O.init_adam_leaf(p)
        ref = p32.astype(np.float64)
        m = np.zeros_like(ref)
        v = np.zeros_like(ref)
        for t in range(1, 11):
            bc1, bc2 = O.bias_corrections(0.9, 0.999, t)
            p, ecc, mu, nu = O.adam_leaf(g, p, ecc, mu, nu, lr=1e-2, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2,
                                         decoupled_weight_decay=True, bias_correction1=bc1, bias_correction2=bc2)
            m = 0.9 * m + 0.1 * g
            v = 0.999 * v + 0.001 * g.astype(np.float64) ** 2
            upd = (m / (1 - 0.9**t)) / (np.sqrt(v / (1 - 0.999**t)) + 1e-8) + 1e-2 * ref
            ref = ref - 1e-2 * upd
        out.append(O.reconstruct_leaf(p, ecc) - ref)
    assert _l2(*out) < 0.05


def test_state_layout_of_init():
    # tests/test_adamw.py:68-91,132-165,168-176: fp32 leaves still get quantized moments and no ECC
    bn = np.array([1.0, 0.5, -0.25, 0.75], dtype=np.float32)
    mu, nu, ecc = O.init_adam_leaf(bn)
    assert isinstance(mu, O.Quantized) and isinstance(nu, O.Quantized) and ecc is None
    assert mu.values.dtype == np.int8 and nu.values.dtype == np.uint8 and mu.scales.shape == (1,)
    w = np.zeros((65, 3), dtype=np.float16)
    mu, nu, ecc = O.init_adam_leaf(w, master_weight_bits=32)
    assert ecc.dtype == np.int16 and ecc.shape == w.shape and mu.scales.shape == (7,)
    _, _, ecc = O.init_adam_leaf(w.astype(BF16), master_weight_bits=None)
    assert ecc is None


def test_exhaustive_bf16_split_reconstruct_is_identity_on_bf16_grid():
    # idea of examples/plot_reconstruction_error.py:145-190: sweep every exponent x mantissa
    bits = np.arange(0, 1 << 16, dtype=np.uint16)
    lp = bits.view(BF16)
    finite = np.isfinite(lp.astype(np.float32))
    x = lp.astype(np.float32)[finite]
    for mwb in (24, 32):
        l2, ecc = O.split_leaf(x, BF16, mwb)
        np.testing.assert_array_equal(ecc, 0)
        # value equality: -0.0 + (+0.0 correction) comes back as +0.0, as it does in the reference
        np.testing.assert_array_equal(O.reconstruct_leaf(l2, ecc), x)


def test_ecc_bounds_and_error_shrinks_for_random_fp32():
    rng = np.random.default_rng(3)
    x = (rng.normal(0, 1, 200000) * np.exp2(rng.integers(-30, 30, 200000))).astype(np.float32)
    for dt, mwb, lim, gain in ((BF16, 24, 127, 100.0), (BF16, 32, 32767, 2e4), (np.float16, 24, 127, 100.0)):
        xs = x if dt is BF16 else np.clip(x, -6e4, 6e4)
        lp, ecc = O.split_leaf(xs, dt, mwb)
        assert np.abs(ecc.astype(np.int32)).max() <= lim
        rec = O.reconstruct_leaf(lp, ecc)
        plain = np.abs(xs - lp.astype(np.float32)).astype(np.float64)
        fixed = np.abs(xs - rec).astype(np.float64)
        normal = np.abs(xs) > (1e-30 if dt is BF16 else 1e-3)
        assert fixed[normal].sum() * gain * 0.5 < plain[normal].sum() + 1e-300


def test_clip_by_global_norm_known_answers():
    # a 3-4-5 triangle: norm 5, clipped to 1 -> 0.6, 0.8 (fp32 division then product, each rounded once)
    g = [np.array([3.0], dtype=np.float32), np.array([4.0], dtype=np.float32)]
    assert O.global_sq_norm(g) == 25.0
    out = O.clip_by_global_norm(g, 1.0)
    assert out[0][0] == np.float32(3.0) / np.float32(5.0) and out[1][0] == np.float32(4.0) / np.float32(5.0)
    # below the threshold nothing changes (norm < max_norm, strict)
    same = O.clip_by_global_norm(g, 5.5)
    assert same[0][0] == 3.0 and same[1][0] == 4.0
    at = O.clip_by_global_norm(g, 5.0)  # norm == max_norm rescales: (g / 5) * 5
    assert at[0][0] == (np.float32(3.0) / np.float32(5.0)) * np.float32(5.0)
    # 16-bit leaves: norm and max_norm are cast to the leaf dtype, quotient and product are rounded to it
    import ml_dtypes

    b = [np.array([3.0, -4.0, 0.0], dtype=ml_dtypes.bfloat16)]
    out = O.clip_by_global_norm(b, 0.3)
    m = np.float32(np.float32(0.3).astype(ml_dtypes.bfloat16))
    want = [(np.float32(np.float32(x / 5.0).astype(ml_dtypes.bfloat16)) * m).astype(ml_dtypes.bfloat16) for x in (3.0, -4.0, 0.0)]
    assert [float(v) for v in out[0]] == [float(w) for w in want] and out[0].dtype == ml_dtypes.bfloat16
