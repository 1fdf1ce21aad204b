"""The C restatement of the oracle against the NumPy one, bit for bit (CPU only)."""

import ml_dtypes
import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

BF16 = np.dtype(ml_dtypes.bfloat16)


def test_every_fp16_pattern_converts_like_numpy():
    bits = np.arange(1 << 16, dtype=np.uint16)
    h = bits.view(np.float16)
    finite = np.isfinite(h.astype(np.float32))
    # dequantize_momentum with code 127 returns exactly the scale: exercises fp16 -> fp32 of every pattern
    scales = h[finite & (h >= 0)]
    vals = np.full(scales.size * 32, 127, dtype=np.int8)
    out = C.dequantize_momentum(vals, scales.copy(), 32)[::32]
    np.testing.assert_array_equal(out.view(np.uint32), scales.astype(np.float32).view(np.uint32))


def test_fp32_to_fp16_rounding_matches_numpy_on_ties_subnormals_and_overflow():
    rng = np.random.default_rng(0)
    x = np.abs(np.concatenate([
        rng.normal(0, 1, 200000) * np.exp2(rng.integers(-30, 17, 200000)),
        np.arange(1 << 16, dtype=np.uint16).view(np.float16).astype(np.float32)[:0x7C00],           # exact halves
        (np.arange(1 << 16, dtype=np.uint16).view(np.float16).astype(np.float64)[:0x7BFF] +
         np.arange(1, 1 << 16, dtype=np.uint16).view(np.float16).astype(np.float64)[:0x7BFF]) / 2,  # exact ties
    ])).astype(np.float32)
    x = x[x < 65520.0]
    # quantize_momentum stores fp16(absmax) per group: one value per group
    groups = np.zeros((x.size, 32), dtype=np.float32)
    groups[:, 0] = x
    _, scales = C.quantize_momentum(groups.ravel(), 32)
    np.testing.assert_array_equal(scales.view(np.uint16), x.astype(np.float16).view(np.uint16))


def test_fp32_to_bf16_matches_ml_dtypes():
    rng = np.random.default_rng(1)
    x = (rng.normal(0, 1, 300000) * np.exp2(rng.integers(-140, 120, 300000))).astype(np.float32)
    lp, _ = C.split(x, BF16, 0)
    np.testing.assert_array_equal(lp.view(np.uint16), x.astype(BF16).view(np.uint16))


@pytest.mark.parametrize("group_size", [32, 8, 40, 1024])
def test_codecs_match(group_size):
    rng = np.random.default_rng(2)
    for n in (1, 31, 65, 4097):
        x = (rng.normal(0, 1, n) * np.exp2(rng.integers(-20, 4, n))).astype(np.float32)
        x[::9] = 0
        for conv, flags in ((O.UNFUSED, 0), (O.FUSED, C.FLAG_SCALE_FLOOR)):
            q = O.quantize_momentum(x, group_size, conv)
            v, s = C.quantize_momentum(x, group_size, flags)
            np.testing.assert_array_equal(v, q.values)
            np.testing.assert_array_equal(s.view(np.uint16), q.scales.view(np.uint16))
            np.testing.assert_array_equal(C.dequantize_momentum(v, s, group_size).view(np.uint32),
                                          O.dequantize_momentum(q, group_size).view(np.uint32))
            q = O.quantize_variance(x * x, group_size, conv)
            v, s = C.quantize_variance(x * x, group_size, flags)
            np.testing.assert_array_equal(v, q.values)
            np.testing.assert_array_equal(s.view(np.uint16), q.scales.view(np.uint16))
            np.testing.assert_array_equal(C.dequantize_variance(v, s, group_size).view(np.uint32),
                                          O.dequantize_variance(q, group_size).view(np.uint32))


@pytest.mark.parametrize("dt,mwb", [(BF16, 24), (BF16, 32), (np.dtype(np.float16), 24), (np.dtype(np.float16), 32)])
def test_split_reconstruct_match(dt, mwb):
    rng = np.random.default_rng(3)
    x = (rng.normal(0, 1, 100000) * np.exp2(rng.integers(-140 if dt == BF16 else -30, 30 if dt == BF16 else 10, 100000))).astype(np.float32)
    x[::11] = 0
    lp, ecc = O.split_leaf(x, dt, mwb)
    clp, cecc = C.split(x, dt, 8 if mwb == 24 else 16)
    np.testing.assert_array_equal(clp.view(np.uint16), lp.view(np.uint16))
    np.testing.assert_array_equal(cecc, ecc)
    np.testing.assert_array_equal(C.reconstruct(lp, ecc).view(np.uint32), O.reconstruct_leaf(lp, ecc).view(np.uint32))


def _numpy_steps(opt, pnp, grads, conv, mwb, quantize, group_size, **kw):
    """Run the NumPy oracle for len(grads) steps; returns the final LeafArrays."""
    param = pnp
    if opt == C.ADAM:
        mu, nu, ecc = O.init_adam_leaf(param, group_size, quantize, mwb)
    else:
        mu, ecc = O.init_momentum_leaf(param, group_size, quantize, mwb, use_momentum=kw.get("momentum", 0.9) > 0 or opt == C.LION)
        nu = None
    for t, g in enumerate(grads, start=1):
        if opt == C.ADAM:
            bc1, bc2 = O.bias_corrections(0.9, 0.999, t)
            r = O.adam_leaf(g, param, ecc, mu, nu, lr=kw["lr"], b1=0.9, b2=0.999, eps=1e-8, weight_decay=kw["wd"],
                            decoupled_weight_decay=kw.get("decoupled", True), bias_correction1=bc1, bias_correction2=bc2,
                            quantize=quantize, group_size=group_size, master_weight_bits=mwb, conv=conv)
            param, ecc, mu, nu = r
        elif opt == C.LION:
            r = O.lion_leaf(g, param, ecc, mu, lr=kw["lr"], b1=0.9, b2=0.99, weight_decay=kw["wd"], quantize=quantize,
                            group_size=group_size, master_weight_bits=mwb, conv=conv)
            param, ecc, mu = r
        else:
            r = O.sgd_leaf(g, param, ecc, mu, lr=kw["lr"], momentum=kw.get("momentum", 0.9), dampening=kw.get("dampening", 0.0),
                           weight_decay=kw["wd"], nesterov=kw.get("nesterov", False), decoupled_weight_decay=kw.get("decoupled", True),
                           quantize=quantize, group_size=group_size, master_weight_bits=mwb, conv=conv)
            param, ecc, mu = r

    def split_q(x):
        if x is None:
            return None, None
        if isinstance(x, O.Quantized):
            return x.values, x.scales
        return x, None

    m, ms = split_q(mu)
    v, vs = split_q(nu)
    return H.LeafArrays(param, ecc, m, ms, v, vs)


CASES = [
    (C.ADAM, dict(lr=1e-3, wd=1e-2)), (C.ADAM, dict(lr=1e-3, wd=1e-2, decoupled=False)),
    (C.LION, dict(lr=1e-4, wd=1e-2, b2=0.99)),
    (C.SGD, dict(lr=1e-2, wd=1e-2, momentum=0.9)), (C.SGD, dict(lr=1e-2, wd=1e-2, momentum=0.9, nesterov=True, decoupled=False)),
    (C.SGD, dict(lr=1e-2, wd=1e-2, momentum=0.9, dampening=0.1)), (C.SGD, dict(lr=1e-2, wd=1e-2, momentum=0.0)),
]


@pytest.mark.parametrize("conv", [O.UNFUSED, O.FUSED], ids=["unfused", "fused"])
@pytest.mark.parametrize("pdt,mwb", [(1, 24), (1, 32), (2, 24), (2, 32), (1, None), (0, None)])
@pytest.mark.parametrize("quantize", [True, False], ids=["quant", "full"])
def test_leaf_steps_match(pdt, mwb, quantize, conv):
    rng = np.random.default_rng(5)
    for opt, kw in CASES:
        for n in (3, 65, 1000):
            pnp = rng.normal(0, 0.02, n).astype(np.float32).astype(H.NP_OF_CODE[pdt])
            grads = [H.make_grad(rng, n, 1e-3, BF16 if pdt else np.float32, outliers=0.01) for _ in range(3)]
            want = _numpy_steps(opt, pnp, grads, conv, mwb, quantize, 32, **kw)
            use_mom = not (opt == C.SGD and kw.get("momentum", 0.9) == 0.0)
            state = C.STATE_NONE if not use_mom else (C.STATE_QUANT if quantize else C.STATE_FULL)
            ecc_bits = 0 if (mwb is None or pdt == 0) else (8 if mwb == 24 else 16)
            got = H.fresh_leaf(pnp, opt, state, ecc_bits)
            for t, g in enumerate(grads, start=1):
                hk = {k: v for k, v in kw.items() if k != "b2"}
                if opt == C.LION:
                    hk["b2"] = 0.99
                H.oracle_step(opt, g, got, state, 32, H.hyper_tuple(opt, conv, t, **hk))
            H.assert_leaf_equal(got, want, f"opt {opt} {kw} n={n}")


@pytest.mark.parametrize("group_size", [1, 8, 40, 64, 1000])
def test_leaf_steps_match_other_group_sizes(group_size):
    rng = np.random.default_rng(6)
    for opt, kw in CASES[:3]:
        n = 2500
        pnp = rng.normal(0, 0.02, n).astype(np.float32).astype(BF16)
        grads = [H.make_grad(rng, n, 1e-3, BF16) for _ in range(3)]
        want = _numpy_steps(opt, pnp, grads, O.UNFUSED, 24, True, group_size, **kw)
        got = H.fresh_leaf(pnp, opt, C.STATE_QUANT, 8, group_size)
        for t, g in enumerate(grads, start=1):
            hk = {k: v for k, v in kw.items() if k != "b2"}
            if opt == C.LION:
                hk["b2"] = 0.99
            H.oracle_step(opt, g, got, C.STATE_QUANT, group_size, H.hyper_tuple(opt, O.UNFUSED, t, **hk))
        H.assert_leaf_equal(got, want, f"opt {opt} g={group_size}")
