"""fo_step through the C ABI against the CPU oracle: bit-exact params, ECC, codes, scales.

Every case runs several steps with a fresh seeded gradient per step so that dequantization
of non-trivial state and bias correction are exercised, on sizes that hit every tail shape
(shorter than a group, one element past a group / block / chunk boundary).
"""

import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 31, 32, 33, 65, 1023, 1024, 1025, 4095, 4096, 4097, 65 * 65, 3 * 4096 + 7, 40000]
PARAM_COMBOS = [(1, 8), (1, 16), (1, 0), (2, 8), (2, 16), (2, 0), (0, 0)]  # (param dtype code, ecc bits)
CONVS = {"fused": O.FUSED, "unfused": O.UNFUSED}


def _run_case(opt, pdt, ecc_bits, state, conv, n, *, gdt=1, steps=4, group_size=32, seed=0, sigma=1e-3, **hp_kw):
    import torch

    rng = np.random.default_rng(seed + n)
    pnp = rng.normal(0, 0.02, n).astype(np.float32).astype(H.NP_OF_CODE[pdt])
    ref = H.fresh_leaf(pnp, opt, state, ecc_bits, group_size)
    dev = ref.copy().to_device()
    for t in range(1, steps + 1):
        g = H.make_grad(rng, n, sigma, H.NP_OF_CODE[gdt], outliers=1e-3)
        hp = H.hyper_tuple(opt, conv, t, **hp_kw)
        H.oracle_step(opt, g, ref, state, group_size, hp)
        H.abi_step(opt, [H.to_torch(g)], [dev], state, group_size, [hp], [0], pdt, gdt, ecc_bits)
        torch.cuda.synchronize()
        H.assert_leaf_equal(dev.to_host(), ref, f"step {t} n={n}")


@pytest.mark.parametrize("conv", ["fused", "unfused"])
@pytest.mark.parametrize("pdt,ecc_bits", PARAM_COMBOS)
def test_adamw_quantized_all_tail_shapes(pdt, ecc_bits, conv):
    for n in SIZES:
        _run_case(C.ADAM, pdt, ecc_bits, C.STATE_QUANT, CONVS[conv], n, lr=1e-3, wd=1e-2)


@pytest.mark.parametrize("conv", ["fused", "unfused"])
@pytest.mark.parametrize("pdt,ecc_bits", PARAM_COMBOS)
def test_lion_quantized_all_tail_shapes(pdt, ecc_bits, conv):
    for n in SIZES:
        _run_case(C.LION, pdt, ecc_bits, C.STATE_QUANT, CONVS[conv], n, lr=1e-4, wd=1e-2, b2=0.99)


@pytest.mark.parametrize("nesterov", [False, True])
@pytest.mark.parametrize("decoupled", [False, True])
@pytest.mark.parametrize("pdt,ecc_bits", PARAM_COMBOS)
def test_sgd_quantized_all_tail_shapes(pdt, ecc_bits, decoupled, nesterov):
    for n in SIZES[::2]:
        _run_case(C.SGD, pdt, ecc_bits, C.STATE_QUANT, O.FUSED, n, lr=1e-2, wd=1e-2, momentum=0.9,
                  decoupled=decoupled, nesterov=nesterov)


@pytest.mark.parametrize("opt", [C.ADAM, C.LION, C.SGD], ids=["adam", "lion", "sgd"])
@pytest.mark.parametrize("pdt,ecc_bits", PARAM_COMBOS)
def test_full_precision_state(opt, pdt, ecc_bits):
    for n in (3, 65, 4097, 40000):
        _run_case(opt, pdt, ecc_bits, C.STATE_FULL, O.UNFUSED, n, lr=1e-3, wd=1e-2, decoupled=(opt != C.SGD))


@pytest.mark.parametrize("pdt,ecc_bits", PARAM_COMBOS)
def test_sgd_without_momentum_buffer(pdt, ecc_bits):
    for n in (3, 65, 4097):
        _run_case(C.SGD, pdt, ecc_bits, C.STATE_NONE, O.FUSED, n, lr=1e-2, wd=1e-2, decoupled=False)


def test_adam_coupled_weight_decay():
    for n in (65, 4097):
        _run_case(C.ADAM, 1, 8, C.STATE_QUANT, O.FUSED, n, lr=1e-3, wd=1e-2, decoupled=False)


@pytest.mark.parametrize("gdt", [0, 1, 2], ids=["g_f32", "g_bf16", "g_f16"])
@pytest.mark.parametrize("pdt,ecc_bits", [(1, 8), (0, 0), (2, 16)])
def test_grad_dtypes(pdt, ecc_bits, gdt):
    for n in (33, 4096 + 65, 40000):
        _run_case(C.ADAM, pdt, ecc_bits, C.STATE_QUANT, O.FUSED, n, gdt=gdt, lr=1e-3, wd=1e-2)


@pytest.mark.parametrize("group_size", [1, 2, 8, 16, 40, 64, 100, 128, 256, 512, 1000, 1024])
@pytest.mark.parametrize("opt", [C.ADAM, C.LION], ids=["adam", "lion"])
def test_other_group_sizes(opt, group_size):
    for n in (1, group_size, group_size + 1, 5000):
        _run_case(opt, 1, 8, C.STATE_QUANT, O.UNFUSED, n, group_size=group_size, lr=1e-3, wd=1e-2)


def test_many_steps_exercise_bias_correction_and_saturation():
    # 100 steps as in the square-matrix sweep, gradient scale changing per step, x100 outliers
    import torch

    rng = np.random.default_rng(7)
    n = 256 * 256
    for opt, kw in ((C.ADAM, dict(lr=1e-3, wd=1e-2)), (C.LION, dict(lr=1e-4, wd=1e-2, b2=0.99)),
                    (C.SGD, dict(lr=1e-2, wd=1e-2, momentum=0.9))):
        for ecc_bits in (8, 16):
            pnp = rng.normal(0, 0.02, n).astype(np.float32).astype(H.BF16)
            ref = H.fresh_leaf(pnp, opt, C.STATE_QUANT, ecc_bits)
            dev = ref.copy().to_device()
            for t in range(1, 101):
                sigma = float(np.exp(rng.uniform(np.log(1e-4), np.log(1e-1))))
                g = H.make_grad(rng, n, sigma, H.BF16, outliers=1e-4)
                hp = H.hyper_tuple(opt, O.FUSED, t, **kw)
                H.oracle_step(opt, g, ref, C.STATE_QUANT, 32, hp)
                H.abi_step(opt, [H.to_torch(g)], [dev], C.STATE_QUANT, 32, [hp], [0], 1, 1, ecc_bits)
            torch.cuda.synchronize()
            H.assert_leaf_equal(dev.to_host(), ref, f"opt {opt} ecc {ecc_bits} after 100 steps")


@pytest.mark.parametrize("opt,conv,hp_kw", [
    (C.ADAM, O.FUSED, dict(lr=1e-3, wd=1e-2)),
    (C.LION, O.FUSED, dict(lr=1e-4, wd=1e-2, b2=0.99)),
    (C.LION, O.UNFUSED, dict(lr=1e-4, wd=1e-2, b2=0.99)),
    (C.SGD, O.FUSED, dict(lr=1e-2, wd=1e-2, momentum=0.9)),
], ids=["adam", "lion-fused", "lion-unfused", "sgd"])
def test_extreme_values_take_the_guarded_paths(opt, conv, hp_kw):
    # zeros, subnormals, huge and tiny gradients and weights: exercises every fallback of the shortcuts
    # (scattered exact zeros also give Lion interpolations that are exactly zero, whose sign is zero)
    import torch

    rng = np.random.default_rng(11)
    n = 8192
    expo = rng.integers(-140, 60, n)
    base = rng.normal(0, 1, n)
    p32 = np.ldexp(base, np.clip(expo, -140, 30)).astype(np.float32)
    p32[::7] = 0.0
    for pdt, ecc_bits in ((1, 8), (1, 16), (2, 16), (0, 0)):
        pnp = (np.clip(p32, -1e3, 1e3) if pdt == 2 else p32).astype(H.NP_OF_CODE[pdt])  # keep fp16 finite
        ref = H.fresh_leaf(pnp, opt, C.STATE_QUANT, ecc_bits)
        dev = ref.copy().to_device()
        for t in range(1, 4):
            g32 = np.ldexp(rng.normal(0, 1, n), rng.integers(-140, 12, n)).astype(np.float32)  # |m| stays below the fp16 scale range
            g32[::5] = 0.0
            g32[64:128] = 0.0  # whole groups of zeros
            hp = H.hyper_tuple(opt, conv, t, **hp_kw)
            H.oracle_step(opt, g32, ref, C.STATE_QUANT, 32, hp)
            H.abi_step(opt, [H.to_torch(g32)], [dev], C.STATE_QUANT, 32, [hp], [0], pdt, 0, ecc_bits)
            torch.cuda.synchronize()
            H.assert_leaf_equal(dev.to_host(), ref, f"extreme opt {opt} pdt {pdt} ecc {ecc_bits} step {t}")


def test_untamed_hyper_parameters_use_ieee_divisions():
    # eps = 0 and eps far below the guard: the Adam denominator must fall back to the true division
    for eps in (0.0, 1e-30):
        _run_case(C.ADAM, 1, 8, C.STATE_QUANT, O.FUSED, 4097, lr=1e-3, wd=0.0, eps=eps, sigma=1e-2)
