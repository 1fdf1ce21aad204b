"""Randomised parity: optimizer, dtypes, ECC width, state kind, convention, leaf sizes (ragged, tiny,
large), parameter and gradient scales, exact zeros and outliers all drawn at random; every buffer of
every leaf must equal the C oracle bit for bit after a few multi-tensor steps."""

import ml_dtypes
import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

SIZES = [1, 31, 32, 33, 2047, 2048, 2049, 4096, 6144 + 5, 100000, 262144]


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_configurations_match_the_oracle(seed):
    import torch

    rng = np.random.default_rng(seed)
    for case in range(25):
        opt = int(rng.choice([C.ADAM, C.LION, C.SGD]))
        pdt = int(rng.choice([0, 1, 1, 1, 2]))
        ecc_bits = 0 if pdt == 0 else int(rng.choice([0, 8, 16]))
        gdt = int(rng.choice([0, 1, 2])) if pdt != 0 else 0
        state = int(rng.choice([C.STATE_QUANT, C.STATE_QUANT, C.STATE_FULL]))
        conv = O.FUSED if rng.random() < 0.7 else O.UNFUSED
        sizes = [int(rng.choice(SIZES)) for _ in range(int(rng.integers(1, 6)))]
        g_np = {0: np.float32, 1: ml_dtypes.bfloat16, 2: np.float16}[gdt]
        pscale = float(rng.choice([0.02, 1.0, 1e-3]))
        refs = []
        for n in sizes:
            p = rng.normal(0, pscale, n).astype(np.float32)
            if rng.random() < 0.3:
                p[rng.random(n) < 0.2] = 0.0
            refs.append(H.fresh_leaf(p.astype(H.NP_OF_CODE[pdt]), opt, state, ecc_bits))
        devs = [r.copy().to_device() for r in refs]
        gscale = float(10 ** rng.uniform(-6, 0))
        kw = dict(lr=float(10 ** rng.uniform(-4, -1)), wd=float(rng.choice([0.0, 1e-2, 0.1])))
        for t in range(1, int(rng.integers(1, 5)) + 1):
            grads = [H.make_grad(rng, n, gscale, g_np, outliers=1e-3) for n in sizes]
            if rng.random() < 0.3:
                for g in grads:
                    g[rng.random(g.shape[0]) < 0.3] = 0
            hp = H.hyper_tuple(opt, conv, t, **kw)
            for g, r in zip(grads, refs):
                H.oracle_step(opt, g, r, state, 32, hp)
            H.abi_step(opt, [H.to_torch(g) for g in grads], devs, state, 32, [hp], [0] * len(sizes), pdt, gdt, ecc_bits)
        torch.cuda.synchronize()
        what = f"seed {seed} case {case}: opt {opt} pdt {pdt} ecc {ecc_bits} gdt {gdt} state {state} {conv} sizes {sizes} gscale {gscale:.3g} {kw}"
        for i, (d, r) in enumerate(zip(devs, refs)):
            H.assert_leaf_equal(d.to_host(), r, f"{what} leaf {i}")
