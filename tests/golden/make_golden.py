"""Generates the golden fixtures in this directory from the NumPy oracle.

    python tests/golden/make_golden.py

The reference is a JAX program and JAX is not installed here, so these vectors come from the
oracle (the restatement of the reference's code), not from a run of the reference itself.
They pin the C oracle and the CUDA library against drift; config 1 of the benchmark
definition (2048x2048 bf16 AdamW, 10 steps) is stored as SHA-256 digests of its final arrays.
"""

import hashlib
import json
import os
import sys

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import flashoptim_oracle as O  # noqa: E402

BF16 = np.dtype(ml_dtypes.bfloat16)


def small_case(seed, n, dtype, mwb, opt, conv, steps=3):
    rng = np.random.default_rng(seed)
    p = rng.normal(0, 0.02, n).astype(np.float32).astype(dtype)
    grads = [rng.normal(0, 1e-3, n).astype(np.float32).astype(BF16) for _ in range(steps)]
    out = {"param0": p.view(np.uint16) if p.dtype.itemsize == 2 else p, "grads": np.stack([g.view(np.uint16) for g in grads])}
    if opt == "adamw":
        mu, nu, ecc = O.init_adam_leaf(p, 32, True, mwb)
        for t, g in enumerate(grads, 1):
            bc1, bc2 = O.bias_corrections(0.9, 0.999, t)
            p, ecc, mu, nu = O.adam_leaf(g, p, ecc, mu, nu, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2,
                                         decoupled_weight_decay=True, bias_correction1=bc1, bias_correction2=bc2,
                                         master_weight_bits=mwb, conv=conv)
        out.update(nu=nu.values, nu_scales=nu.scales.view(np.uint16))
    elif opt == "lion":
        mu, ecc = O.init_momentum_leaf(p, 32, True, mwb)
        for g in grads:
            p, ecc, mu = O.lion_leaf(g, p, ecc, mu, lr=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2, master_weight_bits=mwb, conv=conv)
    else:
        mu, ecc = O.init_momentum_leaf(p, 32, True, mwb)
        for g in grads:
            p, ecc, mu = O.sgd_leaf(g, p, ecc, mu, lr=1e-2, momentum=0.9, dampening=0.0, weight_decay=1e-2, nesterov=False,
                                    decoupled_weight_decay=True, master_weight_bits=mwb, conv=conv)
    out.update(param=p.view(np.uint16) if p.dtype.itemsize == 2 else p, mu=mu.values, mu_scales=mu.scales.view(np.uint16))
    if ecc is not None:
        out["ecc"] = ecc
    return out


def config1_digests():
    """BASELINE config 1: one 2048x2048 bf16 matrix N(0, 0.02), grads bf16 N(0, 1e-3), 10 AdamW steps, seed 0."""
    from oracle import c_oracle as C
    from tests import helpers as H

    digests = {}
    for conv in (O.FUSED, O.UNFUSED):
        rng = np.random.default_rng(0)
        p = rng.normal(0, 0.02, (2048, 2048)).astype(np.float32).astype(BF16)
        leaf = H.fresh_leaf(p.reshape(-1), C.ADAM, C.STATE_QUANT, 8)
        for t in range(1, 11):
            g = rng.normal(0, 1e-3, 2048 * 2048).astype(np.float32).astype(BF16)
            H.oracle_step(C.ADAM, g, leaf, C.STATE_QUANT, 32, H.hyper_tuple(C.ADAM, conv, t, lr=1e-3, wd=1e-2))
        theta = C.reconstruct(leaf.param, leaf.ecc)
        digests[conv.name] = {f: hashlib.sha256(np.ascontiguousarray(getattr(leaf, f)).tobytes()).hexdigest() for f in leaf.fields()}
        digests[conv.name]["reconstructed_fp32"] = hashlib.sha256(theta.tobytes()).hexdigest()
    return digests


def main():
    cases = {}
    for i, (n, dtype, mwb, opt, conv) in enumerate([
        (2048 + 65, BF16, 24, "adamw", O.FUSED), (2048 + 65, BF16, 32, "adamw", O.UNFUSED),
        (1000, np.dtype(np.float16), 32, "adamw", O.FUSED), (777, BF16, 24, "lion", O.FUSED),
        (777, BF16, 24, "lion", O.UNFUSED), (2111, BF16, 32, "sgdw", O.FUSED), (300, np.dtype(np.float32), None, "adamw", O.FUSED),
    ]):
        name = f"case{i}_{opt}_{np.dtype(dtype).name}_mwb{mwb}_{conv.name}"
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **small_case(1000 + i, n, dtype, mwb, opt, conv))
        cases[name] = {"n": n, "dtype": np.dtype(dtype).name, "master_weight_bits": mwb, "optimizer": opt, "convention": conv.name}
    with open(os.path.join(HERE, "cases.json"), "w") as f:
        json.dump(cases, f, indent=1)
    with open(os.path.join(HERE, "config1_digests.json"), "w") as f:
        json.dump(config1_digests(), f, indent=1)


if __name__ == "__main__":
    main()
