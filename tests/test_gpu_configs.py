"""Parity on the benchmark definition's own configurations, through the public surface (tx.init / tx.step),
every buffer of every leaf bit for bit against the C oracle:

  config 2  square bf16 matrices up to 16384 x 16384 under flash_adamw / flash_lion / flash_sgdw, 24- and
            32-bit master weights, gradients with a log-uniform sigma per step and 0.01 % outliers x100;
  config 3  the exact 161-leaf ResNet-50 pytree (bf16 convolutions, fp32 BatchNorm vectors and classifier
            bias) under flash_sgdw with the reference recipe's no-decay group;
  config 4  the exact 148-leaf GPT-2-small pytree under flash_adamw (24-bit master) and flash_lion.

The leaf lists are the ones bench.py times (bench.resnet50_shapes / gpt2_small_shapes).
"""

import os

import numpy as np
import pytest

import bench
from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

OPT_CODE = {"adamw": C.ADAM, "lion": C.LION, "sgdw": C.SGD}
SQUARE_HP = {"adamw": dict(learning_rate=1e-3, weight_decay=1e-2), "lion": dict(learning_rate=1e-4, weight_decay=1e-2),
             "sgdw": dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2)}


def _factory(opt):
    import flashoptim_jax_b200 as fo

    return {"adamw": fo.flash_adamw, "lion": fo.flash_lion, "sgdw": fo.flash_sgdw}[opt]


def _oracle_hyper(opt, t, hp):
    kw = dict(lr=hp["learning_rate"], wd=hp.get("weight_decay", 0.0))
    if opt == "lion":
        kw.update(b1=hp.get("b1", 0.9), b2=hp.get("b2", 0.99))
    if opt == "sgdw":
        kw.update(momentum=hp.get("momentum", 0.0))
    return H.hyper_tuple(OPT_CODE[opt], O.FUSED, t, **kw)


def _grad_like(p, sigma, outliers, gen):
    import torch

    g = torch.empty_like(p)
    bench.fill_grad(g, sigma, outliers, gen)
    return g


def _state_arrays(state, name, has_nu):
    ecc = state.ecc[name]
    return H.LeafArrays(None, None if ecc.dim() == 0 else H.to_numpy(ecc).reshape(-1), H.to_numpy(state.mu[name].values).reshape(-1),
                        H.to_numpy(state.mu[name].scales), H.to_numpy(state.nu[name].values).reshape(-1) if has_nu else None,
                        H.to_numpy(state.nu[name].scales) if has_nu else None)


@pytest.mark.parametrize("mwb", [24, 32])
@pytest.mark.parametrize("opt", ["adamw", "lion", "sgdw"])
@pytest.mark.parametrize("n,steps", [(1024, 10), (4096, 6), (16384, 2)])
def test_square_matrix_sweep(n, steps, opt, mwb):
    import torch

    C.set_threads(os.cpu_count() or 1)
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(n + mwb)
    rng = np.random.default_rng(n)
    hp = SQUARE_HP[opt]
    tx = _factory(opt)(master_weight_bits=mwb, donate=True, **hp)
    params = {"w": (torch.randn((n, n), device=dev, generator=gen) * 0.02).to(torch.bfloat16)}
    ref = H.fresh_leaf(H.to_numpy(params["w"]).reshape(-1), OPT_CODE[opt], C.STATE_QUANT, 8 if mwb == 24 else 16)
    state = tx.init(params)
    for t in range(1, steps + 1):
        sigma = float(10 ** rng.uniform(-4, -1))
        g = _grad_like(params["w"], sigma, 1e-4, gen)
        H.oracle_step(OPT_CODE[opt], H.to_numpy(g).reshape(-1), ref, C.STATE_QUANT, 32, _oracle_hyper(opt, t, hp))
        params, state = tx.step(params, state, {"w": g})
    torch.cuda.synchronize()
    got = _state_arrays(state, "w", opt == "adamw")
    got.param = H.to_numpy(params["w"]).reshape(-1)
    H.assert_leaf_equal(got, ref, f"{opt} {n}x{n} mwb{mwb}")


def _run_pytree(workload, steps=3):
    import torch

    C.set_threads(os.cpu_count() or 1)
    shapes_fn, opt, hparams, sigma, outliers = bench.WORKLOADS[workload]
    shapes = shapes_fn()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(7)
    params = {name: bench.make_param(shape, kind, dev, gen) for name, (shape, kind) in shapes.items()}
    mwb = hparams["master_weight_bits"]
    refs = {}
    for name, p in params.items():
        ecc_bits = 0 if p.dtype == torch.float32 else (8 if mwb == 24 else 16)
        refs[name] = H.fresh_leaf(H.to_numpy(p).reshape(-1), OPT_CODE[opt], C.STATE_QUANT, ecc_bits)
    tx = _factory(opt)(donate=True, **hparams)
    state = tx.init(params)
    groups = hparams.get("param_groups") or []
    for t in range(1, steps + 1):
        grads = {name: _grad_like(p, sigma, outliers, gen) for name, p in params.items()}
        for name, g in grads.items():
            hp = dict(hparams)
            for grp in groups:  # first matching group wins, as in the library
                if grp["params"]((name,), params[name]):
                    hp.update({k: v for k, v in grp.items() if k != "params"})
                    break
            H.oracle_step(OPT_CODE[opt], H.to_numpy(g).reshape(-1), refs[name], C.STATE_QUANT, 32, _oracle_hyper(opt, t, hp))
        params, state = tx.step(params, state, grads)
    torch.cuda.synchronize()
    assert int(state.count) == steps
    for name in shapes:
        got = _state_arrays(state, name, opt == "adamw")
        got.param = H.to_numpy(params[name]).reshape(-1)
        H.assert_leaf_equal(got, refs[name], f"{workload} {name}")
    return shapes


def test_resnet50_pytree_exact_leaf_list():
    shapes = _run_pytree("resnet50")
    kinds = [k for _, k in shapes.values()]
    assert len(shapes) == 161 and sum(bench.numel(s) for s, _ in shapes.values()) == 25557032
    assert sum(k.startswith("f32") for k in kinds) == 107 and sum(k.startswith("bf16") for k in kinds) == 54


@pytest.mark.parametrize("workload", ["gpt2_small", "gpt2_small_lion"])
def test_gpt2_small_pytree_exact_leaf_list(workload):
    shapes = _run_pytree(workload)
    assert len(shapes) == 148 and sum(bench.numel(s) for s, _ in shapes.values()) == 124439808
