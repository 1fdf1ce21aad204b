"""Committed golden vectors (tests/golden): outputs of the reference's own source files, imported
unmodified over a NumPy stand-in for `jax` by tests/golden/make_golden.py and driven through the
reference's public API (`fused=True`: its Pallas kernel text, `fused=False`: its jnp text).

CPU: the NumPy oracle and the C oracle must reproduce them bit for bit, and when a checkout of
the reference is present the generator is re-run and must reproduce the committed files.  GPU:
the CUDA library, through the Python surface (tx.init / tx.step) and the codec entry points,
must reproduce them, and benchmark config 1 (2048x2048 bf16 AdamW, 10 steps) must hash to the
stored digests in both conventions.
"""

import hashlib
import json
import os
import subprocess
import sys

import ml_dtypes
import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = json.load(open(os.path.join(GOLD, "cases.json")))
NP_DT = {"bfloat16": np.dtype(ml_dtypes.bfloat16), "float16": np.dtype(np.float16), "float32": np.dtype(np.float32)}
OPT = {"adamw": C.ADAM, "lion": C.LION, "sgdw": C.SGD}
KW = {"adamw": dict(lr=1e-3, wd=1e-2), "lion": dict(lr=1e-4, wd=1e-2, b2=0.99), "sgdw": dict(lr=1e-2, wd=1e-2, momentum=0.9)}


def _load(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    meta = CASES[name]
    dt = NP_DT[meta["dtype"]]
    p0 = z["param0"].view(dt) if dt.itemsize == 2 else z["param0"]
    want = H.LeafArrays(z["param"].view(dt) if dt.itemsize == 2 else z["param"], z["ecc"] if "ecc" in z else None, z["mu"],
                        z["mu_scales"].view(np.float16), z["nu"] if "nu" in z else None,
                        z["nu_scales"].view(np.float16) if "nu_scales" in z else None)
    grads = [g.view(H.BF16) for g in z["grads"]]
    return meta, p0, grads, want


@pytest.mark.parametrize("name", sorted(CASES))
def test_c_oracle_reproduces_golden(name):
    meta, p0, grads, want = _load(name)
    opt, conv = OPT[meta["optimizer"]], (O.FUSED if meta["convention"] == "fused" else O.UNFUSED)
    ecc_bits = {None: 0, 24: 8, 32: 16}[meta["master_weight_bits"]] if p0.dtype.itemsize == 2 else 0
    leaf = H.fresh_leaf(p0, opt, C.STATE_QUANT, ecc_bits)
    for t, g in enumerate(grads, 1):
        H.oracle_step(opt, g, leaf, C.STATE_QUANT, 32, H.hyper_tuple(opt, conv, t, **KW[meta["optimizer"]]))
    H.assert_leaf_equal(leaf, want, name)


@pytest.mark.parametrize("name", sorted(CASES))
def test_numpy_oracle_reproduces_golden(name):
    meta, p0, grads, want = _load(name)
    conv = O.FUSED if meta["convention"] == "fused" else O.UNFUSED
    mwb, opt = meta["master_weight_bits"], meta["optimizer"]
    p = p0.copy()
    nu = None
    if opt == "adamw":
        mu, nu, ecc = O.init_adam_leaf(p, 32, True, mwb)
        for t, g in enumerate(grads, 1):
            bc1, bc2 = O.bias_corrections(0.9, 0.999, t)
            p, ecc, mu, nu = O.adam_leaf(g, p, ecc, mu, nu, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2,
                                         decoupled_weight_decay=True, bias_correction1=bc1, bias_correction2=bc2,
                                         master_weight_bits=mwb, conv=conv)
    elif opt == "lion":
        mu, ecc = O.init_momentum_leaf(p, 32, True, mwb)
        for g in grads:
            p, ecc, mu = O.lion_leaf(g, p, ecc, mu, lr=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2, master_weight_bits=mwb, conv=conv)
    else:
        mu, ecc = O.init_momentum_leaf(p, 32, True, mwb)
        for g in grads:
            p, ecc, mu = O.sgd_leaf(g, p, ecc, mu, lr=1e-2, momentum=0.9, dampening=0.0, weight_decay=1e-2, nesterov=False,
                                    decoupled_weight_decay=True, master_weight_bits=mwb, conv=conv)
    got = H.LeafArrays(p, ecc, mu.values, mu.scales, None if nu is None else nu.values, None if nu is None else nu.scales)
    H.assert_leaf_equal(got, want, name)


def _codecs():
    z = np.load(os.path.join(GOLD, "codecs.npz"))
    return {k: z[k] for k in z.files}


CODEC_SPLITS = [("bf16_8", H.BF16, 24, 8), ("bf16_16", H.BF16, 32, 16), ("f16_8", np.dtype(np.float16), 24, 8),
                ("f16_16", np.dtype(np.float16), 32, 16)]


def _eq(a, b, what):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.dtype.itemsize == b.dtype.itemsize and a.shape == b.shape, what
    bad = np.flatnonzero(H.bits(a).ravel() != H.bits(b).ravel())
    assert bad.size == 0, f"{what}: {bad.size} differ, first {bad[:5]}"


@pytest.mark.parametrize("which", ["numpy", "c"])
def test_oracle_codecs_reproduce_reference_vectors(which):
    """quantize_/dequantize_momentum/variance, split_leaf, reconstruct_leaf as the reference computed them
    (all-zero group, ragged tail, magnitudes from e-12 to e+4, a value below 2**-119)."""
    z = _codecs()
    x, v, theta = z["x"], z["v"], z["theta"]
    if which == "numpy":
        qm, qv = O.quantize_momentum(x, 32), O.quantize_variance(v, 32)
        qm, qv = (qm.values, qm.scales), (qv.values, qv.scales)
        dqm = O.dequantize_momentum(O.Quantized(z["qm_values"], z["qm_scales"].view(np.float16)), 32)
        dqv = O.dequantize_variance(O.Quantized(z["qv_values"], z["qv_scales"].view(np.float16)), 32)
    else:
        qm, qv = C.quantize_momentum(x, 32), C.quantize_variance(v, 32)
        dqm = C.dequantize_momentum(z["qm_values"], z["qm_scales"].view(np.float16), 32)
        dqv = C.dequantize_variance(z["qv_values"], z["qv_scales"].view(np.float16), 32)
    _eq(qm[0], z["qm_values"], "momentum codes")
    _eq(qm[1], z["qm_scales"], "momentum scales")
    _eq(qv[0], z["qv_values"], "variance codes")
    _eq(qv[1], z["qv_scales"], "variance scales")
    _eq(dqm, z["dqm"], "dequantized momentum")
    _eq(dqv, z["dqv"], "dequantized variance")
    for tag, dt, mwb, ecc_bits in CODEC_SPLITS:
        if which == "numpy":
            lp, ecc = O.split_leaf(theta, dt, mwb)
            rec = O.reconstruct_leaf(z[f"lp_{tag}"].view(dt), z[f"ecc_{tag}"])
        else:
            lp, ecc = C.split(theta, dt, ecc_bits)
            rec = C.reconstruct(z[f"lp_{tag}"].view(dt), z[f"ecc_{tag}"])
        _eq(lp, z[f"lp_{tag}"], f"lp {tag}")
        _eq(ecc, z[f"ecc_{tag}"], f"ecc {tag}")
        _eq(rec, z[f"recon_{tag}"], f"reconstruct {tag}")


REFERENCE = os.environ.get("FLASHOPTIM_REFERENCE", "/root/reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "flashoptim_jax")), reason="no checkout of the reference here")
def test_fixtures_are_the_reference_output():
    """Re-runs the generator (reference sources imported unmodified over the stand-in) and compares
    with the committed fixtures."""
    r = subprocess.run([sys.executable, os.path.join(GOLD, "make_golden.py"), "--reference", REFERENCE, "--check"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "tests")), reason="no checkout of the reference here")
def test_reference_tests_pass_on_the_standin():
    """The stand-in is itself checked by the reference's own test-suite (closed-form steps at 1e-7,
    rounding ties, state layout, fused-vs-unfused agreement); tests that need optax or a GPU skip."""
    standin = os.path.join(os.path.dirname(GOLD), "jax_standin")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([standin, REFERENCE]))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(REFERENCE, "tests"), "-q", "-p", "no:cacheprovider"],
                       capture_output=True, text=True, timeout=600, env=env, cwd="/tmp")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout and "failed" not in r.stdout


@pytest.mark.gpu
def test_cuda_codecs_reproduce_reference_vectors():
    import flashoptim_jax_b200 as fo

    z = _codecs()
    qm = fo.quantize_momentum(H.to_torch(z["x"]), 32)
    qv = fo.quantize_variance(H.to_torch(z["v"]), 32)
    _eq(H.to_numpy(qm.values), z["qm_values"], "momentum codes")
    _eq(H.to_numpy(qm.scales), z["qm_scales"], "momentum scales")
    _eq(H.to_numpy(qv.values), z["qv_values"], "variance codes")
    _eq(H.to_numpy(qv.scales), z["qv_scales"], "variance scales")
    gm = fo.QuantizedArray(H.to_torch(z["qm_values"]), H.to_torch(z["qm_scales"].view(np.float16)))
    gv = fo.QuantizedArray(H.to_torch(z["qv_values"]), H.to_torch(z["qv_scales"].view(np.float16)))
    _eq(H.to_numpy(fo.dequantize_momentum(gm, 32)), z["dqm"], "dequantized momentum")
    _eq(H.to_numpy(fo.dequantize_variance(gv, 32)), z["dqv"], "dequantized variance")
    import torch

    for tag, dt, mwb, _ in CODEC_SPLITS:
        tdt = torch.bfloat16 if dt == H.BF16 else torch.float16
        lp, ecc = fo.split_leaf(H.to_torch(z["theta"]), narrow_dtype=tdt, master_weight_bits=mwb)
        _eq(H.to_numpy(lp), z[f"lp_{tag}"], f"lp {tag}")
        _eq(H.to_numpy(ecc), z[f"ecc_{tag}"], f"ecc {tag}")
        rec = fo.reconstruct_leaf(H.to_torch(z[f"lp_{tag}"].view(dt)), H.to_torch(z[f"ecc_{tag}"]))
        _eq(H.to_numpy(rec), z[f"recon_{tag}"], f"reconstruct {tag}")


@pytest.mark.gpu
@pytest.mark.parametrize("donate", [False, True], ids=["copy", "donate"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_python_surface_reproduces_golden(name, donate):
    import torch

    import flashoptim_jax_b200 as fo

    meta, p0, grads, want = _load(name)
    fused = meta["convention"] == "fused"
    mwb = meta["master_weight_bits"]
    if meta["optimizer"] == "adamw":
        tx = fo.flash_adamw(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=mwb, fused=fused, donate=donate)
    elif meta["optimizer"] == "lion":
        tx = fo.flash_lion(learning_rate=1e-4, weight_decay=1e-2, master_weight_bits=mwb, fused=fused, donate=donate)
    else:
        tx = fo.flash_sgdw(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2, master_weight_bits=mwb, fused=fused, donate=donate)
    params = {"x": H.to_torch(p0)}
    before = params["x"].clone()
    state = tx.init(params)
    for g in grads:
        new_params, state = tx.step(params, state, {"x": H.to_torch(g)})
        if not donate:
            assert torch.equal(params["x"], before)  # inputs stay untouched without donation
        params = new_params
        before = params["x"].clone()
    torch.cuda.synchronize()
    assert int(state.count) == len(grads)
    ecc = state.ecc["x"]
    got = H.LeafArrays(H.to_numpy(params["x"]), None if ecc.dim() == 0 else H.to_numpy(ecc), H.to_numpy(state.mu["x"].values),
                       H.to_numpy(state.mu["x"].scales),
                       H.to_numpy(state.nu["x"].values) if hasattr(state, "nu") else None,
                       H.to_numpy(state.nu["x"].scales) if hasattr(state, "nu") else None)
    H.assert_leaf_equal(got, want, name)


VARIANTS = json.load(open(os.path.join(GOLD, "variants.json")))
SCHEDULES = {"@halving": lambda count: 1e-3 * 0.5 ** int(count)}  # as in tests/golden/make_golden.py
VARIANT_OPT = {"flash_adam": (C.ADAM, False), "flash_adamw": (C.ADAM, True), "flash_lion": (C.LION, True),
               "flash_sgd": (C.SGD, False), "flash_sgdw": (C.SGD, True)}  # constructor -> (optimizer, decoupled weight decay)


def _load_variant(name):
    meta = VARIANTS[name]
    z = np.load(os.path.join(GOLD, f"variant_{name}.npz"))
    dt, gdt = NP_DT[meta["dtype"]], NP_DT[meta["grad_dtype"]]
    view = lambda a, d: a.view(d) if d.itemsize == 2 else a  # noqa: E731
    want = H.LeafArrays(view(z["param"], dt), z["ecc"] if "ecc" in z else None,
                        z["mu"] if "mu" in z else (z["mu_full"] if "mu_full" in z else None),
                        z["mu_scales"].view(np.float16) if "mu_scales" in z else None,
                        z["nu"] if "nu" in z else (z["nu_full"] if "nu_full" in z else None),
                        z["nu_scales"].view(np.float16) if "nu_scales" in z else None)
    return meta, view(z["param0"], dt), [view(g, gdt) for g in z["grads"]], want


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_c_oracle_reproduces_variants(name):
    """The other constructors and options of the reference's surface (coupled weight decay, Nesterov, dampening, no
    momentum buffer, full-precision moments, other group sizes, betas and eps, fp32 / fp16 gradients)."""
    meta, p0, grads, want = _load_variant(name)
    kw = meta["kwargs"]
    opt, decoupled = VARIANT_OPT[meta["constructor"]]
    no_buffer = opt == C.SGD and kw.get("momentum", 0.0) == 0.0
    state = C.STATE_NONE if no_buffer else (C.STATE_QUANT if kw.get("quantize", True) else C.STATE_FULL)
    conv = O.FUSED if kw.get("fused", True) and not no_buffer else O.UNFUSED
    ecc_bits = {None: 0, 24: 8, 32: 16}[kw["master_weight_bits"]] if p0.dtype.itemsize == 2 else 0
    gs = kw.get("group_size", 32)
    hyper = dict(lr=kw["learning_rate"], wd=kw.get("weight_decay", 0.0), decoupled=decoupled)
    for k in ("b1", "b2", "eps", "momentum", "dampening", "nesterov"):
        if k in kw:
            hyper[k] = kw[k]
    if opt == C.LION:
        hyper.setdefault("b2", 0.99)
        hyper.pop("decoupled")
    if opt == C.SGD:
        hyper.setdefault("momentum", 0.0)
    leaf = H.fresh_leaf(p0, opt, state, ecc_bits, gs)
    schedule = SCHEDULES.get(kw["learning_rate"]) if isinstance(kw["learning_rate"], str) else None
    for t, g in enumerate(grads, 1):
        if schedule is not None:
            hyper["lr"] = schedule(t - 1)  # the count before the increment (adamw.py:526)
        H.oracle_step(opt, g, leaf, state, gs, H.hyper_tuple(opt, conv, t, **hyper))
    H.assert_leaf_equal(leaf, want, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_python_surface_reproduces_variants(name):
    """The same constructor calls on this package give the reference's bits."""
    import torch

    import flashoptim_jax_b200 as fo

    meta, p0, grads, want = _load_variant(name)
    tx = getattr(fo, meta["constructor"])(donate=True, **{k: SCHEDULES.get(v, v) if isinstance(v, str) else v for k, v in meta["kwargs"].items()})
    params = {"x": H.to_torch(p0)}
    state = tx.init(params)
    for g in grads:
        params, state = tx.step(params, state, {"x": H.to_torch(g)})
    torch.cuda.synchronize()
    assert int(state.count) == len(grads)

    def moment(name):
        if not hasattr(state, name):
            return None, None
        m = getattr(state, name)["x"]
        if isinstance(m, fo.QuantizedArray):
            return H.to_numpy(m.values), H.to_numpy(m.scales)
        return (None if m.dim() == 0 else H.to_numpy(m)), None

    ecc = state.ecc["x"]
    mu, mu_s = moment("mu")
    nu, nu_s = moment("nu")
    got = H.LeafArrays(H.to_numpy(params["x"]), None if ecc.dim() == 0 else H.to_numpy(ecc), mu, mu_s, nu, nu_s)
    H.assert_leaf_equal(got, want, name)


TREES = json.load(open(os.path.join(GOLD, "trees.json")))


def _tree_kwargs(meta):
    kw = dict(meta["kwargs"])
    kw["param_groups"] = [{k: (tuple(v) if k == "params" and isinstance(v, list) else v) for k, v in g.items()}
                          for g in kw["param_groups"]]
    return kw


def _nest(pairs):
    tree = {}
    for path, value in pairs:
        node = tree
        for key in path[:-1]:
            node = node.setdefault(key, {})
        node[path[-1]] = value
    return tree


def _at(tree, path):
    for key in path:
        tree = tree[key]
    return tree


def _tree_leaf_want(z, tag, dt):
    view = lambda a: a.view(dt) if dt.itemsize == 2 else a  # noqa: E731
    get = lambda f: z[f"{tag}|{f}"] if f"{tag}|{f}" in z else None  # noqa: E731
    scales = lambda f: None if get(f) is None else get(f).view(np.float16)  # noqa: E731
    return H.LeafArrays(view(z[tag + "|param"]), get("ecc"), get("mu") if get("mu") is not None else get("mu_full"), scales("mu_scales"),
                        get("nu") if get("nu") is not None else get("nu_full"), scales("nu_scales"))


@pytest.mark.parametrize("name", sorted(TREES))
def test_param_groups_resolved_as_the_reference_resolves_them(name):
    """Nested pytrees with string, "a/b" and tuple selectors, first match wins, per-group learning rate, weight decay,
    betas, Nesterov, dampening and `fused`: this package's group resolution feeding the C oracle leaf by leaf gives the
    arrays the reference produced."""
    from flashoptim_jax_b200 import utils

    meta = TREES[name]
    kw = _tree_kwargs(meta)
    groups = kw.pop("param_groups")
    z = np.load(os.path.join(GOLD, f"tree_{name}.npz"))
    opt, decoupled = VARIANT_OPT[meta["constructor"]]
    for path, _shape, dtype in meta["leaves"]:
        path, dt, tag = tuple(path), NP_DT[dtype], "/".join(path)
        p0 = z[tag + "|param0"].view(dt) if dt.itemsize == 2 else z[tag + "|param0"]
        cfg = utils._group_config_for_path(path, p0, defaults=kw, param_groups=groups)
        conv = O.FUSED if cfg.get("fused", True) else O.UNFUSED
        ecc_bits = {None: 0, 24: 8, 32: 16}[cfg["master_weight_bits"]] if dt.itemsize == 2 else 0
        hyper = dict(lr=cfg["learning_rate"], wd=cfg.get("weight_decay", 0.0), decoupled=decoupled)
        for k in ("b1", "b2", "eps", "momentum", "dampening", "nesterov"):
            if k in cfg:
                hyper[k] = cfg[k]
        if opt == C.LION:
            hyper.setdefault("b2", 0.99)
            hyper.pop("decoupled")
        leaf = H.fresh_leaf(p0.reshape(-1), opt, C.STATE_QUANT, ecc_bits)
        for t in range(3):
            g = z[f"{tag}|grad{t}"]
            H.oracle_step(opt, (g.view(dt) if dt.itemsize == 2 else g).reshape(-1), leaf, C.STATE_QUANT, 32, H.hyper_tuple(opt, conv, t + 1, **hyper))
        want = _tree_leaf_want(z, tag, dt)
        want.param, want.ecc, want.mu, want.nu = (None if a is None else a.reshape(-1) for a in (want.param, want.ecc, want.mu, want.nu))
        H.assert_leaf_equal(leaf, want, f"{name} {tag}")


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(TREES))
def test_python_surface_reproduces_trees(name):
    import torch

    import flashoptim_jax_b200 as fo

    meta = TREES[name]
    z = np.load(os.path.join(GOLD, f"tree_{name}.npz"))
    leaves = [(tuple(path), NP_DT[dtype]) for path, _shape, dtype in meta["leaves"]]
    view = lambda a, dt: a.view(dt) if dt.itemsize == 2 else a  # noqa: E731
    tx = getattr(fo, meta["constructor"])(donate=True, **_tree_kwargs(meta))
    params = _nest([(path, H.to_torch(view(z["/".join(path) + "|param0"], dt))) for path, dt in leaves])
    state = tx.init(params)
    for t in range(3):
        grads = _nest([(path, H.to_torch(view(z["/".join(path) + f"|grad{t}"], dt))) for path, dt in leaves])
        params, state = tx.step(params, state, grads)
    torch.cuda.synchronize()
    assert int(state.count) == 3
    for path, dt in leaves:
        tag = "/".join(path)
        ecc = _at(state.ecc, path)
        mom = {}
        for field in ("mu", "nu"):
            m = _at(getattr(state, field), path) if hasattr(state, field) else None
            if isinstance(m, fo.QuantizedArray):
                mom[field] = (H.to_numpy(m.values), H.to_numpy(m.scales))
            else:
                mom[field] = (None if m is None or m.dim() == 0 else H.to_numpy(m), None)
        got = H.LeafArrays(H.to_numpy(_at(params, path)), None if ecc.dim() == 0 else H.to_numpy(ecc), *mom["mu"], *mom["nu"])
        H.assert_leaf_equal(got, _tree_leaf_want(z, tag, dt), f"{name} {tag}")
    # the checkpoint form: kinds, dtypes and shapes of the serialized leaves in the reference's order, and a round trip
    stem = {"flash_adam": "flash_adamw", "flash_sgdw": "flash_sgd"}.get(meta["constructor"], meta["constructor"])
    sd = getattr(fo, stem + "_state_dict")(state)
    describe = lambda t: [str(t.dtype).replace("torch.", ""), list(t.shape)]  # noqa: E731
    layout = {"count": describe(torch.as_tensor(sd["count"]))}
    for field in sorted(k for k in sd if k != "count"):
        layout[field] = [{"kind": leaf["kind"], **{k: describe(v) for k, v in leaf.items() if k != "kind"}} for leaf in sd[field]["leaves"]]
    assert layout == meta["state_dict"]
    back = getattr(fo, "load_" + stem + "_state_dict")(sd)
    from flashoptim_jax_b200 import tree as pytree

    for a, b in zip(pytree.tree_leaves(back), pytree.tree_leaves(state)):
        assert torch.equal(torch.as_tensor(a), torch.as_tensor(b))


@pytest.mark.gpu
@pytest.mark.parametrize("convention", ["fused", "unfused"])
def test_config1_digests(convention):
    """BASELINE config 1: 2048x2048 bf16 N(0,0.02), bf16 grads N(0,1e-3), lr 1e-3, betas (0.9,0.999), eps 1e-8,
    wd 1e-2, 24-bit master, 10 steps, seed 0: final codes, scales, ECC, params and reconstructed fp32 weights."""
    import torch

    import flashoptim_jax_b200 as fo

    want = json.load(open(os.path.join(GOLD, "config1_digests.json")))[convention]
    rng = np.random.default_rng(0)
    p = rng.normal(0, 0.02, (2048, 2048)).astype(np.float32).astype(H.BF16)
    tx = fo.flash_adamw(learning_rate=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2, master_weight_bits=24,
                        fused=(convention == "fused"), donate=True)
    params = {"w": H.to_torch(p)}
    state = tx.init(params)
    for _ in range(10):
        g = rng.normal(0, 1e-3, 2048 * 2048).astype(np.float32).astype(H.BF16).reshape(2048, 2048)
        params, state = tx.step(params, state, {"w": H.to_torch(g)})
    theta = fo.reconstruct_weights(params, state.ecc)
    torch.cuda.synchronize()
    got = {"param": params["w"], "ecc": state.ecc["w"], "mu": state.mu["w"].values, "mu_scales": state.mu["w"].scales,
           "nu": state.nu["w"].values, "nu_scales": state.nu["w"].scales, "reconstructed_fp32": theta["w"]}
    for k, t in got.items():
        assert hashlib.sha256(np.ascontiguousarray(H.to_numpy(t)).tobytes()).hexdigest() == want[k], k
