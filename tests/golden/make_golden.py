"""Generates the golden fixtures in this directory from the reference's own source files.

    python tests/golden/make_golden.py [--reference /path/to/flashoptim-jax] [--check]

The reference (`flashoptim_jax`) is a JAX program and JAX is not installable here, so this script
puts `tests/jax_standin` (a NumPy + ml_dtypes stand-in for the `jax` names the reference uses,
with a NumPy interpreter for its Pallas kernels) on `sys.path`, imports the reference's package
UNMODIFIED from its checkout, and drives it through its public API: `flash_adamw / flash_lion /
flash_sgdw(...).init / .step`, `fused=True` (the Pallas kernel text) and `fused=False` (the jnp
text).  The fixtures are therefore outputs of the reference's text, not of the restatement in
`oracle/`.

Primitive semantics that are NumPy's rather than XLA's in these vectors (see
`tests/jax_standin/jax/numpy/__init__.py`): `ldexp` is an exact power-of-two scaling, `**` in the
bias corrections is NumPy's fp32 `powf` (this script asserts that it equals the float64 power
rounded once, for every count it uses), float->int casts act on values already clipped to
range, 16-bit float arithmetic rounds once per operation.  `fused=True` means the kernel text
under strict IEEE fp32, not Triton's generated code.

`--check` regenerates everything in memory and compares with the committed files instead of
writing them.
"""

import argparse
import hashlib
import io
import json
import os
import sys

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
STANDIN = os.path.join(os.path.dirname(HERE), "jax_standin")
BF16 = np.dtype(ml_dtypes.bfloat16)

HYPER = {
    "adamw": dict(learning_rate=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2),
    "lion": dict(learning_rate=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2),
    "sgdw": dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2),
}

SMALL_CASES = [
    (2048 + 65, BF16, 24, "adamw", "fused"), (2048 + 65, BF16, 32, "adamw", "unfused"),
    (1000, np.dtype(np.float16), 32, "adamw", "fused"), (777, BF16, 24, "lion", "fused"),
    (777, BF16, 24, "lion", "unfused"), (2111, BF16, 32, "sgdw", "fused"),
    (300, np.dtype(np.float32), None, "adamw", "fused"),
    (1500, BF16, 24, "sgdw", "unfused"), (1023, np.dtype(np.float16), 24, "lion", "unfused"),
    (4129, BF16, 24, "adamw", "unfused"), (1031, np.dtype(np.float32), None, "sgdw", "unfused"),
    (2048, BF16, None, "adamw", "fused"),
]


# Further cases through the other constructors and options of the public surface: (name, constructor,
# keyword arguments, elements, parameter dtype, gradient dtype).
VARIANT_CASES = [
    ("adam_coupled_fused", "flash_adam", dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=24, fused=True), 1300, "bfloat16", "bfloat16"),
    ("adam_coupled_unfused", "flash_adam", dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=32, fused=False), 1300, "bfloat16", "bfloat16"),
    ("sgd_coupled_nesterov_fused", "flash_sgd", dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2, nesterov=True, master_weight_bits=24, fused=True), 1111, "bfloat16", "bfloat16"),
    ("sgd_coupled_nesterov_unfused", "flash_sgd", dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2, nesterov=True, master_weight_bits=24, fused=False), 1111, "bfloat16", "bfloat16"),
    ("sgdw_dampening_fused", "flash_sgdw", dict(learning_rate=1e-2, momentum=0.9, dampening=0.1, weight_decay=1e-2, master_weight_bits=32, fused=True), 999, "bfloat16", "bfloat16"),
    ("sgdw_dampening_unfused", "flash_sgdw", dict(learning_rate=1e-2, momentum=0.9, dampening=0.1, weight_decay=1e-2, master_weight_bits=24, fused=False), 999, "float16", "bfloat16"),
    ("sgdw_no_momentum", "flash_sgdw", dict(learning_rate=1e-2, momentum=0.0, weight_decay=1e-2, master_weight_bits=24), 700, "bfloat16", "bfloat16"),
    ("adamw_full_state", "flash_adamw", dict(learning_rate=1e-3, weight_decay=1e-2, quantize=False, master_weight_bits=24), 600, "bfloat16", "bfloat16"),
    ("lion_full_state", "flash_lion", dict(learning_rate=1e-4, weight_decay=1e-2, quantize=False, master_weight_bits=32), 600, "bfloat16", "bfloat16"),
    ("sgdw_full_state", "flash_sgdw", dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2, quantize=False, master_weight_bits=None), 600, "float32", "float32"),
    ("adamw_group64_unfused", "flash_adamw", dict(learning_rate=1e-3, weight_decay=1e-2, group_size=64, master_weight_bits=24, fused=False), 1000, "bfloat16", "bfloat16"),
    ("lion_group8_unfused", "flash_lion", dict(learning_rate=1e-4, weight_decay=1e-2, group_size=8, master_weight_bits=24, fused=False), 333, "bfloat16", "bfloat16"),
    ("adamw_fp32_grads_fused", "flash_adamw", dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=24, fused=True), 2100, "bfloat16", "float32"),
    ("adamw_fp16_grads_unfused", "flash_adamw", dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=32, fused=False), 2100, "float16", "float16"),
    ("lion_betas_fused", "flash_lion", dict(learning_rate=3e-4, b1=0.95, b2=0.98, weight_decay=0.1, master_weight_bits=24, fused=True), 1500, "bfloat16", "bfloat16"),
    ("adamw_betas_eps_fused", "flash_adamw", dict(learning_rate=3e-4, b1=0.8, b2=0.95, eps=1e-6, weight_decay=0.1, master_weight_bits=32, fused=True), 1500, "bfloat16", "bfloat16"),
    # a schedule instead of a number ("@name": see SCHEDULES): it sees the count before the increment
    ("adamw_schedule_fused", "flash_adamw", dict(learning_rate="@halving", weight_decay=1e-2, master_weight_bits=24, fused=True), 900, "bfloat16", "bfloat16"),
    ("sgdw_schedule_unfused", "flash_sgdw", dict(learning_rate="@halving", momentum=0.9, weight_decay=1e-2, master_weight_bits=24, fused=False), 900, "bfloat16", "bfloat16"),
]
SCHEDULES = {"@halving": lambda count: 1e-3 * 0.5 ** int(count)}
NP_DTYPES = {"bfloat16": BF16, "float16": np.dtype(np.float16), "float32": np.dtype(np.float32)}

# Nested pytrees with mixed dtypes and param groups (string, "a/b" path and tuple selectors; first match wins):
# (name, constructor, keyword arguments, [(path, shape, dtype), ...]); gradients have each leaf's dtype.
BLOCK_LEAVES = [(("attn", "kernel"), (96, 64), "bfloat16"), (("attn", "bias"), (64,), "bfloat16"),
                (("ln", "scale"), (64,), "float32"), (("ln", "bias"), (64,), "float32"),
                (("head", "kernel"), (64, 33), "bfloat16"), (("head", "bias"), (33,), "float32")]
TREE_CASES = [
    ("block_adamw_groups", "flash_adamw",
     dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=24, fused=True,
          param_groups=[{"params": ("head", "bias"), "learning_rate": 2e-3, "weight_decay": 0.0},
                        {"params": "bias", "weight_decay": 0.0},
                        {"params": "ln/scale", "weight_decay": 0.0, "learning_rate": 5e-4, "b2": 0.99},
                        {"params": "head", "fused": False}]), BLOCK_LEAVES),
    ("block_sgd_groups", "flash_sgd",
     dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-3, master_weight_bits=32, fused=True,
          param_groups=[{"params": "bias", "weight_decay": 0.0, "nesterov": True},
                        {"params": "attn/kernel", "learning_rate": 5e-3, "dampening": 0.1}]), BLOCK_LEAVES),
    ("block_lion_groups", "flash_lion",
     dict(learning_rate=1e-4, weight_decay=1e-2, master_weight_bits=24, fused=False,
          param_groups=[{"params": "ln", "weight_decay": 0.0, "b1": 0.95},
                        {"params": ("attn", "kernel"), "fused": True}]), BLOCK_LEAVES),
]


def tuples_in(groups):
    """JSON has no tuples: selectors stored as lists come back as tuples."""
    return [{k: (tuple(v) if k == "params" and isinstance(v, list) else v) for k, v in g.items()} for g in groups]


def import_reference(path):
    """The reference package, unmodified, on top of the stand-in."""
    if not os.path.isdir(os.path.join(path, "flashoptim_jax")):
        raise SystemExit(f"no flashoptim_jax package under {path}")
    for p in (path, STANDIN):
        if p not in sys.path:
            sys.path.insert(0, p)
    import jax  # noqa: F401  (the stand-in)

    assert os.path.dirname(os.path.dirname(jax.__file__)) == STANDIN, "a real jax is installed: use it instead"
    import flashoptim_jax

    assert os.path.dirname(os.path.dirname(os.path.abspath(flashoptim_jax.__file__))) == os.path.abspath(path)
    return flashoptim_jax


def check_pow(betas, counts):
    """NumPy's fp32 powf against the float64 power rounded once (what oracle and product use)."""
    for b in betas:
        for c in counts:
            got = b ** np.float32(c)
            want = np.float32(float(np.float32(b)) ** float(c))
            assert got.dtype == np.float32 and got == want, (b, c, got, want)


def make_tx(ref, opt, mwb, convention):
    kw = dict(HYPER[opt], master_weight_bits=mwb, fused=(convention == "fused"))
    return {"adamw": ref.flash_adamw, "lion": ref.flash_lion, "sgdw": ref.flash_sgdw}[opt](**kw)


def bits(a):
    a = np.asarray(a)
    return a.view(np.uint16) if a.dtype.itemsize == 2 and a.dtype.kind not in "iu" else a


def small_case(ref, seed, n, dtype, mwb, opt, convention, steps=3):
    rng = np.random.default_rng(seed)
    p = rng.normal(0, 0.02, n).astype(np.float32).astype(dtype)
    grads = [rng.normal(0, 1e-3, n).astype(np.float32).astype(BF16) for _ in range(steps)]
    out = {"param0": bits(p), "grads": np.stack([bits(g) for g in grads])}
    tx = make_tx(ref, opt, mwb, convention)
    params = {"x": p}
    state = tx.init(params)
    for g in grads:
        params, state = tx.step(params, state, {"x": g})
    assert int(state.count) == steps
    out.update(param=bits(params["x"]), mu=np.asarray(state.mu["x"].values), mu_scales=bits(state.mu["x"].scales))
    if opt == "adamw":
        out.update(nu=np.asarray(state.nu["x"].values), nu_scales=bits(state.nu["x"].scales))
    ecc = np.asarray(state.ecc["x"])
    if ecc.shape != ():
        out["ecc"] = ecc
    for k, v in out.items():
        assert v.dtype != np.float64, k
    return out


def variant_case(ref, seed, factory, kwargs, n, dtype, grad_dtype, steps=3):
    """Like small_case for any constructor / keyword arguments; a moment kept in full precision
    (quantize=False) is stored as `mu_full` / `nu_full`, an absent one (momentum 0) not at all."""
    rng = np.random.default_rng(seed)
    p = rng.normal(0, 0.02, n).astype(np.float32).astype(NP_DTYPES[dtype])
    grads = [rng.normal(0, 1e-3, n).astype(np.float32).astype(NP_DTYPES[grad_dtype]) for _ in range(steps)]
    out = {"param0": bits(p), "grads": np.stack([bits(g) for g in grads])}
    tx = getattr(ref, factory)(**{k: SCHEDULES.get(v, v) if isinstance(v, str) else v for k, v in kwargs.items()})
    params = {"x": p}
    state = tx.init(params)
    for g in grads:
        params, state = tx.step(params, state, {"x": g})
    assert int(state.count) == steps
    out["param"] = bits(params["x"])
    for name in ("mu", "nu"):
        if not hasattr(state, name):
            continue
        m = getattr(state, name)["x"]
        if hasattr(m, "values"):
            out[name] = np.asarray(m.values)
            out[name + "_scales"] = bits(m.scales)
        elif np.asarray(m).shape != ():
            out[name + "_full"] = np.asarray(m)
    ecc = np.asarray(state.ecc["x"])
    if ecc.shape != ():
        out["ecc"] = ecc
    for k, v in out.items():
        assert v.dtype != np.float64, k
    return out


def nest(pairs):
    tree = {}
    for path, value in pairs:
        node = tree
        for key in path[:-1]:
            node = node.setdefault(key, {})
        node[path[-1]] = value
    return tree


def tree_case(ref, seed, factory, kwargs, leaves, steps=3):
    """A nested pytree through the reference; arrays are stored under "<a/b>|<field>"."""
    rng = np.random.default_rng(seed)
    p0 = [(path, rng.normal(0, 0.02, shape).astype(np.float32).astype(NP_DTYPES[dt])) for path, shape, dt in leaves]
    out = {}
    for path, p in p0:
        out["/".join(path) + "|param0"] = bits(p)
    tx = getattr(ref, factory)(**dict(kwargs, param_groups=tuples_in(kwargs["param_groups"])))
    params = nest(p0)
    state = tx.init(params)
    for t in range(steps):
        g = [(path, rng.normal(0, 1e-3, shape).astype(np.float32).astype(NP_DTYPES[dt])) for path, shape, dt in leaves]
        for path, a in g:
            out["/".join(path) + f"|grad{t}"] = bits(a)
        params, state = tx.step(params, state, nest(g))
    assert int(state.count) == steps

    def at(tree, path):
        for key in path:
            tree = tree[key]
        return tree

    for path, _, _ in leaves:
        tag = "/".join(path)
        out[tag + "|param"] = bits(at(params, path))
        for name in ("mu", "nu"):
            if not hasattr(state, name):
                continue
            m = at(getattr(state, name), path)
            if hasattr(m, "values"):
                out[f"{tag}|{name}"] = np.asarray(m.values)
                out[f"{tag}|{name}_scales"] = bits(m.scales)
            elif np.asarray(m).shape != ():
                out[f"{tag}|{name}_full"] = np.asarray(m)
        ecc = np.asarray(at(state.ecc, path))
        if ecc.shape != ():
            out[tag + "|ecc"] = ecc
    for k, v in out.items():
        assert v.dtype != np.float64, k
    # the checkpoint form of this state (flash_*_state_dict): kinds, dtypes and shapes of the serialized leaves in order
    to_sd = getattr(ref, {"flash_adam": "flash_adamw", "flash_sgdw": "flash_sgd"}.get(factory, factory) + "_state_dict")
    sd = to_sd(state)
    layout = {"count": [str(np.asarray(sd["count"]).dtype), list(np.asarray(sd["count"]).shape)]}
    for field in sorted(k for k in sd if k != "count"):
        layout[field] = [{"kind": leaf["kind"],
                          **{k: [str(np.asarray(v).dtype), list(np.asarray(v).shape)] for k, v in leaf.items() if k != "kind"}}
                         for leaf in sd[field]["leaves"]]
    return out, layout


def config1_digests(ref):
    """Benchmark config 1: one 2048x2048 bf16 matrix N(0, 0.02), grads bf16 N(0, 1e-3), 10 AdamW steps,
    lr 1e-3, betas (0.9, 0.999), eps 1e-8, wd 1e-2, 24-bit master, seed 0; both texts of the reference."""
    digests = {}
    for convention in ("fused", "unfused"):
        rng = np.random.default_rng(0)
        p = rng.normal(0, 0.02, (2048, 2048)).astype(np.float32).astype(BF16)
        tx = make_tx(ref, "adamw", 24, convention)
        params = {"w": p}
        state = tx.init(params)
        for _ in range(10):
            g = rng.normal(0, 1e-3, 2048 * 2048).astype(np.float32).astype(BF16).reshape(2048, 2048)
            params, state = tx.step(params, state, {"w": g})
        theta = ref.reconstruct_weights(params, state.ecc)["w"]
        assert theta.dtype == np.float32
        arrays = {"param": params["w"], "ecc": state.ecc["w"], "mu": state.mu["w"].values,
                  "mu_scales": state.mu["w"].scales, "nu": state.nu["w"].values, "nu_scales": state.nu["w"].scales,
                  "reconstructed_fp32": theta}
        digests[convention] = {k: hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest() for k, v in arrays.items()}
    return digests


def codec_vectors(ref):
    """Direct calls of the reference's codecs (quantization.py, compression.py) on seeded inputs with
    exact zeros, an all-zero group, a ragged tail, tiny and huge magnitudes."""
    rng = np.random.default_rng(77)
    n = 32 * 40 + 11
    x = (rng.normal(0, 1, n) * np.exp(rng.uniform(-12, 4, n))).astype(np.float32)
    x[64:96] = 0
    x[5] = 0
    v = np.square(x)
    qm = ref.quantize_momentum(x, 32)
    qv = ref.quantize_variance(v, 32)
    theta = (rng.normal(0, 0.02, n) * np.exp(rng.uniform(-3, 3, n))).astype(np.float32)
    theta[7] = 0
    theta[8] = np.float32(2.0 ** -120)  # below the range where JAX's ldexp stays finite; NumPy's is exact
    out = {"x": x, "v": v, "qm_values": qm.values, "qm_scales": bits(qm.scales), "qv_values": qv.values,
           "qv_scales": bits(qv.scales), "dqm": ref.dequantize_momentum(qm, 32), "dqv": ref.dequantize_variance(qv, 32),
           "theta": theta}
    for tag, dt, mwb in (("bf16_8", BF16, 24), ("bf16_16", BF16, 32), ("f16_8", np.float16, 24), ("f16_16", np.float16, 32)):
        lp, ecc = ref.split_leaf(theta, narrow_dtype=dt, master_weight_bits=mwb)
        out[f"lp_{tag}"] = bits(lp)
        out[f"ecc_{tag}"] = np.asarray(ecc)
        out[f"recon_{tag}"] = ref.reconstruct_leaf(lp, ecc)
    return {k: np.asarray(a) for k, a in out.items()}


def npz_bytes(arrays):
    buf = io.BytesIO()
    np.savez_compressed(buf, **arrays)
    return buf.getvalue()


def same_npz(path, arrays):
    if not os.path.exists(path):
        return False
    z = np.load(path)
    return sorted(z.files) == sorted(arrays) and all(
        z[k].dtype == arrays[k].dtype and z[k].shape == arrays[k].shape and np.array_equal(z[k], arrays[k]) for k in arrays)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FLASHOPTIM_REFERENCE", "/root/reference"))
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    ref = import_reference(args.reference)
    check_pow((0.9, 0.999, 0.8, 0.95, 0.99), range(1, 11))

    bad = []
    cases = {}
    files = {}
    for i, (n, dtype, mwb, opt, convention) in enumerate(SMALL_CASES):
        name = f"case{i}_{opt}_{np.dtype(dtype).name}_mwb{mwb}_{convention}"
        files[name + ".npz"] = small_case(ref, 1000 + i, n, dtype, mwb, opt, convention)
        cases[name] = {"n": n, "dtype": np.dtype(dtype).name, "master_weight_bits": mwb, "optimizer": opt,
                       "convention": convention}
    variants = {}
    for i, (name, factory, kwargs, n, dtype, grad_dtype) in enumerate(VARIANT_CASES):
        files[f"variant_{name}.npz"] = variant_case(ref, 2000 + i, factory, kwargs, n, dtype, grad_dtype)
        variants[name] = {"constructor": factory, "kwargs": kwargs, "n": n, "dtype": dtype, "grad_dtype": grad_dtype}
    trees = {}
    for i, (name, factory, kwargs, leaves) in enumerate(TREE_CASES):
        files[f"tree_{name}.npz"], layout = tree_case(ref, 3000 + i, factory, kwargs, leaves)
        trees[name] = {"constructor": factory, "kwargs": json.loads(json.dumps(kwargs)),
                       "leaves": [[list(path), list(shape), dt] for path, shape, dt in leaves], "state_dict": layout}
    files["codecs.npz"] = codec_vectors(ref)
    for fname, arrays in files.items():
        path = os.path.join(HERE, fname)
        if args.check:
            if not same_npz(path, arrays):
                bad.append(fname)
        else:
            with open(path, "wb") as f:
                f.write(npz_bytes(arrays))
    for fname, obj in (("cases.json", cases), ("variants.json", variants), ("trees.json", trees),
                       ("config1_digests.json", config1_digests(ref))):
        path = os.path.join(HERE, fname)
        if args.check:
            if not os.path.exists(path) or json.load(open(path)) != obj:
                bad.append(fname)
        else:
            with open(path, "w") as f:
                json.dump(obj, f, indent=1)
    if bad:
        raise SystemExit("fixtures differ from the reference's output: " + ", ".join(bad))
    print("checked" if args.check else "written", len(files) + 4, "fixtures")


if __name__ == "__main__":
    main()
