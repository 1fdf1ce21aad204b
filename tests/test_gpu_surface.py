"""The Python surface on the GPU: the reference's optimizer tests re-expressed (tests/test_adamw.py,
test_lion.py, test_sgd.py, test_optimizer_surface.py), with float64 textbook optimizers standing in for optax,
plus bit-exact checks of whole mixed pytrees against the oracle."""

import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _t(x, dtype=None):
    import torch

    t = torch.tensor(x, device="cuda")
    return t if dtype is None else t.to(dtype)


def _l2(*ts):
    return float(sum((t.double() ** 2).sum() for t in ts) ** 0.5)


def test_adamw_tracks_textbook_adamw_over_10_steps():
    # tests/test_adamw.py:24-54
    import torch

    import flashoptim_jax_b200 as fo

    p32 = {"w": _t([[0.5, -1.0], [1.5, -0.25]]), "b": _t([0.1, -0.2])}
    grads = {"w": _t([[0.3, -0.1], [0.2, -0.4]]), "b": _t([0.05, -0.02])}
    params = {k: v.to(torch.bfloat16) for k, v in p32.items()}
    tx = fo.flash_adamw(learning_rate=1e-2, weight_decay=1e-2)
    state = tx.init(params)
    ref = {k: v.double() for k, v in p32.items()}
    m = {k: torch.zeros_like(v) for k, v in ref.items()}
    v2 = {k: torch.zeros_like(v) for k, v in ref.items()}
    for t in range(1, 11):
        params, state = tx.step(params, state, grads)
        for k in ref:
            g = grads[k].double()
            m[k] = 0.9 * m[k] + 0.1 * g
            v2[k] = 0.999 * v2[k] + 0.001 * g * g
            ref[k] = ref[k] - 1e-2 * ((m[k] / (1 - 0.9**t)) / ((v2[k] / (1 - 0.999**t)).sqrt() + 1e-8) + 1e-2 * ref[k])
    master = fo.reconstruct_weights(params, state.ecc)
    assert _l2(*[master[k].double() - ref[k] for k in ref]) < 0.05
    assert params["w"].dtype == torch.bfloat16 and int(state.count) == 10


@pytest.mark.parametrize("kind", ["adam", "adamw", "lion", "sgd_nesterov", "sgdw"])
def test_closed_form_single_steps(kind):
    # tests/test_optimizer_surface.py:56-161: fp32 params, quantize=False, no ECC, atol 1e-7
    import torch

    import flashoptim_jax_b200 as fo

    p, g = np.array([1.0, -2.0, 3.0]), np.array([0.2, -0.1, 0.05])
    params, grads = {"x": _t(p.astype(np.float32))}, {"x": _t(g.astype(np.float32))}
    if kind in ("adam", "adamw"):
        f = fo.flash_adam if kind == "adam" else fo.flash_adamw
        tx = f(learning_rate=1e-3, weight_decay=1e-2, quantize=False, master_weight_bits=None, fused=False)
        lr = float(np.float32(1e-3))
        gg = g + 1e-2 * p if kind == "adam" else g
        pp = p if kind == "adam" else p * (1 - lr * 1e-2)
        exp = pp - (lr / 0.1) * (0.1 * gg) / (np.sqrt(0.001 * gg * gg) / np.sqrt(0.001) + 1e-8)
    elif kind == "lion":
        tx = fo.flash_lion(learning_rate=1e-4, weight_decay=1e-2, quantize=False, master_weight_bits=None)
        lr = float(np.float32(1e-4))
        exp = p * (1 - lr * 1e-2) - lr * np.sign(g)
    elif kind == "sgd_nesterov":
        tx = fo.flash_sgd(learning_rate=1e-3, momentum=0.9, weight_decay=1e-2, nesterov=True, quantize=False, master_weight_bits=None)
        lr = float(np.float32(1e-3))
        gg = g + 1e-2 * p
        exp = p - lr * (gg + 0.9 * gg)
    else:
        tx = fo.flash_sgdw(learning_rate=1e-3, momentum=0.9, weight_decay=1e-2, quantize=False, master_weight_bits=None)
        lr = float(np.float32(1e-3))
        exp = p * (1 - lr * 1e-2) - lr * g
    state = tx.init(params)
    actual, _ = tx.step(params, state, grads)
    np.testing.assert_allclose(actual["x"].cpu().numpy(), exp, atol=2e-7, rtol=2e-7)
    assert actual["x"].dtype == torch.float32


def test_param_groups_override_hyper_parameters():
    # tests/test_optimizer_surface.py:239-293
    import flashoptim_jax_b200 as fo

    params = {"trunk": {"w": _t([1.0, -2.0])}, "head": {"w": _t([0.5, -0.75])}}
    grads = {"trunk": {"w": _t([0.2, -0.1])}, "head": {"w": _t([0.4, -0.3])}}
    tx = fo.flash_adamw(learning_rate=1e-3, weight_decay=1e-2, quantize=False, master_weight_bits=None, fused=False,
                        param_groups=[{"params": ["head"], "learning_rate": 5e-3, "weight_decay": 0.0}])
    actual, _ = tx.step(params, tx.init(params), grads)

    def adamw(p, g, lr, wd):
        lr = float(np.float32(lr))
        return p * (1 - lr * wd) - (lr / 0.1) * (0.1 * g) / (np.sqrt(0.001 * g * g) / np.sqrt(0.001) + 1e-8)

    np.testing.assert_allclose(actual["trunk"]["w"].cpu().numpy(), adamw(np.array([1.0, -2.0]), np.array([0.2, -0.1]), 1e-3, 1e-2), atol=2e-7, rtol=2e-7)
    np.testing.assert_allclose(actual["head"]["w"].cpu().numpy(), adamw(np.array([0.5, -0.75]), np.array([0.4, -0.3]), 5e-3, 0.0), atol=2e-7, rtol=2e-7)


def test_schedule_uses_zero_based_counts():
    # tests/test_adamw.py:179-195
    import torch

    import flashoptim_jax_b200 as fo

    calls = []

    def schedule(count):
        calls.append(int(count))
        return torch.tensor(1e-3)

    params = {"x": _t([1.0, -2.0, 3.0], dtype=None).to(torch.bfloat16)}
    grads = {"x": _t([0.2, -0.1, 0.05])}
    tx = fo.flash_adamw(learning_rate=schedule, fused=False)
    state = tx.init(params)
    params, state = tx.step(params, state, grads)
    params, state = tx.step(params, state, grads)
    assert calls == [0, 1] and int(state.count) == 2


@pytest.mark.parametrize("factory_kw", [
    ("adamw", {}), ("adamw", {"master_weight_bits": None}), ("adamw", {"quantize": False}), ("adamw", {"master_weight_bits": 32}),
    ("adamw", {"master_weight_bits": 32, "quantize": False}), ("adam", {}), ("lion", {}), ("lion", {"quantize": False}),
    ("sgd", {"momentum": 0.9}), ("sgd", {"momentum": 0.9, "master_weight_bits": None}), ("sgd", {"momentum": 0.0}),
], ids=lambda fk: fk[0] + "-" + ",".join(f"{k}={v}" for k, v in fk[1].items()))
@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_fused_matches_unfused_on_tail_group_leaf(factory_kw, dtype):
    # tests/test_adamw.py:264-457, test_lion.py:85-245, test_sgd.py:103-285: 65-element leaf, atol/rtol 5e-3 (1e-6 for fp32 params)
    import torch

    import flashoptim_jax_b200 as fo

    name, kw = factory_kw
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    if dtype == "f32":
        kw = {**kw, "master_weight_bits": None}
    factory = {"adamw": fo.flash_adamw, "adam": fo.flash_adam, "lion": fo.flash_lion, "sgd": fo.flash_sgd}[name]
    lr = 1e-4 if name == "lion" else 1e-3
    params = {"x": torch.linspace(-2.0, 2.0, 65, device="cuda").to(tdt)}
    grads = {"x": torch.linspace(-0.3, 0.4, 65, device="cuda")}
    out = {}
    for fused in (False, True):
        tx = factory(learning_rate=lr, fused=fused, **kw)
        state = tx.init(params)
        p, state = tx.step(params, state, grads)
        out[fused] = (fo.reconstruct_weights(p, state.ecc)["x"], p["x"], state)
    tol = 1e-6 if dtype == "f32" else 5e-3
    assert torch.allclose(out[True][0], out[False][0], atol=tol, rtol=tol)
    assert out[True][1].dtype == tdt
    st = out[True][2]
    mwb = kw.get("master_weight_bits", 24)
    if dtype == "f32" or mwb is None:
        assert st.ecc["x"].dtype == torch.int32
    else:
        assert st.ecc["x"].dtype == (torch.int16 if mwb == 32 else torch.int8)
    if name == "sgd" and kw.get("momentum", 0.0) == 0.0:
        assert st.mu["x"].dim() == 0
    elif kw.get("quantize", True):
        assert isinstance(st.mu["x"], fo.QuantizedArray)
    else:
        assert st.mu["x"].dtype == torch.float32


def test_mixed_tree_matches_the_oracle_leaf_by_leaf():
    # GPT-2-like mix (config 4 in miniature): bf16 matrices, zero bf16 biases, fp32 layer norms, one call per bucket
    import torch

    import flashoptim_jax_b200 as fo

    rng = np.random.default_rng(0)
    shapes = {"wte": (500, 96), "wpe": (64, 96), "ln_f": (96,)}
    for i in range(3):
        shapes.update({f"h{i}.ln_1.g": (96,), f"h{i}.ln_1.b": (96,), f"h{i}.attn.w": (96, 288), f"h{i}.attn.b": (288,),
                       f"h{i}.mlp.w": (96, 384), f"h{i}.mlp.b": (384,)})
    pn = {}
    for k, s in shapes.items():
        if k.endswith(".w") or k in ("wte", "wpe"):
            pn[k] = rng.normal(0, 0.02, s).astype(np.float32).astype(H.BF16)
        elif k.endswith(".b"):
            pn[k] = np.zeros(s, dtype=np.float32).astype(H.BF16) if "ln" not in k else np.zeros(s, dtype=np.float32)
        else:
            pn[k] = np.ones(s, dtype=np.float32)
    for name, factory, opt, kw, hkw in (
        ("adamw", fo.flash_adamw, C.ADAM, dict(learning_rate=1e-3, weight_decay=1e-2), dict(lr=1e-3, wd=1e-2)),
        ("lion", fo.flash_lion, C.LION, dict(learning_rate=1e-4, weight_decay=1e-2), dict(lr=1e-4, wd=1e-2, b2=0.99)),
    ):
        tx = factory(donate=True, **kw)
        params = {k: H.to_torch(v) for k, v in pn.items()}
        state = tx.init(params)
        refs = {k: H.fresh_leaf(v.reshape(-1), opt, C.STATE_QUANT, 8 if v.dtype == H.BF16 else 0) for k, v in pn.items()}
        for t in range(1, 4):
            gn = {k: H.make_grad(rng, v.shape, 1e-3, v.dtype, outliers=1e-4) for k, v in pn.items()}
            params, state = tx.step(params, state, {k: H.to_torch(v) for k, v in gn.items()})
            for k in pn:
                H.oracle_step(opt, gn[k].reshape(-1), refs[k], C.STATE_QUANT, 32, H.hyper_tuple(opt, O.FUSED, t, **hkw))
        torch.cuda.synchronize()
        for k in pn:
            ecc = state.ecc[k]
            got = H.LeafArrays(H.to_numpy(params[k]).reshape(-1), None if ecc.dim() == 0 else H.to_numpy(ecc).reshape(-1),
                               H.to_numpy(state.mu[k].values).reshape(-1), H.to_numpy(state.mu[k].scales),
                               H.to_numpy(state.nu[k].values).reshape(-1) if opt == C.ADAM else None,
                               H.to_numpy(state.nu[k].scales) if opt == C.ADAM else None)
            H.assert_leaf_equal(got, refs[k], f"{name} {k}")


def test_step_argument_checks():
    import torch

    import flashoptim_jax_b200 as fo

    params = {"a": torch.zeros(64, dtype=torch.bfloat16, device="cuda"), "b": torch.zeros(3, device="cuda")}
    tx = fo.flash_adamw()
    state = tx.init(params)
    with pytest.raises(ValueError, match="state trees must match parameter structure"):
        tx.step(params, state, {"a": torch.zeros(64, device="cuda")})
    with pytest.raises(ValueError, match="does not match parameter shape"):
        tx.step(params, state, {"a": torch.zeros(63, device="cuda"), "b": torch.zeros(3, device="cuda")})
    # float64 grads are accepted (upcast rule of the reference: everything goes through fp32)
    p2, s2 = tx.step(params, state, {"a": torch.ones(64, dtype=torch.float64, device="cuda"), "b": torch.ones(3, device="cuda")})
    assert p2["a"].dtype == torch.bfloat16 and int(s2.count) == 1 and int(state.count) == 0


@pytest.mark.gpu
def test_donated_steps_replayed_from_the_prepared_launch_equal_plain_steps():
    """With donate=True the second and later steps on the same tensors replay a prepared launch (only gradient
    addresses and scalars are refreshed); new tensor objects, a new gradient dtype or a non-contiguous gradient
    fall back to the general path.  Whatever the route, the results are those of the non-donating steps."""
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree

    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(3)

    def make():
        g = torch.Generator(device=dev).manual_seed(5)
        return {"w": (torch.randn((300, 70), device=dev, generator=g) * 0.02).to(torch.bfloat16),
                "b": torch.zeros(70, device=dev), "v": [(torch.randn(5000, device=dev, generator=g) * 0.02).to(torch.bfloat16)]}

    groups = [{"params": "b", "weight_decay": 0.0}]
    fast = fo.flash_adamw(learning_rate=lambda c: 1e-3 / (1.0 + float(c)), master_weight_bits=32, param_groups=groups, donate=True)
    plain = fo.flash_adamw(learning_rate=lambda c: 1e-3 / (1.0 + float(c)), master_weight_bits=32, param_groups=groups, donate=False)
    pf, pp = make(), make()
    sf, sp = fast.init(pf), plain.init(pp)
    for t in range(8):
        grads = tree.tree_map(lambda p: (torch.randn(p.shape, device=dev, generator=gen) * 1e-3).to(p.dtype), pp)
        if t == 4:  # another gradient dtype for the 16-bit leaves: the prepared launch does not fit
            grads = tree.tree_map(lambda g: g.float(), grads)
        if t == 5:  # new tensor objects for the same values
            pf = tree.tree_map(lambda x: x.clone(), pf)
        if t == 6:  # a non-contiguous gradient
            wide = torch.zeros((300, 140), device=dev, dtype=torch.bfloat16)
            wide[:, ::2] = grads["w"]
            grads = dict(grads, w=wide[:, ::2])
        pf, sf = fast.step(pf, sf, grads)
        pp, sp = plain.step(pp, sp, grads)
    torch.cuda.synchronize()
    assert int(sf.count) == int(sp.count) == 8
    for a, b in zip(tree.tree_leaves(pf), tree.tree_leaves(pp)):
        assert torch.equal(a, b)
    for name in ("mu", "nu", "ecc"):
        for a, b in zip(tree.tree_leaves(getattr(sf, name)), tree.tree_leaves(getattr(sp, name))):
            assert a.dtype == b.dtype and torch.equal(a, b)
