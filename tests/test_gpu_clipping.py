"""Global-norm clipping folded into the step: the sum of squares (fo_sq_norm) against float64, and
the rescaled step against the oracle (element-wise exact once both sides use the device's sum)."""


import ml_dtypes
import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _sq_norm(tensors, accumulate_into=None):
    from flashoptim_jax_b200 import _engine as eng

    return eng.sq_norm_of(tensors, out=accumulate_into, accumulate=accumulate_into is not None)


def test_sum_of_squares_many_arrays_dtypes_alignments():
    import torch

    rng = np.random.default_rng(0)
    sizes = [1, 7, 2048, 2049, 4096 * 3 + 5, 100003, 33] * 30  # 210 arrays: more than one launch holds
    for np_dt in (np.float32, ml_dtypes.bfloat16, np.float16):
        arrays = [rng.normal(0, 0.3, n).astype(np.float32).astype(np_dt) for n in sizes]
        want = O.global_sq_norm(arrays)
        dev = [H.to_torch(a) for a in arrays]
        dev[3] = torch.cat([dev[3][:1], dev[3]])[1:]  # an array that does not start on a 16-byte boundary
        got = float(_sq_norm(dev).cpu())
        assert abs(got - want) <= 2e-6 * want, (np_dt, got, want)
        again = float(_sq_norm(dev).cpu())
        assert again == got  # same inputs, same bits
        both = float(_sq_norm(dev[:50], accumulate_into=_sq_norm(dev[50:])).cpu())
        assert abs(both - want) <= 2e-6 * want
    empty = float(_sq_norm([torch.zeros(0, device="cuda")], accumulate_into=torch.full((1,), 5.0, dtype=torch.float64, device="cuda")).cpu())
    assert empty == 5.0


@pytest.mark.parametrize("opt,gdt,scale,max_norm", [
    (C.ADAM, 1, 3e-2, 1.0), (C.ADAM, 1, 1e-5, 1.0), (C.ADAM, 0, 1e-2, 0.37), (C.LION, 2, 3e-2, 1.0), (C.SGD, 1, 3.0, 0.05),
])
def test_clipped_step_equals_oracle(opt, gdt, scale, max_norm):
    import torch

    from flashoptim_jax_b200 import _engine as eng

    rng = np.random.default_rng(opt * 7 + gdt)
    g_np = {0: np.float32, 1: ml_dtypes.bfloat16, 2: np.float16}[gdt]
    sizes = [2048 * 3, 2048 + 77, 31, 5000]
    refs = [H.fresh_leaf(rng.normal(0, 0.05, n).astype(np.float32).astype(ml_dtypes.bfloat16), opt, C.STATE_QUANT, 16) for n in sizes]
    devs = [r.copy().to_device() for r in refs]
    clipped_steps = 0
    for t in range(1, 4):
        grads = [H.make_grad(rng, n, scale, g_np) for n in sizes]
        if t == 2:
            grads[0][::5] = g_np(0)  # exact zeros, both signs
            grads[0][1::10] = -g_np(0)
        dev_g = [H.to_torch(g) for g in grads]
        sq = _sq_norm(dev_g)
        sq_host = float(sq.cpu())
        assert abs(sq_host - O.global_sq_norm(grads)) <= 2e-6 * sq_host
        clipped_steps += np.float32(np.sqrt(sq_host)) >= np.float32(max_norm)
        hp = H.hyper_tuple(opt, O.FUSED, t, lr=1e-2, wd=1e-2)
        for g, r in zip(O.clip_by_global_norm(grads, max_norm, sq_norm=sq_host), refs):
            H.oracle_step(opt, g, r, C.STATE_QUANT, 32, hp)
        with eng.grad_clip(sq, max_norm):
            pass  # the context is what the Python surface uses; the raw call below passes the same two values
        H.abi_step(opt, dev_g, devs, C.STATE_QUANT, 32, [hp], [0] * len(sizes), 1, gdt, 16, grad_sq_norm=sq, max_grad_norm=max_norm)
    torch.cuda.synchronize()
    assert clipped_steps == (0 if scale == 1e-5 else 3)
    for i, (d, r) in enumerate(zip(devs, refs)):
        H.assert_leaf_equal(d.to_host(), r, f"leaf {i}")


def test_wrapper_matches_reference_recipe_structure():
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.clipping import clip_by_global_norm, global_sq_norm

    g = torch.Generator(device="cpu").manual_seed(0)
    params = {"w": (torch.randn(300, 70, generator=g) * 0.02).bfloat16().cuda(), "b": torch.zeros(70).cuda()}
    grads = {"w": (torch.randn(300, 70, generator=g) * 0.1).bfloat16().cuda(), "b": (torch.randn(70, generator=g) * 0.1).cuda()}
    tx = clip_by_global_norm(fo.flash_adamw(learning_rate=1e-3, master_weight_bits=32), 1.0)
    state = tx.init(params)
    assert set(state) == {"clip", "opt"} and state["clip"] == ()
    new_params, new_state = tx.step(params, state, grads)
    # the same step on gradients clipped by the oracle, using the device's sum of squares
    sq = float(global_sq_norm(grads).cpu())
    leaves = [H.to_numpy(t) for t in tree.tree_leaves(grads)]
    clipped = tree.tree_unflatten(tree.tree_structure(grads), [H.to_torch(a) for a in O.clip_by_global_norm(leaves, 1.0, sq_norm=sq)])
    plain = fo.flash_adamw(learning_rate=1e-3, master_weight_bits=32)
    want_params, want_state = plain.step(params, plain.init(params), clipped)
    for a, b in zip(tree.tree_leaves(new_params), tree.tree_leaves(want_params)):
        assert torch.equal(a, b)
    for a, b in zip(tree.tree_leaves(new_state["opt"]), tree.tree_leaves(want_state)):
        assert torch.equal(torch.as_tensor(a), torch.as_tensor(b))
    assert int(new_state["opt"].count) == 1
