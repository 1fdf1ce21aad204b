"""Reduce-scatter and all-gather folded into the step, exercised on ONE GPU: the "ranks" are
separate buffers in the same memory, stepped one after the other, and the peer offsets are the
distances between those buffers.  Expected: every rank's slice is updated with the mean gradient
(fp32 sum in the order own, peers ascending; divided by the rank count; rounded once to the
gradient dtype), and every replica of the parameters ends up holding every slice."""

import ml_dtypes
import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _mean_grad(gs, k, np_dtype):
    order = [k] + [j for j in range(len(gs)) if j != k]
    acc = gs[order[0]].astype(np.float32)
    for j in order[1:]:
        acc = (acc + gs[j].astype(np.float32)).astype(np.float32)
    mean = (acc / np.float32(len(gs))).astype(np.float32)
    return mean.astype(np_dtype)


@pytest.mark.parametrize("world,opt,ecc_bits,gdt", [(2, C.ADAM, 16, 1), (3, C.ADAM, 8, 1), (4, C.LION, 8, 1),
                                                    (8, C.ADAM, 16, 1), (3, C.SGD, 16, 0), (8, C.ADAM, 8, 0), (2, C.ADAM, 16, 2)])
def test_virtual_ranks_match_oracle_on_mean_gradient(world, opt, ecc_bits, gdt):
    import torch

    rng = np.random.default_rng(world * 100 + opt * 10 + gdt)
    g_np = {0: np.float32, 1: ml_dtypes.bfloat16, 2: np.float16}[gdt]
    per = 5 * 2048 + 7 * 32  # whole groups per rank; the last rank's slice ends ragged
    n = per * world - 13
    lo = [k * per for k in range(world)]
    hi = [min(n, (k + 1) * per) for k in range(world)]
    p0 = rng.normal(0, 0.05, n).astype(np.float32).astype(ml_dtypes.bfloat16)
    grads_steps = []
    for t in range(3):
        gs = [H.make_grad(rng, n, 1e-3, g_np) for _ in range(world)]
        if t == 1:  # exact cancellations and tiny sums: the out-of-range handling of the mean
            gs[1][::7] = -gs[0][::7]
            for g in gs:
                g[3::11] = g_np(0) if gdt else np.float32(1e-38)
        grads_steps.append(gs)

    # oracle: one leaf per rank slice
    refs = [H.fresh_leaf(p0[lo[k]:hi[k]].copy(), opt, C.STATE_QUANT, ecc_bits) for k in range(world)]
    # device: a replica of the parameters and a full gradient buffer per rank, state for the own slice only
    P = [H.to_torch(p0.copy()) for _ in range(world)]
    G = [torch.zeros(n, dtype={0: torch.float32, 1: torch.bfloat16, 2: torch.float16}[gdt], device="cuda") for _ in range(world)]
    devs = []
    for k in range(world):
        st = H.fresh_leaf(p0[lo[k]:hi[k]].copy(), opt, C.STATE_QUANT, ecc_bits).to_device()
        st.param = P[k][lo[k]:hi[k]]
        devs.append(st)
    for t in range(3):
        hp = H.hyper_tuple(opt, O.FUSED, t + 1, lr=1e-2, wd=1e-2)
        for k in range(world):
            G[k].copy_(H.to_torch(grads_steps[t][k]))
            H.oracle_step(opt, _mean_grad([g[lo[k]:hi[k]] for g in grads_steps[t]], k, g_np), refs[k], C.STATE_QUANT, 32, hp)
        for k in range(world):
            others = [j for j in range(world) if j != k]
            H.abi_step(opt, [G[k][lo[k]:hi[k]]], [devs[k]], C.STATE_QUANT, 32, [hp], [0], 1, gdt, ecc_bits,
                       peer_param_offsets=[P[j].data_ptr() - P[k].data_ptr() for j in others],
                       peer_grad_offsets=[G[j].data_ptr() - G[k].data_ptr() for j in others])
        torch.cuda.synchronize()
    for k in range(world):
        H.assert_leaf_equal(devs[k].to_host(), refs[k], f"rank {k} slice")
    want = np.concatenate([H.bits(r.param) for r in refs])
    for j in range(world):
        got = H.bits(H.to_numpy(P[j]))
        assert np.array_equal(got, want), f"replica {j} differs at {np.flatnonzero(got != want)[:5]}"


def test_grad_peers_alone_and_argument_errors():
    import torch

    rng = np.random.default_rng(5)
    n = 4096 + 64
    p0 = rng.normal(0, 0.05, n).astype(np.float32).astype(ml_dtypes.bfloat16)
    g0, g1 = (H.make_grad(rng, n, 1e-3, ml_dtypes.bfloat16) for _ in range(2))
    ref = H.fresh_leaf(p0.copy(), C.SGD, C.STATE_QUANT, 16)
    dev = ref.copy().to_device()
    hp = H.hyper_tuple(C.SGD, O.FUSED, 1, lr=0.1, wd=0.0, momentum=0.9)
    H.oracle_step(C.SGD, _mean_grad([g0, g1], 0, ml_dtypes.bfloat16), ref, C.STATE_QUANT, 32, hp)
    G0, G1 = H.to_torch(g0), H.to_torch(g1)
    H.abi_step(C.SGD, [G0], [dev], C.STATE_QUANT, 32, [hp], [0], 1, 1, 16, peer_grad_offsets=[G1.data_ptr() - G0.data_ptr()])
    torch.cuda.synchronize()
    H.assert_leaf_equal(dev.to_host(), ref, "gradient peers without parameter replicas")
    # any group size other than 32 cannot take peers
    rc = H.abi_step(C.SGD, [G0], [dev], C.STATE_QUANT, 64, [hp], [0], 1, 1, 16, expect_ok=False,
                    peer_grad_offsets=[G1.data_ptr() - G0.data_ptr()])
    assert rc == 2


@pytest.mark.parametrize("world,gdt", [(2, 1), (4, 1), (3, 0)])
def test_virtual_ranks_with_global_norm_clipping(world, gdt):
    """Averaging over the ranks and clipping in the same launch: the mean is formed first, the clip acts on it
    (the sum of squares is that of the mean gradients of all slices, as a sharded caller would all-reduce it)."""
    import torch

    from flashoptim_jax_b200 import _engine as eng

    rng = np.random.default_rng(40 + world)
    g_np = {0: np.float32, 1: ml_dtypes.bfloat16}[gdt]
    per = 3 * 2048 + 5 * 32
    n = per * world - 9
    lo = [k * per for k in range(world)]
    hi = [min(n, (k + 1) * per) for k in range(world)]
    p0 = rng.normal(0, 0.05, n).astype(np.float32).astype(ml_dtypes.bfloat16)
    refs = [H.fresh_leaf(p0[lo[k]:hi[k]].copy(), C.ADAM, C.STATE_QUANT, 16) for k in range(world)]
    P = [H.to_torch(p0.copy()) for _ in range(world)]
    G = [torch.zeros(n, dtype=torch.float32 if gdt == 0 else torch.bfloat16, device="cuda") for _ in range(world)]
    devs = []
    for k in range(world):
        st = H.fresh_leaf(p0[lo[k]:hi[k]].copy(), C.ADAM, C.STATE_QUANT, 16).to_device()
        st.param = P[k][lo[k]:hi[k]]
        devs.append(st)
    for t in range(2):
        gs = [H.make_grad(rng, n, 2e-2, g_np) for _ in range(world)]
        means = [_mean_grad([g[lo[k]:hi[k]] for g in gs], k, g_np) for k in range(world)]
        sq = eng.sq_norm_of([H.to_torch(m) for m in means])
        sq_host = float(sq.cpu())
        assert np.float32(np.sqrt(sq_host)) > np.float32(0.5)  # the clip bites
        hp = H.hyper_tuple(C.ADAM, O.FUSED, t + 1, lr=1e-2, wd=1e-2)
        for k, g in enumerate(O.clip_by_global_norm(means, 0.5, sq_norm=sq_host)):
            H.oracle_step(C.ADAM, g, refs[k], C.STATE_QUANT, 32, hp)
        for k in range(world):
            G[k].copy_(H.to_torch(gs[k]))
        for k in range(world):
            others = [j for j in range(world) if j != k]
            H.abi_step(C.ADAM, [G[k][lo[k]:hi[k]]], [devs[k]], C.STATE_QUANT, 32, [hp], [0], 1, gdt, 16,
                       peer_param_offsets=[P[j].data_ptr() - P[k].data_ptr() for j in others],
                       peer_grad_offsets=[G[j].data_ptr() - G[k].data_ptr() for j in others],
                       grad_sq_norm=sq, max_grad_norm=0.5)
        torch.cuda.synchronize()
    for k in range(world):
        H.assert_leaf_equal(devs[k].to_host(), refs[k], f"rank {k} slice")
