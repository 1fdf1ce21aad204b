"""The multi-tensor launch: many leaves, many hyper sets, unaligned leaves, guard bytes, device scalars."""

import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _leaves(rng, sizes, opt, ecc_bits, pdt=1):
    refs = []
    for n in sizes:
        p = rng.normal(0, 0.05, n).astype(np.float32).astype(H.NP_OF_CODE[pdt])
        refs.append(H.fresh_leaf(p, opt, C.STATE_QUANT, ecc_bits))
    return refs


def test_resnet_like_tree_in_one_call():
    # many tiny leaves (BatchNorm-sized vectors) next to conv-sized ones, SGDW with momentum (config 3 shapes in miniature)
    import torch

    rng = np.random.default_rng(0)
    sizes = [7 * 7 * 3 * 64, 64, 64, 64 * 64, 3 * 3 * 64 * 64, 256, 256, 1000, 2048 * 10, 1, 33, 2049] * 14  # 168 leaves
    refs = _leaves(rng, sizes, C.SGD, 8)
    devs = [r.copy().to_device() for r in refs]
    for t in range(1, 4):
        grads = [H.make_grad(rng, n, 1e-3, H.BF16) for n in sizes]
        hp = H.hyper_tuple(C.SGD, O.FUSED, t, lr=0.1, wd=1e-4, momentum=0.9)
        for g, r in zip(grads, refs):
            H.oracle_step(C.SGD, g, r, C.STATE_QUANT, 32, hp)
        H.abi_step(C.SGD, [H.to_torch(g) for g in grads], devs, C.STATE_QUANT, 32, [hp], [0] * len(sizes), 1, 1, 8)
    torch.cuda.synchronize()
    for i, (d, r) in enumerate(zip(devs, refs)):
        H.assert_leaf_equal(d.to_host(), r, f"leaf {i} n={sizes[i]}")


def test_more_leaves_than_one_launch_holds_and_many_hyper_sets():
    import torch

    rng = np.random.default_rng(1)
    sizes = [int(s) for s in rng.integers(1, 5000, 700)]  # > 320 leaves: several launches inside one call
    refs = _leaves(rng, sizes, C.ADAM, 16)
    devs = [r.copy().to_device() for r in refs]
    lrs = [1e-3 * (1 + k) for k in range(16)]  # 16 hyper sets, the most one call carries
    hyper_of = [i % 16 for i in range(len(sizes))]
    for t in range(1, 3):
        grads = [H.make_grad(rng, n, 1e-3, H.BF16) for n in sizes]
        hps = [H.hyper_tuple(C.ADAM, O.FUSED, t, lr=lr, wd=1e-2 * (k % 3)) for k, lr in enumerate(lrs)]
        for g, r, k in zip(grads, refs, hyper_of):
            H.oracle_step(C.ADAM, g, r, C.STATE_QUANT, 32, hps[k])
        H.abi_step(C.ADAM, [H.to_torch(g) for g in grads], devs, C.STATE_QUANT, 32, hps, hyper_of, 1, 1, 16)
    torch.cuda.synchronize()
    for i, (d, r) in enumerate(zip(devs, refs)):
        H.assert_leaf_equal(d.to_host(), r, f"leaf {i} n={sizes[i]} hyper {hyper_of[i]}")
    # a 17th set is refused, nothing is launched
    hps17 = hps + [hps[0]]
    rc = H.abi_step(C.ADAM, [H.to_torch(H.make_grad(rng, n, 1e-3, H.BF16)) for n in sizes[:2]], devs[:2], C.STATE_QUANT, 32, hps17,
                    [0, 16], 1, 1, 16, expect_ok=False)
    assert rc == 4


def test_unaligned_leaves_and_guard_bytes():
    # leaves carved out of one allocation at odd offsets, with sentinel bytes between them that must survive
    import torch

    rng = np.random.default_rng(2)
    n = 5000
    for opt, ecc_bits in ((C.ADAM, 16), (C.ADAM, 8), (C.LION, 8)):
        for offset in (1, 3, 8):
            p = rng.normal(0, 0.05, n).astype(np.float32).astype(H.BF16)
            ref = H.fresh_leaf(p, opt, C.STATE_QUANT, ecc_bits)

            def carve(arr, fill):
                if arr is None:
                    return None, None
                t = H.to_torch(arr)
                pad = 64
                big = torch.full((t.numel() + 2 * pad + offset,), fill, dtype=t.dtype, device="cuda")
                view = big[pad + offset: pad + offset + t.numel()]
                view.copy_(t.reshape(-1))
                return big, view

            bigs, views = {}, {}
            for f in ref.fields():
                fill = 77 if getattr(ref, f) is not None and getattr(ref, f).dtype.kind in "iu" else 1.5
                bigs[f], views[f] = carve(getattr(ref, f), fill)
            dev = H.LeafArrays(*[views[f] for f in ref.fields()])
            for t in range(1, 3):
                g = H.make_grad(rng, n, 1e-3, H.BF16)
                gbig, gview = carve(g, 1.5)
                hp = H.hyper_tuple(opt, O.FUSED, t, lr=1e-3, wd=1e-2, **({"b2": 0.99} if opt == C.LION else {}))
                H.oracle_step(opt, g, ref, C.STATE_QUANT, 32, hp)
                H.abi_step(opt, [gview], [dev], C.STATE_QUANT, 32, [hp], [0], 1, 1, ecc_bits)
            torch.cuda.synchronize()
            H.assert_leaf_equal(dev.to_host(), ref, f"opt {opt} offset {offset}")
            for f, big in bigs.items():
                if big is None:
                    continue
                inner = views[f].numel()
                guard = torch.cat([big[: 64 + offset], big[64 + offset + inner:]])
                fill = 77 if big.dtype in (torch.int8, torch.uint8, torch.int16) else 1.5
                assert torch.all(guard == fill), f"{f}: bytes outside the leaf were written"


def test_device_scalars_override_host_values():
    # lr, bc1, bc2 read from device memory (a traced schedule / step count needs no host round trip)
    import torch

    rng = np.random.default_rng(3)
    n = 3 * 2048 + 100
    p = rng.normal(0, 0.05, n).astype(np.float32).astype(H.BF16)
    ref = H.fresh_leaf(p, C.ADAM, C.STATE_QUANT, 8)
    dev = ref.copy().to_device()
    for t in range(1, 4):
        g = H.make_grad(rng, n, 1e-3, H.BF16)
        hp = H.hyper_tuple(C.ADAM, O.FUSED, t, lr=1e-3 * t, wd=1e-2)
        H.oracle_step(C.ADAM, g, ref, C.STATE_QUANT, 32, hp)
        scal = torch.tensor([float(hp[0]), float(hp[7]), float(hp[8])], dtype=torch.float32, device="cuda")
        wrong = (np.float32(123.0),) + tuple(hp[1:7]) + (np.float32(0.5), np.float32(0.25), hp[9], scal.data_ptr())
        H.abi_step(C.ADAM, [H.to_torch(g)], [dev], C.STATE_QUANT, 32, [wrong], [0], 1, 1, 8)
        torch.cuda.synchronize()
    H.assert_leaf_equal(dev.to_host(), ref, "device scalars")


def test_empty_and_zero_length_leaves():
    import torch

    rng = np.random.default_rng(4)
    refs = _leaves(rng, [100, 64], C.ADAM, 8)
    devs = [r.copy().to_device() for r in refs]
    empty = H.LeafArrays(*[torch.empty(0, dtype=dt, device="cuda") for dt in (torch.bfloat16, torch.int8, torch.int8, torch.float16, torch.uint8, torch.float16)])
    grads = [H.make_grad(rng, 100, 1e-3, H.BF16), H.make_grad(rng, 64, 1e-3, H.BF16)]
    hp = H.hyper_tuple(C.ADAM, O.FUSED, 1, lr=1e-3, wd=1e-2)
    for g, r in zip(grads, refs):
        H.oracle_step(C.ADAM, g, r, C.STATE_QUANT, 32, hp)
    H.abi_step(C.ADAM, [H.to_torch(grads[0]), torch.empty(0, dtype=torch.bfloat16, device="cuda"), H.to_torch(grads[1])],
               [devs[0], empty, devs[1]], C.STATE_QUANT, 32, [hp], [0, 0, 0], 1, 1, 8)
    torch.cuda.synchronize()
    for d, r in zip(devs, refs):
        H.assert_leaf_equal(d.to_host(), r, "around an empty leaf")
    assert H.abi_step(C.ADAM, [], [], C.STATE_QUANT, 32, [hp], [], 1, 1, 8) == 0


def test_runs_on_a_side_stream():
    import torch

    rng = np.random.default_rng(5)
    n = 40000
    p = rng.normal(0, 0.05, n).astype(np.float32).astype(H.BF16)
    ref = H.fresh_leaf(p, C.LION, C.STATE_QUANT, 8)
    dev = ref.copy().to_device()
    g = H.make_grad(rng, n, 1e-3, H.BF16)
    hp = H.hyper_tuple(C.LION, O.FUSED, 1, lr=1e-4, wd=1e-2, b2=0.99)
    H.oracle_step(C.LION, g, ref, C.STATE_QUANT, 32, hp)
    gt = H.to_torch(g)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        H.abi_step(C.LION, [gt], [dev], C.STATE_QUANT, 32, [hp], [0], 1, 1, 8, stream=s.cuda_stream)
    s.synchronize()
    H.assert_leaf_equal(dev.to_host(), ref, "side stream")
