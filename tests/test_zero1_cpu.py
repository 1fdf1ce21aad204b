"""ZeRO-1 host logic on CPU ranks (gloo): shard tables, flat-buffer views, collectives plumbing.

The device kernels cannot run here, so the tests inject a step function that applies the
CPU oracle to each LeafWork in place; what is under test is everything around the kernel.
With identical gradients on both ranks the mean is exact, so the sharded result must equal
the unsharded one bit for bit.
"""

import os
import socket

import ml_dtypes
import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashoptim_jax_b200.zero1 import LEAF_ALIGN, SHARD_ALIGN, Zero1Optimizer, plan_bucket


def test_plan_bucket_covers_every_element_once_on_group_boundaries():
    sizes = [5, 4096, 33, 100000, 2048, 1]
    from flashoptim_jax_b200.zero1 import flat_position

    for world, n_slices in ((1, 1), (2, 1), (3, 2), (4, 4), (8, 3), (2, None)):
        lay = plan_bucket(torch.bfloat16, list(range(len(sizes))), sizes, world, n_slices)
        assert lay.piece % SHARD_ALIGN == 0 and lay.shard == lay.piece * lay.n_slices and lay.total == lay.shard * world
        assert all(s % LEAF_ALIGN == 0 for s in lay.starts)
        seen = {i: [] for i in range(len(sizes))}
        for r, segs in enumerate(lay.segments):
            for seg in segs:
                assert 0 <= seg.offset and seg.offset + (seg.hi - seg.lo) <= lay.shard
                assert seg.offset // lay.piece == seg.slice == (seg.offset + seg.hi - seg.lo - 1) // lay.piece
                assert seg.lo % 32 == 0  # a cut inside a leaf falls on a group boundary
                assert lay.starts[seg.leaf] + seg.lo == flat_position(lay, r, seg.offset)
                seen[seg.leaf].append((seg.lo, seg.hi))
        for i, n in enumerate(sizes):
            spans = sorted(seen[i])
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _np_view(t: torch.Tensor) -> np.ndarray:
    """NumPy view sharing memory with a CPU tensor (bf16 through its bit pattern)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.numpy()


def oracle_step_fn(opt, work):
    """Stand-in for eng.launch on CPU tensors: the C oracle, in place, leaf by leaf."""
    from oracle import c_oracle as C

    for w in work:
        _, pdt, gdt, ecc_bits, state, group = w.bucket
        h = C.Hyper(*[float(x) for x in w.hyper[:9]])
        arr = lambda t: None if t is None else _np_view(t)  # noqa: E731
        C.step_leaf(opt, arr(w.grad), arr(w.param), arr(w.ecc), arr(w.mu), arr(w.mu_scales), arr(w.nu), arr(w.nu_scales),
                    state=state, group_size=group, hyper=h, flags=int(w.hyper[9]))
    return 1


def _make_params():
    g = torch.Generator().manual_seed(0)
    return {
        "emb": (torch.randn(300, 70, generator=g) * 0.02).to(torch.bfloat16),
        "layers": [{"w": (torch.randn(64, 65, generator=g) * 0.02).to(torch.bfloat16), "norm": torch.ones(65)} for _ in range(3)],
        "bias": torch.zeros(7),
    }


def _make_grads(step: int):
    g = torch.Generator().manual_seed(100 + step)
    return {
        "emb": (torch.randn(300, 70, generator=g) * 1e-3).to(torch.bfloat16),
        "layers": [{"w": (torch.randn(64, 65, generator=g) * 1e-3).to(torch.bfloat16), "norm": torch.randn(65, generator=g) * 1e-3}
                   for _ in range(3)],
        "bias": torch.randn(7, generator=g) * 1e-3,
    }


def _run(kind, hp, steps=3, n_slices=None):
    z = Zero1Optimizer(kind, _make_params(), step_fn=oracle_step_fn, n_slices=n_slices, **hp)
    for t in range(steps):
        z.step(_make_grads(t))
    return z


def _worker(rank, world, port, kind, hp, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        z = _run(kind, hp, n_slices=3 if kind == "adamw" else None)  # adamw: three slices per bucket
        state = z.gather_state(dst=0)
        local = z.local_state_dict()
        z.load_local_state_dict(local)  # round trip of the per-rank shard
        sd = z.state_dict()  # collective: the reference's checkpoint form, on every rank
        shard_dir = os.path.join(os.path.dirname(out), "shards")
        z.save_shards(shard_dir)
        fresh = Zero1Optimizer(kind, _make_params(), step_fn=oracle_step_fn, n_slices=3 if kind == "adamw" else None, **hp)
        fresh.load_shards(shard_dir)
        same = fresh.count == z.count and all(
            (a is None and b is None) or torch.equal(a, b) for k in z.state for a, b in zip(z.state[k], fresh.state[k]))
        again = Zero1Optimizer(kind, _make_params(), step_fn=oracle_step_fn, **hp)  # another slicing of the same buckets
        again.load_state_dict(sd)
        sd2 = again.state_dict()
        if rank == 0:
            from flashoptim_jax_b200 import tree, utils

            flat = lambda d: [x for name in ("mu", "nu", "ecc") if name in d for x in tree.tree_leaves(utils._tree_from_state_dict(d[name]))]  # noqa: E731
            torch.save({"params": tree.tree_leaves(z.params), "state": tree.tree_leaves(state), "count": z.count,
                        "segments": len(local["segments"]), "state_dict": flat(sd), "state_dict_again": flat(sd2),
                        "shards_round_trip": same, "sd_count": int(sd["count"])}, out)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("kind,hp", [
    ("adamw", dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=32)),
    ("lion", dict(learning_rate=1e-4, weight_decay=1e-2)),
    ("sgdw", dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2, nesterov=True)),
], ids=["adamw", "lion", "sgdw"])
def test_two_ranks_match_one_rank_bit_for_bit(tmp_path, kind, hp):
    from flashoptim_jax_b200 import tree

    single = _run(kind, hp)
    want_params = tree.tree_leaves(single.params)
    want_state = tree.tree_leaves(single.gather_state())
    out = str(tmp_path / "rank0.pt")
    mp.spawn(_worker, args=(2, _free_port(), kind, hp, out), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    assert got["count"] == single.count == 3
    for a, b in zip(got["params"], want_params):
        assert a.dtype == b.dtype and torch.equal(a.view(torch.uint8) if a.dtype != torch.float32 else a, b.view(torch.uint8) if b.dtype != torch.float32 else b)
    assert len(got["state"]) == len(want_state)
    for a, b in zip(got["state"], want_state):
        assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    # the device-side gather gives the unsharded optimizer's state dict, also after re-sharding; per-rank files round-trip
    from flashoptim_jax_b200 import utils

    want_sd = single.state_dict()
    want_flat = [x for name in ("mu", "nu", "ecc") if name in want_sd for x in tree.tree_leaves(utils._tree_from_state_dict(want_sd[name]))]
    assert got["sd_count"] == 3 and got["shards_round_trip"]
    for key in ("state_dict", "state_dict_again"):
        assert len(got[key]) == len(want_flat)
        for a, b in zip(got[key], want_flat):
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)


def test_state_dict_has_the_reference_checkpoint_form():
    z = _run("adamw", dict(learning_rate=1e-3), steps=1)
    sd = z.state_dict()
    assert set(sd) == {"count", "mu", "nu", "ecc"} and int(sd["count"]) == 1
    for name in ("mu", "nu", "ecc"):
        assert set(sd[name]) == {"treedef", "leaves"} and len(sd[name]["leaves"]) == 8
    assert sd["mu"]["leaves"][0]["kind"] == "quantized" and set(sd["mu"]["leaves"][0]) == {"kind", "values", "scales"}
    kinds = {leaf["kind"] for leaf in sd["ecc"]["leaves"]}
    assert kinds == {"array"}
    other = Zero1Optimizer("adamw", _make_params(), step_fn=oracle_step_fn, learning_rate=1e-3)
    other.load_state_dict(sd)
    assert other.count == 1 and all((a is None and b is None) or torch.equal(a, b) for k in z.state for a, b in zip(z.state[k], other.state[k]))
    with pytest.raises(ValueError):
        bad = dict(sd, mu={"treedef": sd["mu"]["treedef"], "leaves": sd["mu"]["leaves"][:-1]})
        other.load_state_dict(bad)


def test_gathered_state_has_the_reference_layout():
    from flashoptim_jax_b200.quantization import QuantizedArray

    z = _run("adamw", dict(learning_rate=1e-3), steps=1)
    st = z.gather_state()
    assert set(st) == {"count", "mu", "nu", "ecc"} and int(st["count"]) == 1
    assert isinstance(st["mu"]["emb"], QuantizedArray) and st["mu"]["emb"].values.shape == (300, 70)
    assert st["mu"]["emb"].scales.shape == (300 * 70 // 32 + 1,)
    assert st["ecc"]["emb"].dtype == torch.int8 and st["ecc"]["bias"].dtype == torch.int32 and st["ecc"]["bias"].shape == ()
    assert isinstance(st["nu"]["layers"][1]["norm"], QuantizedArray)


def test_views_and_argument_checks():
    z = Zero1Optimizer("adamw", _make_params(), step_fn=oracle_step_fn)
    bf16 = [b for b, lay in enumerate(z.buckets) if lay.dtype == torch.bfloat16][0]
    assert z.params["emb"].data_ptr() == z.flat_params[bf16].data_ptr()  # leaves are views into the flat buffer
    assert z.grads["emb"].data_ptr() == z.flat_grads[bf16].data_ptr()
    with pytest.raises(ValueError, match="must match parameter structure"):
        z.step({"emb": torch.zeros(1)})
    with pytest.raises(ValueError, match="group_size must be 32"):
        Zero1Optimizer("adamw", _make_params(), step_fn=oracle_step_fn, group_size=64)
    with pytest.raises(TypeError, match="unexpected hyper-parameters"):
        Zero1Optimizer("lion", _make_params(), step_fn=oracle_step_fn, eps=1e-8)
    with pytest.raises(ValueError, match="unknown optimizer"):
        Zero1Optimizer("rmsprop", _make_params())
