"""ZeRO-1 on GPUs: one rank must equal the plain tx.step; two NCCL ranks (when two GPUs are
visible) must equal one rank bit for bit when every rank holds the same gradients."""

import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _params(device):
    import torch

    g = torch.Generator(device="cpu").manual_seed(0)
    return {
        "emb": (torch.randn(3000, 70, generator=g) * 0.02).to(torch.bfloat16).to(device),
        "layers": [{"w": (torch.randn(640, 65, generator=g) * 0.02).to(torch.bfloat16).to(device), "norm": torch.ones(65, device=device)}
                   for _ in range(3)],
        "bias": torch.zeros(7, device=device),
    }


def _grads(step, device):
    import torch

    g = torch.Generator(device="cpu").manual_seed(100 + step)
    return {
        "emb": (torch.randn(3000, 70, generator=g) * 1e-3).to(torch.bfloat16).to(device),
        "layers": [{"w": (torch.randn(640, 65, generator=g) * 1e-3).to(torch.bfloat16).to(device),
                    "norm": (torch.randn(65, generator=g) * 1e-3).to(device)} for _ in range(3)],
        "bias": (torch.randn(7, generator=g) * 1e-3).to(device),
    }


HP = dict(learning_rate=1e-3, weight_decay=1e-2, master_weight_bits=32)


def test_one_rank_equals_plain_step():
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    dev = torch.device("cuda", 0)
    z = Zero1Optimizer("adamw", _params(dev), **HP)
    tx = fo.flash_adamw(donate=True, **HP)
    params = _params(dev)
    state = tx.init(params)
    for t in range(3):
        z.step(_grads(t, dev))
        params, state = tx.step(params, state, _grads(t, dev))
    torch.cuda.synchronize()
    for a, b in zip(tree.tree_leaves(z.params), tree.tree_leaves(params)):
        assert torch.equal(a, b)
    zs = z.gather_state()
    for name in ("mu", "nu", "ecc"):
        for a, b in zip(tree.tree_leaves(zs[name]), tree.tree_leaves(getattr(state, name))):
            assert a.dtype == b.dtype and torch.equal(a.cpu(), b.cpu())


def _worker(rank, world, port, out, mode="nccl", own_grads=False, use_switch=False):
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # nccl: three slices exercise the pipelined NCCL path; fused_ag: all-gather by peer stores inside the
        # kernel; fused: reduce-scatter by peer loads inside the kernel as well
        z = Zero1Optimizer("adamw", _params(dev), n_slices=3 if mode == "nccl" else 1, fused_allgather=mode != "nccl",
                           fused_reduce_scatter=mode == "fused", use_switch=use_switch, **HP)
        assert bool(use_switch) == (any(z.mc_param_offsets) and any(z.mc_grad_offsets))
        for t in range(3):
            z.step(_grads(t + (100 * rank if own_grads else 0), dev))
        torch.cuda.synchronize()
        state = z.gather_state(dst=0)
        if rank == 0:
            torch.save({"params": [p.cpu() for p in tree.tree_leaves(z.params)], "state": [s.cpu() for s in tree.tree_leaves(state)]}, out)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["nccl", "fused_ag", "fused"])
def test_two_nccl_ranks_equal_one_rank(tmp_path, mode):
    import torch
    import torch.multiprocessing as mp

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dev = torch.device("cuda", 0)
    single = Zero1Optimizer("adamw", _params(dev), **HP)
    for t in range(3):
        single.step(_grads(t, dev))
    want_p = [p.cpu() for p in tree.tree_leaves(single.params)]
    want_s = [s.cpu() for s in tree.tree_leaves(single.gather_state())]
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), out, mode), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    for a, b in zip(got["params"], want_p):
        assert torch.equal(a, b)
    for a, b in zip(got["state"], want_s):
        assert a.dtype == b.dtype and torch.equal(a, b)


@pytest.mark.parametrize("mode", ["fused", "nccl"])
def test_two_ranks_with_their_own_gradients_step_on_the_mean(tmp_path, mode):
    """Different gradients on the two ranks: the result is the one-rank step on their mean (fp32 sum, halved,
    rounded once to the gradient dtype) - by the kernel's own averaging, and by NCCL's for two ranks."""
    import torch
    import torch.multiprocessing as mp

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dev = torch.device("cuda", 0)
    single = Zero1Optimizer("adamw", _params(dev), **HP)
    for t in range(3):
        g0, g1 = _grads(t, dev), _grads(t + 100, dev)
        mean = tree.tree_map(lambda a, b: ((a.float() + b.float()) * 0.5).to(a.dtype), g0, g1)
        single.step(mean)
    want_p = [p.cpu() for p in tree.tree_leaves(single.params)]
    want_s = [s.cpu() for s in tree.tree_leaves(single.gather_state())]
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), out, mode, True), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    for a, b in zip(got["params"], want_p):
        assert torch.equal(a, b)
    for a, b in zip(got["state"], want_s):
        assert a.dtype == b.dtype and torch.equal(a, b)


def test_one_rank_with_max_grad_norm_equals_the_clipping_wrapper():
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.clipping import clip_by_global_norm
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    dev = torch.device("cuda", 0)
    z = Zero1Optimizer("adamw", _params(dev), max_grad_norm=0.05, **HP)
    tx = clip_by_global_norm(fo.flash_adamw(donate=True, **HP), 0.05)
    params = _params(dev)
    state = tx.init(params)
    for t in range(3):
        z.step(_grads(t, dev))
        params, state = tx.step(params, state, _grads(t, dev))
    torch.cuda.synchronize()
    for a, b in zip(tree.tree_leaves(z.params), tree.tree_leaves(params)):
        assert torch.equal(a, b)
    plain = Zero1Optimizer("adamw", _params(dev), **HP)
    for t in range(3):
        plain.step(_grads(t, dev))
    assert any(not torch.equal(a, b) for a, b in zip(tree.tree_leaves(z.params), tree.tree_leaves(plain.params)))  # the clip did bite


def test_two_ranks_through_the_switch_with_equal_gradients(tmp_path):
    """use_switch=True: multicast stores and multicast load-reduces.  The switch's 16-bit addition is not
    round-to-nearest in general, but g + g is exact in any arithmetic: with equal gradients on both ranks
    the result is still the one-rank result, bit for bit."""
    import torch
    import torch.multiprocessing as mp

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dev = torch.device("cuda", 0)
    single = Zero1Optimizer("adamw", _params(dev), **HP)
    for t in range(3):
        single.step(_grads(t, dev))
    want_p = [p.cpu() for p in tree.tree_leaves(single.params)]
    want_s = [s.cpu() for s in tree.tree_leaves(single.gather_state())]
    out = str(tmp_path / "r0.pt")
    try:
        mp.spawn(_worker, args=(2, _free_port(), out, "fused", False, True), nprocs=2, join=True)
    except Exception as e:  # no multicast mapping on this system
        if "multicast" in str(e):
            pytest.skip("symmetric memory without multicast support")
        raise
    got = torch.load(out, weights_only=False)
    for a, b in zip(got["params"], want_p):
        assert torch.equal(a, b)
    for a, b in zip(got["state"], want_s):
        assert a.dtype == b.dtype and torch.equal(a, b)


def test_step_from_host_equals_step():
    import torch

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    dev = torch.device("cuda", 0)
    a = Zero1Optimizer("adamw", _params(dev), **HP)
    b = Zero1Optimizer("adamw", _params(dev), **HP)
    for t in range(3):
        g = _grads(t, dev)
        host = tree.tree_map(lambda x: x.cpu().pin_memory(), g)
        a.step(g)
        b.step_from_host(host, n_groups=3)
    torch.cuda.synchronize()
    assert b.count == 3
    for x, y in zip(tree.tree_leaves(a.params), tree.tree_leaves(b.params)):
        assert torch.equal(x, y)
    for x, y in zip(tree.tree_leaves(a.gather_state()), tree.tree_leaves(b.gather_state())):
        assert torch.equal(torch.as_tensor(x), torch.as_tensor(y))


def test_step_from_host_steps_every_segment_of_a_sliced_leaf():
    """One rank, three slices per bucket: leaves straddle slice boundaries, so a leaf has several segments and
    step_from_host must step them all."""
    import torch

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    dev = torch.device("cuda", 0)
    a = Zero1Optimizer("adamw", _params(dev), n_slices=3, **HP)
    b = Zero1Optimizer("adamw", _params(dev), n_slices=3, **HP)
    assert any(len({seg.slice for seg in layout.segments[0] if seg.leaf == leaf}) > 1
               for layout in b.buckets for leaf in layout.leaves)  # some leaf does straddle
    for t in range(3):
        g = _grads(t, dev)
        host = tree.tree_map(lambda x: x.cpu().pin_memory(), g)
        a.step(g)
        b.step_from_host(host, n_groups=4)
    torch.cuda.synchronize()
    for x, y in zip(tree.tree_leaves(a.params), tree.tree_leaves(b.params)):
        assert torch.equal(x, y)
    for x, y in zip(tree.tree_leaves(a.gather_state()), tree.tree_leaves(b.gather_state())):
        assert torch.equal(torch.as_tensor(x), torch.as_tensor(y))


def _rank_grad(rank, n):
    import torch

    g = torch.Generator(device="cpu").manual_seed(5000 + rank)
    return (torch.randn(n, generator=g) * 1e-3).to(torch.bfloat16)


MEAN_N = 3 * 4096 + 32 * 5


def _mean_worker(rank, world, port, out, route):
    """Plain SGD from zero parameters with learning rate 1: the stored parameter is minus the averaged gradient."""
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        z = Zero1Optimizer("sgd", {"w": torch.zeros(MEAN_N, dtype=torch.bfloat16, device=dev)}, learning_rate=1.0, momentum=0.0,
                           weight_decay=0.0, master_weight_bits=32, fused_allgather=route != "nccl",
                           fused_reduce_scatter=route != "nccl", use_switch=route == "switch")
        z.step({"w": _rank_grad(rank, MEAN_N).to(dev)})
        torch.cuda.synchronize()
        if rank == 0:
            torch.save(z.params["w"].cpu(), out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("route", ["peer", "switch", "nccl"])
def test_mean_of_per_rank_gradients_by_route(tmp_path, route, world):
    """Every rank has its own gradients.  Against the mean formed in fp32 and rounded once to bf16: the
    kernel's own averaging over peer loads is that value exactly; the NVLink switch adds in its own
    arithmetic and NCCL rounds at every hop, so both may land on a neighbouring bf16 value: at most one
    place (2^-7 relative) away through the switch, at most one place per hop for NCCL."""
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = str(tmp_path / "w.pt")
    try:
        mp.spawn(_mean_worker, args=(world, _free_port(), out, route), nprocs=world, join=True)
    except Exception as e:
        if route == "switch" and "multicast" in str(e):
            pytest.skip("symmetric memory without multicast support")
        raise
    got = -torch.load(out).float()
    total = torch.zeros(MEAN_N)
    for r in range(world):
        total += _rank_grad(r, MEAN_N).float()  # fp32 sum in rank order, rank 0 first: the order of rank 0's kernel
    exact = (total / world).to(torch.bfloat16).float()
    off = (got != exact)
    if route == "peer":
        # rank 0 owns the first slice and sums in the order own, peers ascending = 0, 1, 2, ...; other ranks start
        # with their own values, which can move an fp32 sum by one place before the single rounding to bf16
        first = MEAN_N // world // 32 * 32
        assert not off[:first].any()
        places = 1.0
    elif route == "switch":
        places = 1.0
    else:
        places = float(world - 1)
    scale = exact.abs()
    if route == "nccl":
        # NCCL rounds its partial sums, which are as large as the largest addend even where the mean cancels
        scale = torch.stack([_rank_grad(r, MEAN_N).float().abs() for r in range(world)]).max(dim=0).values
    ulp = torch.where(scale == 0, torch.full_like(scale, 2.0 ** -133), 2.0 ** (torch.floor(torch.log2(scale)) - 7))
    assert ((got - exact).abs() <= places * ulp + 1e-30).all(), float(((got - exact).abs() / ulp).max())
    print(f"{route} x{world}: {int(off.sum())} of {MEAN_N} means differ from the once-rounded fp32 mean")


def test_checkpoint_export_and_import_on_the_device(tmp_path):
    """One rank on a GPU: state_dict() is the plain optimizer's flash_adamw_state_dict, master_weights() is
    reconstruct_weights, set_master_weights() is set_fp32_params, and the per-rank file round-trips."""
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree, utils
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    dev = torch.device("cuda", 0)
    z = Zero1Optimizer("adamw", _params(dev), **HP)
    tx = fo.flash_adamw(donate=True, **HP)
    params = _params(dev)
    state = tx.init(params)
    for t in range(2):
        z.step(_grads(t, dev))
        params, state = tx.step(params, state, _grads(t, dev))
    want, got = fo.flash_adamw_state_dict(state), z.state_dict()
    assert int(got["count"]) == int(want["count"]) == 2
    for name in ("mu", "nu", "ecc"):
        a = tree.tree_leaves(utils._tree_from_state_dict(got[name]))
        b = tree.tree_leaves(utils._tree_from_state_dict(want[name]))
        assert len(a) == len(b)
        for x, y in zip(a, b):
            assert x.is_cuda and x.dtype == y.dtype and x.shape == y.shape and torch.equal(x, y)
    theta = z.master_weights()
    for x, y in zip(tree.tree_leaves(theta), tree.tree_leaves(fo.reconstruct_weights(params, state.ecc))):
        assert x.dtype == torch.float32 and torch.equal(x, y)
    # import: perturbed master weights go in, come out again exactly where 24/32 bits can hold them
    moved = tree.tree_map(lambda t: (t * 1.0009765625).contiguous(), theta)
    z.set_master_weights(moved)
    want_p, want_e = fo.set_fp32_params(moved, params, master_weight_bits=HP["master_weight_bits"])
    for x, y in zip(tree.tree_leaves(z.params), tree.tree_leaves(want_p)):
        assert torch.equal(x, y)
    for x, y in zip(tree.tree_leaves(utils._tree_from_state_dict(z.state_dict()["ecc"])), tree.tree_leaves(want_e)):
        assert x.dtype == y.dtype and torch.equal(x, y)
    z.save_shards(str(tmp_path))
    other = Zero1Optimizer("adamw", _params(dev), **HP)
    other.load_shards(str(tmp_path))
    assert other.count == 2
    for k in z.state:
        for a, b in zip(z.state[k], other.state[k]):
            assert (a is None and b is None) or torch.equal(a, b)


def _clip_worker(rank, world, port, out, own_grads):
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        z = Zero1Optimizer("adamw", _params(dev), fused_allgather=True, fused_reduce_scatter=True, max_grad_norm=0.05, **HP)
        for t in range(3):
            z.step(_grads(t + (100 * rank if own_grads else 0), dev))
        torch.cuda.synchronize()
        state = z.gather_state(dst=0)
        if rank == 0:
            torch.save({"params": [p.cpu() for p in tree.tree_leaves(z.params)], "state": [s.cpu() for s in tree.tree_leaves(state)]}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("own_grads", [False, True], ids=["equal-grads", "own-grads"])
def test_two_ranks_clip_by_global_norm_with_the_fused_reduce_scatter(tmp_path, own_grads):
    """Clipping together with the reduce-scatter by peer loads: the sweep that sums the squares also forms this
    rank's averaged slice.  The result is the one-rank clipped step on the mean gradient, bit for bit (the
    norm is a sum of doubles in another order: equal to the last place of the float it is rounded to here)."""
    import torch
    import torch.multiprocessing as mp

    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dev = torch.device("cuda", 0)
    single = Zero1Optimizer("adamw", _params(dev), max_grad_norm=0.05, **HP)
    for t in range(3):
        g0 = _grads(t, dev)
        if own_grads:
            g1 = _grads(t + 100, dev)
            g0 = tree.tree_map(lambda a, b: ((a.float() + b.float()) * 0.5).to(a.dtype), g0, g1)
        single.step(g0)
    want_p = [p.cpu() for p in tree.tree_leaves(single.params)]
    want_s = [s.cpu() for s in tree.tree_leaves(single.gather_state())]
    out = str(tmp_path / "r0.pt")
    mp.spawn(_clip_worker, args=(2, _free_port(), out, own_grads), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    for a, b in zip(got["params"], want_p):
        assert torch.equal(a, b)
    for a, b in zip(got["state"], want_s):
        assert a.dtype == b.dtype and torch.equal(a, b)
