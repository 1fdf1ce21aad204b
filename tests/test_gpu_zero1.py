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
