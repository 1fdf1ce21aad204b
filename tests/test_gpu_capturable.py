"""A step with no host scalar in it: count, learning rate and bias corrections formed on the device
(fo_step_scalars), the whole `tx.step` captured in a CUDA graph and replayed."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_device_bias_corrections_equal_the_host_formula():
    import torch

    from flashoptim_jax_b200 import _engine as eng

    for b1, b2 in ((0.9, 0.999), (0.95, 0.99), (0.8, 0.9999)):
        count = torch.zeros((), dtype=torch.int32, device="cuda")
        outs = [eng.step_scalars(count, 3e-4, b1, b2, write_count=True) for _ in range(3000)]
        got = torch.stack(outs).cpu().numpy()
        assert int(count) == 3000
        want1 = np.array([eng.bias_correction(b1, c) for c in range(1, 3001)], dtype=np.float32)
        want2 = np.array([eng.bias_correction(b2, c) for c in range(1, 3001)], dtype=np.float32)
        assert np.array_equal(got[:, 0], np.full(3000, np.float32(3e-4)))
        assert np.array_equal(got[:, 1].view(np.uint32), want1.view(np.uint32))
        assert np.array_equal(got[:, 2].view(np.uint32), want2.view(np.uint32))


def _tree(seed, scale, device="cuda"):
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)
    return {"w": (torch.randn(257, 130, generator=g) * scale).bfloat16().to(device),
            "norm": (torch.randn(130, generator=g) * scale).to(device)}


def test_step_captured_in_a_cuda_graph_replays_like_eager_steps():
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree

    groups = [{"params": "norm", "weight_decay": 0.0, "learning_rate": 1e-3}]
    lrs = [1e-3, 8e-4, 6e-4, 4e-4, 2e-4]
    # eager steps with host scalars
    want_p = _tree(0, 0.02)
    plain_state = None
    for t, lr in enumerate(lrs):
        plain = fo.flash_adamw(learning_rate=lr, master_weight_bits=32, donate=True, param_groups=groups)
        if plain_state is None:
            plain_state = plain.init(want_p)
        want_p, plain_state = plain.step(want_p, plain_state, _tree(100 + t, 1e-3))

    lr_dev = torch.tensor(lrs[0], dtype=torch.float32, device="cuda")
    tx = fo.flash_adamw(learning_rate=lr_dev, master_weight_bits=32, donate=True, capturable=True, param_groups=groups)
    params = _tree(0, 0.02)
    state = tx.init(params)
    static_grads = _tree(100, 1e-3)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # step 1, eager: also moves the counter to the device
        params, state = tx.step(params, state, static_grads)
    torch.cuda.current_stream().wait_stream(side)
    assert state.count.is_cuda and int(state.count) == 1
    graph = torch.cuda.CUDAGraph()
    for leaf, new in zip(tree.tree_leaves(static_grads), tree.tree_leaves(_tree(101, 1e-3))):
        leaf.copy_(new)
    lr_dev.fill_(lrs[1])
    with torch.cuda.graph(graph):  # step 2, captured (capture does not run it)
        params, state = tx.step(params, state, static_grads)
    graph.replay()
    for t in (2, 3, 4):  # steps 3..5: new gradients and learning rate, the same graph
        for leaf, new in zip(tree.tree_leaves(static_grads), tree.tree_leaves(_tree(100 + t, 1e-3))):
            leaf.copy_(new)
        lr_dev.fill_(lrs[t])
        graph.replay()
    torch.cuda.synchronize()
    assert int(state.count) == 5
    for a, b in zip(tree.tree_leaves(params), tree.tree_leaves(want_p)):
        assert torch.equal(a, b)
    for name in ("mu", "nu", "ecc"):
        for a, b in zip(tree.tree_leaves(getattr(state, name)), tree.tree_leaves(getattr(plain_state, name))):
            assert torch.equal(torch.as_tensor(a), torch.as_tensor(b))


@pytest.mark.parametrize("name,kw", [("flash_lion", dict(weight_decay=1e-2)), ("flash_sgdw", dict(momentum=0.9, weight_decay=1e-2))])
def test_capturable_lion_and_sgd_equal_the_host_scalar_steps(name, kw):
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree

    make = getattr(fo, name)
    lrs = [1e-3, 5e-4, 2e-4]
    want_p, plain_state = _tree(0, 0.02), None
    for t, lr in enumerate(lrs):
        plain = make(learning_rate=lr, master_weight_bits=24, donate=True, **kw)
        if plain_state is None:
            plain_state = plain.init(want_p)
        want_p, plain_state = plain.step(want_p, plain_state, _tree(100 + t, 1e-3))
    lr_dev = torch.tensor(lrs[0], dtype=torch.float32, device="cuda")
    tx = make(learning_rate=lr_dev, master_weight_bits=24, donate=True, capturable=True, **kw)
    params = _tree(0, 0.02)
    state = tx.init(params)
    for t, lr in enumerate(lrs):
        lr_dev.fill_(lr)
        params, state = tx.step(params, state, _tree(100 + t, 1e-3))
    torch.cuda.synchronize()
    assert state.count.is_cuda and int(state.count) == 3
    for a, b in zip(tree.tree_leaves(params), tree.tree_leaves(want_p)):
        assert torch.equal(a, b)
    for field in ("mu", "ecc"):
        for a, b in zip(tree.tree_leaves(getattr(state, field)), tree.tree_leaves(getattr(plain_state, field))):
            assert torch.equal(torch.as_tensor(a), torch.as_tensor(b))


def test_device_schedule_equals_its_host_formula_and_drives_a_capturable_step():
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import _engine as eng
    from flashoptim_jax_b200 import tree
    from flashoptim_jax_b200.schedules import warmup_cosine

    sched = warmup_cosine(total_steps=400, warmup_steps=37, peak_lr=3e-4)
    count = torch.zeros((), dtype=torch.int32, device="cuda")
    outs = [eng.step_scalars(count, sched, 0.9, 0.999, write_count=True) for _ in range(450)]
    got = torch.stack(outs).cpu().numpy()[:, 0]
    want = np.array([sched(c) for c in range(450)], dtype=np.float32)  # the schedule sees the zero-based count
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))

    # the same schedule on the host (called with the count) and on the device (capturable) give the same steps
    host_tx = fo.flash_adamw(learning_rate=sched, master_weight_bits=32, donate=True)
    dev_tx = fo.flash_adamw(learning_rate=sched, master_weight_bits=32, donate=True, capturable=True)
    hp, dp = _tree(0, 0.02), _tree(0, 0.02)
    hs, ds = host_tx.init(hp), dev_tx.init(dp)
    for t in range(4):
        hp, hs = host_tx.step(hp, hs, _tree(100 + t, 1e-3))
        dp, ds = dev_tx.step(dp, ds, _tree(100 + t, 1e-3))
    torch.cuda.synchronize()
    for a, b in zip(tree.tree_leaves(hp), tree.tree_leaves(dp)):
        assert torch.equal(a, b)
