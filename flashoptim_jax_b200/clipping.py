"""Global-norm gradient clipping in front of a flash optimizer, with the scaling done inside the
step kernel.

Mirrors `_wrap_flash_with_clip` of the reference's GPT-2 recipe (examples/train_gpt2_pretrain.py:56-70),
which chains `optax.clip_by_global_norm(max_norm)` before `tx.step`:

    norm = sqrt(sum over leaves of sum(g*g));  g <- g if norm < max_norm else (g / norm.astype(g.dtype)) * max_norm

There the clip is a separate pass that reads and rewrites every gradient; here one read-only sweep
(`fo_sq_norm`) leaves the sum of squares in device memory and the step kernel rescales the gradients
as it loads them, with no host round trip.
"""

from __future__ import annotations

from typing import Any

from . import _engine as eng
from . import tree as pytree
from ._dev import as_tensor
from .utils import FlashOptimizer


def global_sq_norm(grads: Any):
    """One-element float64 CUDA tensor with the sum of squares of every leaf of `grads`."""
    return eng.sq_norm_of([as_tensor(g) for g in pytree.tree_leaves(grads)])


def clip_by_global_norm(tx: FlashOptimizer, max_norm: float) -> FlashOptimizer:
    """`tx` with global-norm clipping of the gradients at `max_norm`; state is {"clip": (), "opt": tx's state}
    (the empty clip state is what optax's transformation carries)."""
    max_norm = float(max_norm)

    def init_fn(params: Any):
        return {"clip": (), "opt": tx.init(params)}

    def step_fn(params: Any, state: Any, grads: Any):
        sq = global_sq_norm(grads)
        with eng.grad_clip(sq, max_norm):
            params, opt_state = tx.step(params, state["opt"], grads)
        return params, {"clip": (), "opt": opt_state}

    return FlashOptimizer(init=init_fn, step=step_fn)
