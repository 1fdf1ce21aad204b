"""flash_lion: the reference's API (flashoptim_jax/lion.py:192-249) over the CUDA step.

`fused=True` follows the kernel text b*mu + (1-b)*g with (1-b) formed in fp32
(momentum_kernel.py:77-79); `fused=False` follows the jnp text mu + (1-b)*(g - mu) with
(1-b) formed in Python floats (lion.py:50-52).  Both run the same CUDA kernel.
"""

from __future__ import annotations

from typing import Any, Dict, List, NamedTuple, Optional

import torch

from . import _engine as eng
from . import _lib
from . import utils
from ._dev import as_tensor


class FlashLionState(NamedTuple):
    count: torch.Tensor
    mu: Any
    ecc: Any


def lion_hyper(config: Dict[str, Any], lr: float):
    """The 0-d operands of the momentum kernel in Lion mode for one param group (lion.py:92-104)."""
    is_fused = bool(config["fused"])
    flags = _lib.FO_FLAG_DECOUPLED_WD | (_lib.FO_FLAG_SCALE_FLOOR if is_fused else _lib.FO_FLAG_LION_LERP)
    return (
        eng.F32(lr), eng.F32(config["weight_decay"]), eng.F32(config["b1"]), eng.F32(config["b2"]),
        eng.one_minus(config["b1"], is_fused), eng.one_minus(config["b2"], is_fused),
        eng.F32(0.0), eng.F32(1.0), eng.F32(1.0), flags,
    )


def flash_lion(learning_rate=1e-4, b1: float = 0.9, b2: float = 0.99, weight_decay: float = 0.0, quantize: bool = True,
               master_weight_bits: Optional[int] = 24, group_size: int = 32, fused: bool = True,
               param_groups: Optional[List[Dict[str, Any]]] = None, donate: bool = False,
               capturable: bool = False) -> utils.FlashOptimizer:
    name = "flash_lion"
    utils._validate_master_weight_bits(master_weight_bits)
    utils._validate_fused_group_size(group_size, quantize=quantize, fused=fused)
    defaults = {
        "learning_rate": learning_rate, "b1": b1, "b2": b2, "weight_decay": weight_decay, "quantize": quantize,
        "master_weight_bits": master_weight_bits, "group_size": group_size, "fused": fused,
    }

    def init_fn(params: Any) -> FlashLionState:
        entries, treedef = eng.init_common(params, defaults, param_groups, name)
        mus = [eng.init_moment(leaf, c["group_size"], c["quantize"], torch.int8) for _, leaf, c in entries]
        eccs = [eng.init_ecc(leaf, c["master_weight_bits"]) for _, leaf, c in entries]
        return FlashLionState(count=torch.zeros((), dtype=torch.int32), mu=treedef.unflatten(mus), ecc=treedef.unflatten(eccs))

    def capturable_step_fn(params: Any, state: FlashLionState, grads: Any):
        """The same step with no host scalar in it (counter and learning rate stay on the device, see
        flash_adamw(capturable=True)): capturable in a CUDA graph."""
        param_pl, grad_leaves, (ecc_leaves, mu_leaves), treedef = eng.flatten_step_inputs(
            name, params, grads, [state.ecc, state.mu])
        leaves = [as_tensor(leaf) for _, leaf in param_pl]
        configs = [utils._group_config_for_path(path, leaf, defaults, param_groups) for (path, _), leaf in zip(param_pl, leaves)]
        count, pointers, _alive = eng.device_step_scalars(state.count, leaves, configs)
        work, new_p, new_e, new_m = [], [], [], []
        for leaf, ptr, config, g, e, m in zip(leaves, pointers, configs, grad_leaves, ecc_leaves, mu_leaves):
            w, p_out, e_out, m_out, _ = eng.make_work(leaf, g, e, m, None, config, lion_hyper(config, 0.0) + (ptr,), donate, has_nu=False)
            work.append(w)
            new_p.append(p_out); new_e.append(e_out); new_m.append(m_out)
        eng.launch(_lib.FO_OPT_LION, work)
        return treedef.unflatten(new_p), FlashLionState(count=count, mu=treedef.unflatten(new_m), ecc=treedef.unflatten(new_e))

    cache = eng.DonatedStepCache()

    def step_fn(params: Any, state: FlashLionState, grads: Any):
        old_count = as_tensor(state.count, dtype=torch.int32).cpu()
        if donate:
            hit = cache.replay(params, [state.ecc, state.mu], grads, lambda config: lion_hyper(
                config, utils._resolve_learning_rate(config["learning_rate"], old_count)))
            if hit is not None:
                ecc_t, mu_t = hit[1]
                return hit[0], FlashLionState(count=torch.tensor(int(old_count) + 1, dtype=torch.int32), mu=mu_t, ecc=ecc_t)
        configs = []
        param_pl, grad_leaves, (ecc_leaves, mu_leaves), treedef = eng.flatten_step_inputs(
            name, params, grads, [state.ecc, state.mu])
        work, new_p, new_e, new_m = [], [], [], []
        resolve, hypers = utils.GroupResolver(defaults, param_groups), {}
        for (path, leaf), g, e, m in zip(param_pl, grad_leaves, ecc_leaves, mu_leaves):
            leaf = as_tensor(leaf)
            config = resolve(path, leaf)
            hyper = hypers.get(id(config))
            if hyper is None:  # once per param group
                hyper = hypers[id(config)] = lion_hyper(config, utils._resolve_learning_rate(config["learning_rate"], old_count))
            w, p_out, e_out, m_out, _ = eng.make_work(leaf, g, e, m, None, config, hyper, donate, has_nu=False)
            work.append(w)
            configs.append(config)
            new_p.append(p_out); new_e.append(e_out); new_m.append(m_out)
        eng.launch(_lib.FO_OPT_LION, work)
        new_state = FlashLionState(count=torch.tensor(int(old_count) + 1, dtype=torch.int32),
                                   mu=treedef.unflatten(new_m), ecc=treedef.unflatten(new_e))
        new_params = treedef.unflatten(new_p)
        if donate:
            cache.remember(_lib.FO_OPT_LION, work, configs, new_params, [new_state.ecc, new_state.mu])
        return new_params, new_state

    return utils.FlashOptimizer(init=init_fn, step=capturable_step_fn if capturable else step_fn)


def flash_lion_state_dict(state: FlashLionState) -> Dict[str, Any]:
    """flashoptim_jax/lion.py:234-240."""
    return {"count": as_tensor(state.count), "mu": utils._tree_state_dict(state.mu), "ecc": utils._tree_state_dict(state.ecc)}


def load_flash_lion_state_dict(state_dict: Dict[str, Any]) -> FlashLionState:
    """flashoptim_jax/lion.py:243-249."""
    return FlashLionState(count=as_tensor(state_dict["count"], dtype=torch.int32),
                          mu=utils._tree_from_state_dict(state_dict["mu"]),
                          ecc=utils._tree_from_state_dict(state_dict["ecc"]))
