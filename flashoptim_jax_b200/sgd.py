"""flash_sgd / flash_sgdw: the reference's API (flashoptim_jax/sgd.py:221-329) over the CUDA step.

momentum, dampening, nesterov and coupled (flash_sgd) or decoupled (flash_sgdw) weight
decay as in the reference.  momentum == 0 keeps no buffer: the state holds the 0-d int32
sentinel and a buffer-less kernel variant runs (the reference falls back to its jnp path
there, sgd.py:99-101).  The two reference texts agree on the SGD arithmetic; `fused` only
selects the group-scale guard (momentum_kernel.py:98 vs quantization.py:41).
"""

from __future__ import annotations

from typing import Any, Dict, List, NamedTuple, Optional

import torch

from . import _engine as eng
from . import _lib
from . import utils
from ._dev import as_tensor


class FlashSGDState(NamedTuple):
    count: torch.Tensor
    mu: Any
    ecc: Any


def _validate_sgd_hparams(momentum: float, dampening: float, nesterov: bool) -> None:
    """flashoptim_jax/sgd.py:130-133."""
    if nesterov and (momentum <= 0.0 or dampening != 0.0):
        raise ValueError("Nesterov momentum requires positive momentum and zero dampening")


def sgd_hyper(config: Dict[str, Any], lr: float, decoupled_weight_decay: bool):
    """The 0-d operands of the momentum kernel in SGD mode for one param group (sgd.py:102-116)."""
    flags = (_lib.FO_FLAG_DECOUPLED_WD if decoupled_weight_decay else 0)
    flags |= _lib.FO_FLAG_NESTEROV if config["nesterov"] else 0
    flags |= _lib.FO_FLAG_SCALE_FLOOR if config["fused"] else 0
    return (
        eng.F32(lr), eng.F32(config["weight_decay"]), eng.F32(config["momentum"]), eng.F32(0.0),
        eng.F32(1.0 - float(config["dampening"])), eng.F32(0.0), eng.F32(0.0), eng.F32(1.0), eng.F32(1.0), flags,
    )


def _make_sgd_transform(learning_rate, momentum, dampening, weight_decay, nesterov, quantize, master_weight_bits,
                        group_size, fused, decoupled_weight_decay, param_groups, name, donate, capturable=False) -> utils.FlashOptimizer:
    utils._validate_master_weight_bits(master_weight_bits)
    utils._validate_fused_group_size(group_size, quantize=quantize, fused=fused)
    _validate_sgd_hparams(momentum, dampening, nesterov)
    defaults = {
        "learning_rate": learning_rate, "momentum": momentum, "dampening": dampening, "weight_decay": weight_decay,
        "nesterov": nesterov, "quantize": quantize, "master_weight_bits": master_weight_bits, "group_size": group_size,
        "fused": fused,
    }

    def init_fn(params: Any) -> FlashSGDState:
        entries, treedef = eng.init_common(
            params, defaults, param_groups, name,
            per_leaf_check=lambda c: _validate_sgd_hparams(c["momentum"], c["dampening"], c["nesterov"]))
        mus, eccs = [], []
        for _, leaf, c in entries:
            if c["momentum"] > 0.0:
                mus.append(eng.init_moment(leaf, c["group_size"], c["quantize"], torch.int8))
            else:
                mus.append(utils.no_state_leaf(leaf.device))
            eccs.append(eng.init_ecc(leaf, c["master_weight_bits"]))
        return FlashSGDState(count=torch.zeros((), dtype=torch.int32), mu=treedef.unflatten(mus), ecc=treedef.unflatten(eccs))

    def capturable_step_fn(params: Any, state: FlashSGDState, grads: Any):
        """The same step with no host scalar in it (counter and learning rate stay on the device, see
        flash_adamw(capturable=True)): capturable in a CUDA graph."""
        param_pl, grad_leaves, (ecc_leaves, mu_leaves), treedef = eng.flatten_step_inputs(
            name, params, grads, [state.ecc, state.mu])
        leaves = [as_tensor(leaf) for _, leaf in param_pl]
        configs = [utils._group_config_for_path(path, leaf, defaults, param_groups) for (path, _), leaf in zip(param_pl, leaves)]
        count, pointers, _alive = eng.device_step_scalars(state.count, leaves, configs)
        work, new_p, new_e, new_m = [], [], [], []
        for leaf, ptr, config, g, e, m in zip(leaves, pointers, configs, grad_leaves, ecc_leaves, mu_leaves):
            use_momentum = config["momentum"] > 0.0
            if use_momentum and not utils._has_state_leaf(m):
                raise ValueError(f"{name}: momentum > 0 needs a momentum buffer in the state; re-run init()")
            hyper = sgd_hyper(config, 0.0, decoupled_weight_decay) + (ptr,)
            w, p_out, e_out, m_out, _ = eng.make_work(leaf, g, e, m, None, config, hyper, donate, has_nu=False,
                                                      use_momentum=use_momentum)
            work.append(w)
            new_p.append(p_out); new_e.append(e_out); new_m.append(m_out)
        eng.launch(_lib.FO_OPT_SGD, work)
        return treedef.unflatten(new_p), FlashSGDState(count=count, mu=treedef.unflatten(new_m), ecc=treedef.unflatten(new_e))

    cache = eng.DonatedStepCache()

    def step_fn(params: Any, state: FlashSGDState, grads: Any):
        old_count = as_tensor(state.count, dtype=torch.int32).cpu()
        if donate:
            hit = cache.replay(params, [state.ecc, state.mu], grads, lambda config: sgd_hyper(
                config, utils._resolve_learning_rate(config["learning_rate"], old_count), decoupled_weight_decay))
            if hit is not None:
                ecc_t, mu_t = hit[1]
                return hit[0], FlashSGDState(count=torch.tensor(int(old_count) + 1, dtype=torch.int32), mu=mu_t, ecc=ecc_t)
        configs = []
        param_pl, grad_leaves, (ecc_leaves, mu_leaves), treedef = eng.flatten_step_inputs(
            name, params, grads, [state.ecc, state.mu])
        work, new_p, new_e, new_m = [], [], [], []
        resolve, hypers = utils.GroupResolver(defaults, param_groups), {}
        for (path, leaf), g, e, m in zip(param_pl, grad_leaves, ecc_leaves, mu_leaves):
            leaf = as_tensor(leaf)
            config = resolve(path, leaf)
            use_momentum = config["momentum"] > 0.0
            if use_momentum and not utils._has_state_leaf(m):
                raise ValueError(f"{name}: momentum > 0 needs a momentum buffer in the state; re-run init()")
            hyper = hypers.get(id(config))
            if hyper is None:  # once per param group
                hyper = hypers[id(config)] = sgd_hyper(config, utils._resolve_learning_rate(config["learning_rate"], old_count),
                                                       decoupled_weight_decay)
            w, p_out, e_out, m_out, _ = eng.make_work(leaf, g, e, m, None, config, hyper, donate, has_nu=False,
                                                      use_momentum=use_momentum)
            work.append(w)
            configs.append(config)
            new_p.append(p_out); new_e.append(e_out); new_m.append(m_out)
        eng.launch(_lib.FO_OPT_SGD, work)
        new_state = FlashSGDState(count=torch.tensor(int(old_count) + 1, dtype=torch.int32),
                                  mu=treedef.unflatten(new_m), ecc=treedef.unflatten(new_e))
        new_params = treedef.unflatten(new_p)
        if donate:
            cache.remember(_lib.FO_OPT_SGD, work, configs, new_params, [new_state.ecc, new_state.mu])
        return new_params, new_state

    return utils.FlashOptimizer(init=init_fn, step=capturable_step_fn if capturable else step_fn)


def flash_sgd(learning_rate=1e-3, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
              nesterov: bool = False, quantize: bool = True, master_weight_bits: Optional[int] = 24, group_size: int = 32,
              fused: bool = True, param_groups: Optional[List[Dict[str, Any]]] = None, donate: bool = False,
              capturable: bool = False) -> utils.FlashOptimizer:
    """SGD with weight decay added to the gradient (flashoptim_jax/sgd.py:267-287)."""
    return _make_sgd_transform(learning_rate, momentum, dampening, weight_decay, nesterov, quantize, master_weight_bits,
                               group_size, fused, False, param_groups, "flash_sgd", donate, capturable)


def flash_sgdw(learning_rate=1e-3, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
               nesterov: bool = False, quantize: bool = True, master_weight_bits: Optional[int] = 24, group_size: int = 32,
               fused: bool = True, param_groups: Optional[List[Dict[str, Any]]] = None, donate: bool = False,
              capturable: bool = False) -> utils.FlashOptimizer:
    """SGD with decoupled weight decay (flashoptim_jax/sgd.py:290-310)."""
    return _make_sgd_transform(learning_rate, momentum, dampening, weight_decay, nesterov, quantize, master_weight_bits,
                               group_size, fused, True, param_groups, "flash_sgdw", donate, capturable)


def flash_sgd_state_dict(state: FlashSGDState) -> Dict[str, Any]:
    """flashoptim_jax/sgd.py:314-320."""
    return {"count": as_tensor(state.count), "mu": utils._tree_state_dict(state.mu), "ecc": utils._tree_state_dict(state.ecc)}


def load_flash_sgd_state_dict(state_dict: Dict[str, Any]) -> FlashSGDState:
    """flashoptim_jax/sgd.py:323-329."""
    return FlashSGDState(count=as_tensor(state_dict["count"], dtype=torch.int32),
                         mu=utils._tree_from_state_dict(state_dict["mu"]),
                         ecc=utils._tree_from_state_dict(state_dict["ecc"]))
