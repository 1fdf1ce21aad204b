"""flash_adam / flash_adamw: the reference's API (flashoptim_jax/adamw.py:544-654) over the
CUDA multi-tensor step.

`fused` keeps its place in the signature.  Both settings run the same CUDA kernel; the
flag selects which of the reference's two texts the arithmetic follows bit for bit:
  fused=True   the Pallas kernel body (adamw.py:76-131): (1-beta) formed in fp32, group
               scale guard max(absmax, 1e-12), the new parameter stored directly;
  fused=False  the jnp path that runs on CPU (adamw.py:356-423, 463): (1-beta) formed in
               Python floats, guard where(absmax > 0, absmax, 1), parameter returned as
               param + lp(new - param).
`donate=True` (not in the reference, where donation is a jax.jit argument) lets step()
overwrite the tensors it is given, which is how the kernel is meant to run; without it
step() copies params and state first so the inputs stay untouched.
"""

from __future__ import annotations

from typing import Any, Dict, List, NamedTuple, Optional

import torch

from . import _engine as eng
from . import _lib
from . import utils
from ._dev import as_tensor


class FlashAdamState(NamedTuple):
    count: torch.Tensor
    mu: Any
    nu: Any
    ecc: Any


def adam_hyper(config: Dict[str, Any], lr: float, count: int, decoupled_weight_decay: bool):
    """The 0-d operands of the Adam kernel for one param group at step `count` (adamw.py:526-528)."""
    is_fused = bool(config["fused"])
    flags = (_lib.FO_FLAG_DECOUPLED_WD if decoupled_weight_decay else 0)
    flags |= _lib.FO_FLAG_SCALE_FLOOR if is_fused else _lib.FO_FLAG_LP_DELTA
    return (
        eng.F32(lr), eng.F32(config["weight_decay"]), eng.F32(config["b1"]), eng.F32(config["b2"]),
        eng.one_minus(config["b1"], is_fused), eng.one_minus(config["b2"], is_fused), eng.F32(config["eps"]),
        eng.bias_correction(config["b1"], count), eng.bias_correction(config["b2"], count), flags,
    )


def _make_adam_transform(learning_rate, b1, b2, eps, weight_decay, quantize, master_weight_bits, group_size, fused,
                         decoupled_weight_decay, param_groups, name, donate, capturable=False) -> utils.FlashOptimizer:
    utils._validate_master_weight_bits(master_weight_bits)
    utils._validate_fused_group_size(group_size, quantize=quantize, fused=fused)
    defaults = {
        "learning_rate": learning_rate, "b1": b1, "b2": b2, "eps": eps, "weight_decay": weight_decay,
        "quantize": quantize, "master_weight_bits": master_weight_bits, "group_size": group_size, "fused": fused,
    }

    def init_fn(params: Any) -> FlashAdamState:
        entries, treedef = eng.init_common(params, defaults, param_groups, name)
        mus, nus, eccs = [], [], []
        for _, leaf, config in entries:
            mus.append(eng.init_moment(leaf, config["group_size"], config["quantize"], torch.int8))
            nus.append(eng.init_moment(leaf, config["group_size"], config["quantize"], torch.uint8))
            eccs.append(eng.init_ecc(leaf, config["master_weight_bits"]))
        return FlashAdamState(count=torch.zeros((), dtype=torch.int32), mu=treedef.unflatten(mus),
                              nu=treedef.unflatten(nus), ecc=treedef.unflatten(eccs))

    def capturable_step_fn(params: Any, state: FlashAdamState, grads: Any):
        """The same step with no host scalar in it: the counter stays on the device, and the learning rate
        (a number or a 0-d CUDA tensor the caller updates), count + 1 and the bias corrections (adamw.py:510,
        526-528) are formed there by fo_step_scalars, so the call can be captured in a CUDA graph and replayed."""
        param_pl, grad_leaves, (ecc_leaves, mu_leaves, nu_leaves), treedef = eng.flatten_step_inputs(
            name, params, grads, [state.ecc, state.mu, state.nu])
        leaves = [as_tensor(leaf) for _, leaf in param_pl]
        configs = [utils._group_config_for_path(path, leaf, defaults, param_groups) for (path, _), leaf in zip(param_pl, leaves)]
        count, pointers, _alive = eng.device_step_scalars(state.count, leaves, configs)
        work: List[eng.LeafWork] = []
        new_p, new_e, new_m, new_v = [], [], [], []
        for leaf, ptr, config, g, e, m, v in zip(leaves, pointers, configs, grad_leaves, ecc_leaves, mu_leaves, nu_leaves):
            hyper = adam_hyper(config, 0.0, 1, decoupled_weight_decay) + (ptr,)  # lr, bc1, bc2 come from the device
            w, p_out, e_out, m_out, v_out = eng.make_work(leaf, g, e, m, v, config, hyper, donate, has_nu=True)
            work.append(w)
            new_p.append(p_out); new_e.append(e_out); new_m.append(m_out); new_v.append(v_out)
        eng.launch(_lib.FO_OPT_ADAM, work)
        new_state = FlashAdamState(count=count, mu=treedef.unflatten(new_m), nu=treedef.unflatten(new_v), ecc=treedef.unflatten(new_e))
        return treedef.unflatten(new_p), new_state

    cache = eng.DonatedStepCache()

    def step_fn(params: Any, state: FlashAdamState, grads: Any):
        old_count = as_tensor(state.count, dtype=torch.int32).cpu()
        count = int(old_count) + 1  # adamw.py:510
        if donate:
            hit = cache.replay(params, [state.ecc, state.mu, state.nu], grads, lambda config: adam_hyper(
                config, utils._resolve_learning_rate(config["learning_rate"], old_count), count, decoupled_weight_decay))
            if hit is not None:
                ecc_t, mu_t, nu_t = hit[1]
                return hit[0], FlashAdamState(count=torch.tensor(count, dtype=torch.int32), mu=mu_t, nu=nu_t, ecc=ecc_t)
        configs: List[Dict[str, Any]] = []
        param_pl, grad_leaves, (ecc_leaves, mu_leaves, nu_leaves), treedef = eng.flatten_step_inputs(
            name, params, grads, [state.ecc, state.mu, state.nu])
        work: List[eng.LeafWork] = []
        new_p, new_e, new_m, new_v = [], [], [], []
        resolve, hypers = utils.GroupResolver(defaults, param_groups), {}
        for (path, leaf), g, e, m, v in zip(param_pl, grad_leaves, ecc_leaves, mu_leaves, nu_leaves):
            leaf = as_tensor(leaf)
            config = resolve(path, leaf)
            hyper = hypers.get(id(config))
            if hyper is None:  # once per param group
                lr = utils._resolve_learning_rate(config["learning_rate"], old_count)  # zero-based count (adamw.py:526)
                hyper = hypers[id(config)] = adam_hyper(config, lr, count, decoupled_weight_decay)
            w, p_out, e_out, m_out, v_out = eng.make_work(leaf, g, e, m, v, config, hyper, donate, has_nu=True)
            work.append(w)
            configs.append(config)
            new_p.append(p_out); new_e.append(e_out); new_m.append(m_out); new_v.append(v_out)
        eng.launch(_lib.FO_OPT_ADAM, work)
        new_state = FlashAdamState(count=torch.tensor(count, dtype=torch.int32), mu=treedef.unflatten(new_m),
                                   nu=treedef.unflatten(new_v), ecc=treedef.unflatten(new_e))
        new_params = treedef.unflatten(new_p)
        if donate:
            cache.remember(_lib.FO_OPT_ADAM, work, configs, new_params, [new_state.ecc, new_state.mu, new_state.nu])
        return new_params, new_state

    return utils.FlashOptimizer(init=init_fn, step=capturable_step_fn if capturable else step_fn)


def flash_adam(learning_rate=1e-3, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
               quantize: bool = True, master_weight_bits: Optional[int] = 24, group_size: int = 32, fused: bool = True,
               param_groups: Optional[List[Dict[str, Any]]] = None, donate: bool = False,
               capturable: bool = False) -> utils.FlashOptimizer:
    """Adam with weight decay added to the gradient (flashoptim_jax/adamw.py:595-613)."""
    return _make_adam_transform(learning_rate, b1, b2, eps, weight_decay, quantize, master_weight_bits, group_size, fused,
                                False, param_groups, "flash_adam", donate, capturable)


def flash_adamw(learning_rate=1e-3, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, weight_decay: float = 1e-2,
                quantize: bool = True, master_weight_bits: Optional[int] = 24, group_size: int = 32, fused: bool = True,
                param_groups: Optional[List[Dict[str, Any]]] = None, donate: bool = False,
                capturable: bool = False) -> utils.FlashOptimizer:
    """AdamW, decoupled weight decay (flashoptim_jax/adamw.py:616-634)."""
    return _make_adam_transform(learning_rate, b1, b2, eps, weight_decay, quantize, master_weight_bits, group_size, fused,
                                True, param_groups, "flash_adamw", donate, capturable)


def flash_adamw_state_dict(state: FlashAdamState) -> Dict[str, Any]:
    """Checkpointable form of the state (flashoptim_jax/adamw.py:639-644)."""
    return {"count": as_tensor(state.count), "mu": utils._tree_state_dict(state.mu),
            "nu": utils._tree_state_dict(state.nu), "ecc": utils._tree_state_dict(state.ecc)}


def load_flash_adamw_state_dict(state_dict: Dict[str, Any]) -> FlashAdamState:
    """Inverse of flash_adamw_state_dict (flashoptim_jax/adamw.py:647-654)."""
    return FlashAdamState(count=as_tensor(state_dict["count"], dtype=torch.int32),
                          mu=utils._tree_from_state_dict(state_dict["mu"]),
                          nu=utils._tree_from_state_dict(state_dict["nu"]),
                          ecc=utils._tree_from_state_dict(state_dict["ecc"]))
