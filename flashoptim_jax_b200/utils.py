"""Host-side pieces shared by the optimizers: the FlashOptimizer pair, param-group
resolution, argument validation with the reference's error messages, the "no buffer"
sentinels and state-dict (de)serialisation.

Behaviour follows flashoptim_jax/utils.py; line references are given per function.
"""

from __future__ import annotations

from collections.abc import Iterable
from typing import Any, Callable, Dict, List, NamedTuple, Optional, Tuple

import torch

from . import tree as pytree
from ._dev import FUSED_PARAM_DTYPES, LOW_PRECISION, as_tensor, dtype_name
from .quantization import QuantizedArray

BLOCK_SIZE = 1024  # tile of the reference's fused kernels; group_size must divide it when fused (utils.py:19,165-171)
GROUP_SIZE = 32
MAX_GROUP_SIZE = 1024  # largest group the CUDA kernels handle

ParamGroupSpec = Dict[str, Any]


class FlashOptimizer(NamedTuple):
    """`init(params) -> state` and `step(params, state, grads) -> (params, state)` (utils.py:70-73)."""

    init: Callable[[Any], Any]
    step: Callable[[Any, Any, Any], Tuple[Any, Any]]


def _is_quantized_leaf(x: Any) -> bool:
    return isinstance(x, QuantizedArray)


def no_ecc_leaf(device=None) -> torch.Tensor:
    return torch.zeros((), dtype=torch.int32, device=device)


def no_state_leaf(device=None) -> torch.Tensor:
    """0-d int32 zero marking an absent optimizer-state slot (utils.py:99-101)."""
    return torch.zeros((), dtype=torch.int32, device=device)


def _has_state_leaf(x: Any) -> bool:
    """False for the 0-d int32 sentinel, True for real state (utils.py:104-109)."""
    if _is_quantized_leaf(x):
        return True
    t = as_tensor(x)
    return not (t.dim() == 0 and t.dtype == torch.int32)


# ---- param groups (utils.py:112-154) -------------------------------------------------------


def _selector_matches(path: Tuple[Any, ...], leaf: Any, selector: Any) -> bool:
    if callable(selector):
        return bool(selector(path, leaf))
    if isinstance(selector, tuple):
        return path == selector
    if isinstance(selector, str):
        segments = [str(entry) for entry in path]
        return "/".join(segments) == selector if "/" in selector else selector in segments
    return False


def _path_matches(path: Tuple[Any, ...], leaf: Any, spec: Any) -> bool:
    if isinstance(spec, Iterable) and not isinstance(spec, (str, bytes, tuple)):
        return any(_selector_matches(path, leaf, s) for s in spec)
    return _selector_matches(path, leaf, spec)


def _group_config_for_path(path, leaf, defaults: Dict[str, Any], param_groups: Optional[List[ParamGroupSpec]]) -> Dict[str, Any]:
    """Defaults overridden by the first param group whose matcher accepts the leaf."""
    config = dict(defaults)
    for group in param_groups or ():
        if "params" not in group:
            raise ValueError("Each param group must define a 'params' matcher")
        if _path_matches(path, leaf, group["params"]):
            config.update({k: v for k, v in group.items() if k != "params"})
            break
    return config


class GroupResolver:
    """_group_config_for_path for all leaves of one step: the merged config of a group is built once and the same
    dict is handed to each of its leaves, so that per-group work (hyper-parameter tuples) can be keyed on it."""

    def __init__(self, defaults: Dict[str, Any], param_groups: Optional[List[ParamGroupSpec]]):
        self.defaults, self.groups = defaults, list(param_groups or ())
        for group in self.groups:
            if "params" not in group:
                raise ValueError("Each param group must define a 'params' matcher")
        self._configs: Dict[int, Dict[str, Any]] = {}

    def __call__(self, path, leaf) -> Dict[str, Any]:
        index = -1
        for i, group in enumerate(self.groups):
            if _path_matches(path, leaf, group["params"]):
                index = i
                break
        config = self._configs.get(index)
        if config is None:
            config = dict(self.defaults)
            if index >= 0:
                config.update({k: v for k, v in self.groups[index].items() if k != "params"})
            self._configs[index] = config
        return config


# ---- validation (utils.py:157-266) ----------------------------------------------------------


def _validate_master_weight_bits(master_weight_bits: Optional[int]) -> None:
    if master_weight_bits not in (None, 24, 32):
        raise ValueError(f"master_weight_bits must be one of (None, 24, 32), got {master_weight_bits}")


def _validate_fused_group_size(group_size: int, *, quantize: bool, fused: bool) -> None:
    if fused and quantize and BLOCK_SIZE % group_size != 0:
        raise ValueError(
            f"group_size must divide BLOCK_SIZE ({BLOCK_SIZE}) when fused=True "
            f"and quantize=True, got group_size={group_size}"
        )
    if quantize and not (1 <= group_size <= MAX_GROUP_SIZE):
        raise ValueError(f"group_size must lie in [1, {MAX_GROUP_SIZE}] for the CUDA kernels, got group_size={group_size}")


def _use_ecc_leaf(param: Any, master_weight_bits: Optional[int]) -> bool:
    if master_weight_bits is None:
        return False
    dt = as_tensor(param).dtype
    return dt in LOW_PRECISION and master_weight_bits > 16


def _path_str(path: Tuple[Any, ...]) -> str:
    return "/".join(str(entry) for entry in path) or "<root>"


def _validate_param_dtypes(params: Any, defaults, param_groups, name: str) -> None:
    """Every leaf must be fp32 / bf16 / fp16: the only dtypes the kernels exist for.

    The reference raises this for fused leaves only (utils.py:184-203) and lets its jnp
    path take any float dtype; here both settings of `fused` run the same CUDA kernels.
    """
    supported = ", ".join(dtype_name(dt) for dt in FUSED_PARAM_DTYPES)
    for path, leaf in _tree_leaves_with_paths(params)[0]:
        config = _group_config_for_path(path, leaf, defaults, param_groups)
        dt = as_tensor(leaf).dtype
        if dt not in FUSED_PARAM_DTYPES:
            fused_txt = "fused=True" if config["fused"] else "fused=False (CUDA build)"
            raise ValueError(
                f"{name} {fused_txt} only supports parameter dtypes ({supported}), "
                f"got {dtype_name(dt)} for parameter '{_path_str(path)}'"
            )


def _validate_meaningful_master_weight_bits(params: Any, defaults, param_groups, name: str) -> None:
    """Reject a master_weight_bits that no matched leaf can use (utils.py:206-266)."""
    path_leaves = _tree_leaves_with_paths(params)[0]
    if not path_leaves:
        return
    groups = list(param_groups or [])
    for group in groups:
        if "params" not in group:
            raise ValueError("Each param group must define a 'params' matcher")
    matched = [False] * len(groups)
    meaningful = [False] * len(groups)
    defaults_matched = defaults_meaningful = False
    default_bits = defaults["master_weight_bits"]
    for path, leaf in path_leaves:
        hit = next((i for i, g in enumerate(groups) if _path_matches(path, leaf, g["params"])), None)
        if hit is not None and "master_weight_bits" in groups[hit]:
            matched[hit] = True
            bits = groups[hit]["master_weight_bits"]
            if bits is not None and _use_ecc_leaf(leaf, bits):
                meaningful[hit] = True
            continue
        defaults_matched = True
        if default_bits is not None and _use_ecc_leaf(leaf, default_bits):
            defaults_meaningful = True
    if defaults_matched and default_bits is not None and not defaults_meaningful:
        raise ValueError(
            f"{name} master_weight_bits={default_bits} has no effect because "
            "all matched parameters are already fp32 or otherwise ineligible for ECC"
        )
    for i, group in enumerate(groups):
        bits = group.get("master_weight_bits")
        if matched[i] and bits is not None and not meaningful[i]:
            raise ValueError(
                f"{name} param_groups[{i}]['master_weight_bits']={bits} has no effect because all matched "
                "parameters are already fp32 or otherwise ineligible for ECC"
            )


def _tree_leaves_with_paths(tree: Any, is_leaf=None):
    """[(path, leaf)], treedef — paths as tuples of keys/indices/field names (utils.py:269-274)."""
    return pytree.tree_flatten_with_path(tree, is_leaf=is_leaf)


def _resolve_learning_rate(learning_rate, count: torch.Tensor) -> float:
    """Value of a constant or of schedule(count), count being the zero-based step (utils.py:277-284)."""
    if callable(learning_rate):
        learning_rate = learning_rate(count)
    if isinstance(learning_rate, torch.Tensor):
        return float(learning_rate.to(torch.float32))
    try:
        return float(learning_rate)
    except TypeError:
        import numpy as np

        return float(np.asarray(learning_rate, dtype=np.float32))


# ---- state-dict (utils.py:377-413) -----------------------------------------------------------


def _serialize_state_leaf(leaf: Any) -> Dict[str, Any]:
    if isinstance(leaf, QuantizedArray):
        return {"kind": "quantized", "values": as_tensor(leaf.values), "scales": as_tensor(leaf.scales)}
    return {"kind": "array", "value": as_tensor(leaf)}


def _deserialize_state_leaf(leaf: Dict[str, Any]) -> Any:
    kind = leaf["kind"]
    if kind == "quantized":
        return QuantizedArray(values=as_tensor(leaf["values"]), scales=as_tensor(leaf["scales"]))
    if kind == "array":
        return as_tensor(leaf["value"])
    raise ValueError(f"Unsupported serialized state leaf kind: {kind}")


def _tree_state_dict(tree: Any) -> Dict[str, Any]:
    leaves, treedef = pytree.tree_flatten(tree, is_leaf=_is_quantized_leaf)
    return {"treedef": treedef, "leaves": [_serialize_state_leaf(leaf) for leaf in leaves]}


def _tree_from_state_dict(state_dict: Dict[str, Any]) -> Any:
    return state_dict["treedef"].unflatten([_deserialize_state_leaf(leaf) for leaf in state_dict["leaves"]])
