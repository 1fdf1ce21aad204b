"""fp32 master weight <-> (16-bit parameter, ECC) on the GPU.

Mirrors flashoptim_jax/compression.py: a bf16/fp16 parameter plus an int8 (24-bit master)
or int16 (32-bit master) error-correction code reconstructs the fp32 weight to within
1/127 resp. 1/32767 of half an ULP of the stored value.  Leaves that cannot carry ECC
(fp32 parameters, master_weight_bits=None) get a 0-d int32 sentinel instead.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch

from . import _lib
from . import tree as pytree
from ._dev import DTYPE_CODE, ECC_BITS_OF, LOW_PRECISION, as_tensor, require_cuda, stream_ptr


def _validate_master_weight_bits(master_weight_bits: Optional[int]) -> None:
    if master_weight_bits not in (None, 24, 32):
        raise ValueError(f"master_weight_bits must be one of (None, 24, 32), got {master_weight_bits}")


def no_ecc_leaf(device=None) -> torch.Tensor:
    """0-d int32 zero: the marker of "no ECC buffer" (flashoptim_jax/utils.py:94-96)."""
    return torch.zeros((), dtype=torch.int32, device=device)


def cast_tree_bf16(tree: Any) -> Any:
    """Cast every leaf of a pytree to bfloat16 (flashoptim_jax/compression.py:35-37)."""
    return pytree.tree_map(lambda x: as_tensor(x).to(torch.bfloat16), tree)


def _ecc_dtype_for(narrow_dtype: torch.dtype, master_weight_bits: Optional[int]) -> Optional[torch.dtype]:
    """ECC dtype implied by the stored dtype and the master width (flashoptim_jax/compression.py:39-54)."""
    _validate_master_weight_bits(master_weight_bits)
    if master_weight_bits is None or narrow_dtype not in LOW_PRECISION:
        return None
    extra_bytes = master_weight_bits // 8 - 2
    if extra_bytes <= 0:
        return None
    return torch.int8 if extra_bytes == 1 else torch.int16


def has_ecc(theta_lp: torch.Tensor, rho: torch.Tensor) -> bool:
    """Whether (param, ecc) is a real low-precision/ECC pair (flashoptim_jax/compression.py:77-81)."""
    return as_tensor(theta_lp).dtype in LOW_PRECISION and as_tensor(rho).dtype in ECC_BITS_OF


def split_leaf(theta, narrow_dtype: torch.dtype = torch.bfloat16, master_weight_bits: Optional[int] = 24) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 leaf -> (stored param, ECC or sentinel) (flashoptim_jax/compression.py:84-104)."""
    theta = as_tensor(theta)
    require_cuda(theta, "theta")
    theta32 = theta.to(torch.float32).contiguous()
    ecc_dtype = _ecc_dtype_for(narrow_dtype, master_weight_bits)
    if narrow_dtype not in LOW_PRECISION:
        return theta32.to(narrow_dtype), no_ecc_leaf(theta.device)
    lp = torch.empty(theta.shape, dtype=narrow_dtype, device=theta.device)
    ecc = None if ecc_dtype is None else torch.empty(theta.shape, dtype=ecc_dtype, device=theta.device)
    with torch.cuda.device(theta.device):
        _lib.check(_lib.lib().fo_split(
            theta32.data_ptr(), lp.data_ptr(), 0 if ecc is None else ecc.data_ptr(),
            DTYPE_CODE[narrow_dtype], 0 if ecc is None else ECC_BITS_OF[ecc_dtype], theta32.numel(), stream_ptr(theta.device)))
    return lp, (no_ecc_leaf(theta.device) if ecc is None else ecc)


def reconstruct_leaf(theta_lp, rho) -> torch.Tensor:
    """(stored param, ECC) -> fp32 (flashoptim_jax/compression.py:107-121)."""
    theta_lp = as_tensor(theta_lp)
    rho = as_tensor(rho)
    if not has_ecc(theta_lp, rho):
        return theta_lp.to(torch.float32)
    require_cuda(theta_lp, "theta_lp")
    lp = theta_lp.contiguous()
    ecc = rho.contiguous()
    out = torch.empty(lp.shape, dtype=torch.float32, device=lp.device)
    with torch.cuda.device(lp.device):
        _lib.check(_lib.lib().fo_reconstruct(
            lp.data_ptr(), ecc.data_ptr(), out.data_ptr(), DTYPE_CODE[lp.dtype], ECC_BITS_OF[ecc.dtype], lp.numel(), stream_ptr(lp.device)))
    return out


def reconstruct_weights(params_lp: Any, errors: Any) -> Any:
    """fp32 weights of a whole pytree (flashoptim_jax/compression.py:124-126)."""
    return pytree.tree_map(reconstruct_leaf, params_lp, errors)


def set_fp32_params(fp32_params: Any, param_template: Any, master_weight_bits: Optional[int] = 24) -> Tuple[Any, Any]:
    """fp32 weights -> (stored params, ECC tree) with the template's dtypes (flashoptim_jax/compression.py:129-146)."""
    leaves, treedef = pytree.tree_flatten(fp32_params)
    template_leaves, template_def = pytree.tree_flatten(param_template)
    if treedef != template_def:
        raise ValueError("fp32_params and param_template must have matching tree structure")
    pairs = [split_leaf(leaf, narrow_dtype=as_tensor(t).dtype, master_weight_bits=master_weight_bits)
             for leaf, t in zip(leaves, template_leaves)]
    return treedef.unflatten([p for p, _ in pairs]), treedef.unflatten([e for _, e in pairs])
