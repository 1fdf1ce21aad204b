"""Shared test plumbing: the oracle drivers (oracle/driver.py) plus raw C-ABI calls on device tensors."""

from __future__ import annotations

import ctypes
from typing import List

from oracle import c_oracle as C  # noqa: F401
from oracle import flashoptim_oracle as O  # noqa: F401
from oracle.driver import (BF16, NP_OF_CODE, LeafArrays, assert_leaf_equal, bits, fresh_leaf, hyper_tuple, make_grad,  # noqa: F401
                           oracle_step, to_numpy, to_torch)


def abi_step(opt: int, grads: List, leaves: List[LeafArrays], state: int, group_size: int, hypers: List, hyper_of: List[int],
             param_dtype: int, grad_dtype: int, ecc_bits: int, stream: int = 0, expect_ok: bool = True,
             peer_param_offsets=None, peer_grad_offsets=None, grad_sq_norm=None, max_grad_norm: float = 0.0) -> int:
    """One fo_step call through the C ABI on torch device tensors (in place)."""
    from flashoptim_jax_b200 import _lib

    L = (_lib.FoLeaf * len(leaves))()
    for i, (g, lf) in enumerate(zip(grads, leaves)):
        L[i].grad = g.data_ptr()
        L[i].param = lf.param.data_ptr()
        for name in ("ecc", "mu", "mu_scales", "nu", "nu_scales"):
            t = getattr(lf, name)
            setattr(L[i], name, None if t is None else t.data_ptr())
        L[i].n = lf.param.numel()
        L[i].hyper = hyper_of[i]
    H = (_lib.FoHyper * len(hypers))()
    for i, hp in enumerate(hypers):
        for k, name in enumerate(("lr", "wd", "b1", "b2", "one_minus_b1", "one_minus_b2", "eps", "bc1", "bc2")):
            setattr(H[i], name, float(hp[k]))
        H[i].flags = int(hp[9])
        H[i].dev_scalars = hp[10] if len(hp) > 10 else None
    d = _lib.FoStepDesc(struct_size=ctypes.sizeof(_lib.FoStepDesc), opt=opt, param_dtype=param_dtype, grad_dtype=grad_dtype,
                        ecc_bits=ecc_bits, state=state, group_size=group_size, n_leaves=len(leaves), n_hypers=len(hypers),
                        leaves=ctypes.cast(L, ctypes.c_void_p), hypers=ctypes.cast(H, ctypes.c_void_p))
    if grad_sq_norm is not None:
        d.grad_sq_norm, d.max_grad_norm = grad_sq_norm.data_ptr(), float(max_grad_norm)
    keep = []
    for name, offs in (("peer_param_offsets", peer_param_offsets), ("peer_grad_offsets", peer_grad_offsets)):
        if offs is not None:
            arr = (ctypes.c_int64 * len(offs))(*[int(o) for o in offs])
            keep.append(arr)
            setattr(d, name, ctypes.cast(arr, ctypes.c_void_p))
            d.n_peers = len(offs)
    rc = _lib.lib().fo_step(ctypes.byref(d), stream)
    if expect_ok:
        _lib.check(rc)
    return rc


