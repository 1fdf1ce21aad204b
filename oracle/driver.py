"""Drivers around the CPU oracle (TEST INFRASTRUCTURE ONLY): NumPy <-> torch conversion, the buffers of
one leaf, zero-initialised state, hyper-parameter tuples in the C layout, one oracle step, bit-exact
comparison.  Used by the tests, by the smoke check and by the benchmark's checker / CPU-baseline legs;
nothing in the product package imports it."""

from __future__ import annotations

from typing import Optional

import ml_dtypes
import numpy as np

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O

BF16 = np.dtype(ml_dtypes.bfloat16)
NP_OF_CODE = {0: np.dtype(np.float32), 1: BF16, 2: np.dtype(np.float16)}


def to_torch(a: Optional[np.ndarray], device="cuda"):
    import torch

    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype == BF16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(a.copy()).to(device)


def to_numpy(t) -> Optional[np.ndarray]:
    import torch

    if t is None:
        return None
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(BF16)
    return t.numpy()


def bits(a: np.ndarray) -> np.ndarray:
    """Bit pattern view, for exact comparisons that also tell -0 from +0."""
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


class LeafArrays:
    """One leaf's buffers as NumPy arrays (oracle side) or torch tensors (device side)."""

    def __init__(self, param, ecc, mu, mu_scales, nu, nu_scales):
        self.param, self.ecc, self.mu, self.mu_scales, self.nu, self.nu_scales = param, ecc, mu, mu_scales, nu, nu_scales

    def fields(self):
        return ("param", "ecc", "mu", "mu_scales", "nu", "nu_scales")

    def copy(self):
        return LeafArrays(*[None if getattr(self, f) is None else getattr(self, f).copy() for f in self.fields()])

    def to_device(self):
        return LeafArrays(*[to_torch(getattr(self, f)) for f in self.fields()])

    def to_host(self):
        return LeafArrays(*[to_numpy(getattr(self, f)) for f in self.fields()])


def fresh_leaf(param: np.ndarray, opt: int, state: int, ecc_bits: int, group_size: int = 32) -> LeafArrays:
    """Zero-initialised optimizer state for a parameter array (what tx.init produces)."""
    n = param.size
    G = (n + group_size - 1) // group_size
    ecc = None if ecc_bits == 0 else np.zeros(param.shape, dtype=np.int8 if ecc_bits == 8 else np.int16)
    mu = mu_s = nu = nu_s = None
    if state == C.STATE_QUANT:
        mu, mu_s = np.zeros(param.shape, np.int8), np.zeros(G, np.float16)
        if opt == C.ADAM:
            nu, nu_s = np.zeros(param.shape, np.uint8), np.zeros(G, np.float16)
    elif state == C.STATE_FULL:
        mu = np.zeros(param.shape, np.float32)
        if opt == C.ADAM:
            nu = np.zeros(param.shape, np.float32)
    return LeafArrays(param.copy(), ecc, mu, mu_s, nu, nu_s)


def hyper_tuple(opt: int, conv: O.Convention, count: int, *, lr, wd=0.0, b1=0.9, b2=0.999, eps=1e-8, momentum=0.9,
                dampening=0.0, nesterov=False, decoupled=True):
    """(lr, wd, b1, b2, omb1, omb2, eps, bc1, bc2, flags) as the library and the C oracle take them."""
    f = np.float32
    flags = 0
    if conv.scale_floor:
        flags |= C.FLAG_SCALE_FLOOR
    if opt == C.ADAM:
        bc1, bc2 = O.bias_corrections(b1, b2, count)
        flags |= (C.FLAG_DECOUPLED if decoupled else 0) | (C.FLAG_LP_DELTA if conv.adam_bf16_delta else 0)
        return (f(lr), f(wd), f(b1), f(b2), O.one_minus(b1, conv), O.one_minus(b2, conv), f(eps), bc1, bc2, flags)
    if opt == C.LION:
        flags |= C.FLAG_DECOUPLED | (C.FLAG_LION_LERP if conv.lion_lerp else 0)
        return (f(lr), f(wd), f(b1), f(b2), O.one_minus(b1, conv), O.one_minus(b2, conv), f(0), f(1), f(1), flags)
    flags |= (C.FLAG_DECOUPLED if decoupled else 0) | (C.FLAG_NESTEROV if nesterov else 0)
    return (f(lr), f(wd), f(momentum), f(0), f(1.0 - dampening), f(0), f(0), f(1), f(1), flags)


def oracle_step(opt: int, grad: np.ndarray, leaf: LeafArrays, state: int, group_size: int, hp) -> None:
    """One in-place step of the C oracle."""
    h = C.Hyper(*[float(x) for x in hp[:9]])
    C.step_leaf(opt, np.ascontiguousarray(grad), leaf.param, leaf.ecc, leaf.mu, leaf.mu_scales, leaf.nu, leaf.nu_scales,
                state=state, group_size=group_size, hyper=h, flags=int(hp[9]))


def assert_leaf_equal(dev: LeafArrays, ref: LeafArrays, what: str = "") -> None:
    """Bit-exact comparison of every buffer of a leaf."""
    for f in dev.fields():
        a, b = getattr(dev, f), getattr(ref, f)
        assert (a is None) == (b is None), f"{what}: {f} presence differs"
        if a is None:
            continue
        ab, bb = bits(a).ravel(), bits(b).ravel()
        bad = np.flatnonzero(ab != bb)
        assert bad.size == 0, (
            f"{what}: {f} differs at {bad.size}/{ab.size} positions; first {bad[:5]}: "
            f"device {np.asarray(a).ravel()[bad[:5]]} oracle {np.asarray(b).ravel()[bad[:5]]}"
        )


def make_grad(rng: np.random.Generator, shape, sigma: float, dtype, outliers: float = 0.0) -> np.ndarray:
    g = rng.normal(0.0, sigma, size=shape).astype(np.float32)
    if outliers > 0:
        mask = rng.random(size=shape) < outliers
        g = np.where(mask, g * np.float32(100.0), g).astype(np.float32)
    return g.astype(dtype)
