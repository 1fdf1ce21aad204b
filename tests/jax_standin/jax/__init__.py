"""Stand-in for the `jax` top-level module (NumPy arrays, eager evaluation).

Only the names the reference package and its tests use.  Arrays are plain `numpy.ndarray`
(16-bit floats through ml_dtypes); every operation runs eagerly, one IEEE fp32 rounding per
written operation, which is how un-jitted JAX dispatches the reference's CPU path.
"""
from __future__ import annotations

from typing import Any, NamedTuple, Tuple

import numpy as _np

from . import tree_util  # noqa: F401
from . import numpy  # noqa: F401

Array = _np.ndarray


class ShapeDtypeStruct(NamedTuple):
    shape: Tuple[int, ...]
    dtype: Any


def default_backend() -> str:
    return "cpu"


def block_until_ready(x):
    return x


def jit(fn=None, **_kwargs):
    """Eager: `jit` is the identity here (donation included)."""
    if fn is None:
        return lambda f: f
    return fn


from . import experimental  # noqa: E402,F401
