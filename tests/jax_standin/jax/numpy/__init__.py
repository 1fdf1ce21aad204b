"""Stand-in for `jax.numpy` over NumPy + ml_dtypes.

Semantics that are NumPy's here and XLA's in a live JAX (everything else is a single IEEE
operation in both):

* `ldexp(x, k)` is NumPy's exact scaling by 2**k.  JAX evaluates `x * 2**k` in fp32, which is the
  same value whenever 2**k is a finite normal fp32 (|k| <= 126), i.e. for every parameter with
  |theta| >= 2**-119; below that JAX overflows 2**k and NumPy does not.
* `python_float ** float32_array` (the bias corrections) is NumPy's `powf`; XLA's fp32 `pow`
  may differ in the last place.
* float -> int8/uint8/int16 `astype` is a C cast; all call sites clip to the target range first.
* 16-bit float arithmetic (ml_dtypes) is evaluated in fp32 and rounded to nearest-even once per
  operation, as XLA's CPU backend does.
* Python scalars are weakly typed in both (NumPy >= 2): `f32_array * 0.9` stays fp32.  A float64
  result anywhere would mean a 64-bit intermediate a 32-bit JAX cannot have, so every function
  here refuses to return one.
"""
from __future__ import annotations

import numpy as _np
import ml_dtypes as _ml

float32 = _np.float32
float16 = _np.float16
bfloat16 = _ml.bfloat16
int8 = _np.int8
int16 = _np.int16
int32 = _np.int32
uint8 = _np.uint8
uint16 = _np.uint16
uint32 = _np.uint32
bool_ = _np.bool_
ndarray = _np.ndarray
dtype = _np.dtype
inf = _np.inf
pi = _np.pi


def _chk(x):
    dt = getattr(x, "dtype", None)
    if dt is not None and dt in (_np.float64, _np.int64) and getattr(x, "ndim", 0) >= 0:
        if dt == _np.float64:
            raise TypeError("a float64 intermediate appeared; 32-bit JAX never forms one")
        return x.astype(_np.int32)
    return x


def _in(x):
    """A bare Python float entering a function is a weakly typed fp32 value in JAX."""
    if isinstance(x, float):
        return _np.float32(x)
    return x


def _default_dtype(x, dt):
    if dt is not None:
        return dt
    if isinstance(x, bool):
        return _np.bool_
    if isinstance(x, int):
        return _np.int32
    if isinstance(x, float):
        return _np.float32
    if isinstance(x, (list, tuple)):
        probe = _np.asarray(x)
        if probe.dtype == _np.float64:
            return _np.float32
        if probe.dtype == _np.int64:
            return _np.int32
    return None


def asarray(x, dtype=None):
    return _np.asarray(x, dtype=_default_dtype(x, dtype))


def array(x, dtype=None):
    return _np.array(x, dtype=_default_dtype(x, dtype))


def zeros(shape, dtype=float32):
    return _np.zeros(shape, dtype=dtype)


def ones(shape, dtype=float32):
    return _np.ones(shape, dtype=dtype)


def full(shape, fill_value, dtype=None):
    return _np.full(shape, fill_value, dtype=_default_dtype(fill_value, dtype))


def zeros_like(x, dtype=None):
    return _np.zeros_like(_np.asarray(x), dtype=dtype)


def full_like(x, fill_value, dtype=None):
    return _np.full_like(_np.asarray(x), fill_value, dtype=dtype)


def arange(*args, dtype=None):
    return _np.arange(*args, dtype=dtype or _np.int32)


def linspace(start, stop, num=50, dtype=None):
    # float64 grid rounded once; used by the reference's tests only
    return _np.linspace(start, stop, num).astype(dtype or _np.float32)


def ravel(x):
    return _np.ravel(x)


def pad(x, pad_width):
    return _np.pad(x, pad_width)


def max(x, axis=None, keepdims=False):  # noqa: A001
    return _chk(_np.max(x, axis=axis, keepdims=keepdims))


def maximum(a, b):
    return _chk(_np.maximum(a, b))


def abs(x):  # noqa: A001
    return _chk(_np.abs(_in(x)))


def where(c, a, b):
    return _chk(_np.where(c, a, b))


def floor(x):
    return _chk(_np.floor(_in(x)))


def clip(x, lo, hi):
    return _chk(_np.clip(x, lo, hi))


def sqrt(x):
    return _chk(_np.sqrt(_in(x)))


def square(x):
    return _chk(_np.square(_in(x)))


def sign(x):
    return _chk(_np.sign(_in(x)))


def ldexp(x, k):
    return _chk(_np.ldexp(x, k))


def vdot(a, b):
    return _chk(_np.vdot(_np.asarray(a, dtype=_np.float32), _np.asarray(b, dtype=_np.float32)))


def sum(x, axis=None):  # noqa: A001
    return _chk(_np.sum(x, axis=axis))


def mean(x, axis=None):
    return _chk(_np.mean(x, axis=axis))


def allclose(a, b, rtol=1e-5, atol=1e-8):
    return bool(_np.allclose(_np.asarray(a, dtype=_np.float64), _np.asarray(b, dtype=_np.float64), rtol=rtol, atol=atol))


def array_equal(a, b):
    return bool(_np.array_equal(a, b))
