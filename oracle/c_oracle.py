"""ctypes front-end of the C restatement of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads oracle/_build/libflashoptim_oracle.so (built by oracle/Makefile) and exposes the
in-place leaf step and the codecs on NumPy arrays.  Used by the tests as the fast checker
for large shapes and by the benchmark as the timed CPU baseline; never by the product.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import ml_dtypes
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libflashoptim_oracle.so")

F32, BF16, F16 = 0, 1, 2
ADAM, LION, SGD = 0, 1, 2
STATE_QUANT, STATE_FULL, STATE_NONE = 0, 1, 2
FLAG_DECOUPLED, FLAG_NESTEROV, FLAG_LION_LERP, FLAG_LP_DELTA, FLAG_SCALE_FLOOR = 1, 2, 4, 8, 16


class Hyper(ctypes.Structure):
    _fields_ = [(k, ctypes.c_float) for k in ("lr", "wd", "b1", "b2", "omb1", "omb2", "eps", "bc1", "bc2")]


def build(force: bool = False) -> str:
    """Compile the shared object if it is missing or older than its source."""
    src = os.path.join(_HERE, "flashoptim_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.orc_step_leaf.restype = ctypes.c_int
        _lib.orc_step_leaf.argtypes = [
            ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
            ctypes.c_uint64, ctypes.c_int, ctypes.POINTER(Hyper), ctypes.c_int,
        ]
        for name in ("orc_quantize_momentum", "orc_quantize_variance"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_int]
        for name in ("orc_dequantize_momentum", "orc_dequantize_variance"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int]
        for name in ("orc_split", "orc_reconstruct"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint64]
        _lib.orc_set_threads.restype = ctypes.c_int
        _lib.orc_set_threads.argtypes = [ctypes.c_int]
    return _lib


def set_threads(n: int) -> int:
    """Set the OpenMP thread count (n <= 0 leaves it); returns the count in effect."""
    return lib().orc_set_threads(int(n))


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    if dt == np.dtype(np.float32):
        return F32
    if dt == np.dtype(ml_dtypes.bfloat16):
        return BF16
    if dt == np.dtype(np.float16):
        return F16
    raise ValueError(f"unsupported dtype {dt}")


def _ptr(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def step_leaf(opt, grad, param, ecc, mu, mu_scales, nu, nu_scales, *, state, group_size, hyper: Hyper, flags) -> None:
    """In-place optimizer step over one leaf; arrays are C-contiguous NumPy arrays (or None)."""
    ecc_bits = 0 if ecc is None else ecc.dtype.itemsize * 8
    rc = lib().orc_step_leaf(
        opt, _ptr(grad), dtype_code(grad.dtype), _ptr(param), dtype_code(param.dtype), _ptr(ecc), ecc_bits,
        _ptr(mu), _ptr(mu_scales), _ptr(nu), _ptr(nu_scales), state,
        param.size, group_size, ctypes.byref(hyper), flags,
    )
    if rc != 0:
        raise ValueError("orc_step_leaf rejected its arguments")


def quantize_momentum(x: np.ndarray, group_size: int = 32, flags: int = 0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    values = np.empty(x.shape, dtype=np.int8)
    scales = np.empty((x.size + group_size - 1) // group_size, dtype=np.float16)
    lib().orc_quantize_momentum(_ptr(x), _ptr(values), _ptr(scales), x.size, group_size, flags)
    return values, scales


def quantize_variance(x: np.ndarray, group_size: int = 32, flags: int = 0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    values = np.empty(x.shape, dtype=np.uint8)
    scales = np.empty((x.size + group_size - 1) // group_size, dtype=np.float16)
    lib().orc_quantize_variance(_ptr(x), _ptr(values), _ptr(scales), x.size, group_size, flags)
    return values, scales


def dequantize_momentum(values: np.ndarray, scales: np.ndarray, group_size: int = 32) -> np.ndarray:
    out = np.empty(values.shape, dtype=np.float32)
    lib().orc_dequantize_momentum(_ptr(np.ascontiguousarray(values)), _ptr(np.ascontiguousarray(scales)), _ptr(out), values.size, group_size)
    return out


def dequantize_variance(values: np.ndarray, scales: np.ndarray, group_size: int = 32) -> np.ndarray:
    out = np.empty(values.shape, dtype=np.float32)
    lib().orc_dequantize_variance(_ptr(np.ascontiguousarray(values)), _ptr(np.ascontiguousarray(scales)), _ptr(out), values.size, group_size)
    return out


def split(theta: np.ndarray, narrow_dtype, ecc_bits: int):
    theta = np.ascontiguousarray(theta, dtype=np.float32)
    lp = np.empty(theta.shape, dtype=narrow_dtype)
    ecc = None if ecc_bits == 0 else np.empty(theta.shape, dtype=np.int8 if ecc_bits == 8 else np.int16)
    lib().orc_split(_ptr(theta), _ptr(lp), _ptr(ecc), dtype_code(narrow_dtype), ecc_bits, theta.size)
    return lp, ecc


def reconstruct(lp: np.ndarray, ecc: Optional[np.ndarray]) -> np.ndarray:
    lp = np.ascontiguousarray(lp)
    out = np.empty(lp.shape, dtype=np.float32)
    ecc_bits = 0 if ecc is None else ecc.dtype.itemsize * 8
    lib().orc_reconstruct(_ptr(lp), _ptr(ecc), _ptr(out), dtype_code(lp.dtype), ecc_bits, lp.size)
    return out
