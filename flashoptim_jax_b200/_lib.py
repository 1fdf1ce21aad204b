"""ctypes binding of libflashoptim_b200.so (the C ABI declared in include/flashoptim_b200.h).

There is no fallback: if the shared object is missing or does not load, importing the
package's compute entry points raises, telling the user to build it.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FLASHOPTIM_B200_LIB names another build of the same library (e.g. one compiled with other tuning macros)
LIB_PATH = os.environ.get("FLASHOPTIM_B200_LIB") or os.path.join(_HERE, "lib", "libflashoptim_b200.so")

FO_OK = 0
FO_F32, FO_BF16, FO_F16 = 0, 1, 2
FO_OPT_ADAM, FO_OPT_LION, FO_OPT_SGD = 0, 1, 2
FO_STATE_QUANT, FO_STATE_FULL, FO_STATE_NONE = 0, 1, 2
FO_FLAG_DECOUPLED_WD, FO_FLAG_NESTEROV, FO_FLAG_LION_LERP, FO_FLAG_LP_DELTA, FO_FLAG_SCALE_FLOOR = 1, 2, 4, 8, 16
FO_MAX_HYPERS = 16
FO_MAX_PEERS = 7
FO_SELFTEST_STATIC_MAX_COUNTERS = 4
FO_SELFTEST_SQRT, FO_SELFTEST_SOFTSIGN, FO_SELFTEST_RECONSTRUCT, FO_SELFTEST_SPLIT = 0, 1, 2, 3
FO_SELFTEST_GROUP_DIV, FO_SELFTEST_CODE_TABLES, FO_SELFTEST_RCP, FO_SELFTEST_PACKED = 4, 5, 6, 7

EXPORTS = (
    "fo_step", "fo_quantize_momentum", "fo_dequantize_momentum", "fo_quantize_variance",
    "fo_dequantize_variance", "fo_split", "fo_reconstruct", "fo_selftest", "fo_selftest_static", "fo_version",
    "fo_status_string", "fo_last_error", "fo_sq_norm", "fo_mean_sq_norm", "fo_step_scalars", "fo_step_scalars_schedule",
)
FO_SQ_NORM_WORKSPACE_BYTES = 16384


class FoHyper(ctypes.Structure):
    _fields_ = [
        ("lr", ctypes.c_float), ("wd", ctypes.c_float),
        ("b1", ctypes.c_float), ("b2", ctypes.c_float),
        ("one_minus_b1", ctypes.c_float), ("one_minus_b2", ctypes.c_float),
        ("eps", ctypes.c_float),
        ("bc1", ctypes.c_float), ("bc2", ctypes.c_float),
        ("flags", ctypes.c_uint32),
        ("dev_scalars", ctypes.c_void_p),
    ]


class FoLeaf(ctypes.Structure):
    _fields_ = [
        ("grad", ctypes.c_void_p), ("param", ctypes.c_void_p), ("ecc", ctypes.c_void_p),
        ("mu", ctypes.c_void_p), ("mu_scales", ctypes.c_void_p),
        ("nu", ctypes.c_void_p), ("nu_scales", ctypes.c_void_p),
        ("n", ctypes.c_uint64), ("hyper", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
    ]


class FoStepDesc(ctypes.Structure):
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("opt", ctypes.c_int32), ("param_dtype", ctypes.c_int32), ("grad_dtype", ctypes.c_int32),
        ("ecc_bits", ctypes.c_int32), ("state", ctypes.c_int32), ("group_size", ctypes.c_int32),
        ("n_leaves", ctypes.c_uint32), ("n_hypers", ctypes.c_uint32),
        ("leaves", ctypes.c_void_p), ("hypers", ctypes.c_void_p),
        ("n_peers", ctypes.c_uint32), ("reserved", ctypes.c_uint32), ("peer_param_offsets", ctypes.c_void_p),
        ("peer_grad_offsets", ctypes.c_void_p),
        ("grad_sq_norm", ctypes.c_void_p), ("max_grad_norm", ctypes.c_float), ("reserved2", ctypes.c_uint32),
        ("mc_param_offset", ctypes.c_int64), ("mc_grad_offset", ctypes.c_int64),
    ]


class FoArray(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("n", ctypes.c_uint64)]


class NativeLibraryError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared object once; raise loudly when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m flashoptim_jax_b200.build` "
            "(needs nvcc; there is no CPU or eager fallback)"
        )
    try:
        cdll = ctypes.CDLL(LIB_PATH)
    except OSError as e:
        raise NativeLibraryError(f"cannot load {LIB_PATH}: {e}") from e
    vp, u64, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int32
    cdll.fo_step.restype = ctypes.c_int
    cdll.fo_step.argtypes = [ctypes.POINTER(FoStepDesc), vp]
    for name in ("fo_quantize_momentum", "fo_quantize_variance"):
        fn = getattr(cdll, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [vp, vp, vp, u64, i32, i32, vp]
    for name in ("fo_dequantize_momentum", "fo_dequantize_variance"):
        fn = getattr(cdll, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [vp, vp, vp, u64, i32, vp]
    for name in ("fo_split", "fo_reconstruct"):
        fn = getattr(cdll, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [vp, vp, vp, i32, i32, u64, vp]
    cdll.fo_selftest.restype = ctypes.c_int
    cdll.fo_selftest.argtypes = [i32, ctypes.c_int64, ctypes.POINTER(ctypes.c_uint64), vp]
    cdll.fo_selftest_static.restype = ctypes.c_int
    cdll.fo_selftest_static.argtypes = [i32, ctypes.c_int64, ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint32, vp]
    cdll.fo_sq_norm.restype = ctypes.c_int
    cdll.fo_sq_norm.argtypes = [ctypes.POINTER(FoArray), ctypes.c_uint32, i32, i32, vp, vp, vp]
    cdll.fo_mean_sq_norm.restype = ctypes.c_int
    cdll.fo_mean_sq_norm.argtypes = [vp, vp, ctypes.c_uint64, i32, vp, ctypes.c_uint32, i32, vp, vp, vp]
    cdll.fo_step_scalars.restype = ctypes.c_int
    cdll.fo_step_scalars.argtypes = [vp, vp, ctypes.c_float, ctypes.c_float, ctypes.c_float, vp, vp, vp]
    cdll.fo_step_scalars_schedule.restype = ctypes.c_int
    cdll.fo_step_scalars_schedule.argtypes = [vp, i32, ctypes.POINTER(ctypes.c_float), ctypes.c_float, ctypes.c_float, vp, vp, vp]
    cdll.fo_version.restype = ctypes.c_int
    cdll.fo_version.argtypes = []
    cdll.fo_status_string.restype = ctypes.c_char_p
    cdll.fo_status_string.argtypes = [ctypes.c_int]
    cdll.fo_last_error.restype = ctypes.c_char_p
    cdll.fo_last_error.argtypes = []
    _lib = cdll
    return _lib


def check(status: int) -> None:
    """Turn a non-zero status into an exception carrying the library's message."""
    if status != FO_OK:
        l = lib()
        kind = l.fo_status_string(status).decode()
        detail = l.fo_last_error().decode()
        exc = ValueError if status in (1, 2, 4) else RuntimeError
        raise exc(f"flashoptim_b200: {kind}: {detail}")
