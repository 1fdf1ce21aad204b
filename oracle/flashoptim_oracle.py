"""CPU oracle for the flashoptim optimizer-step hot path (TEST INFRASTRUCTURE ONLY).

This module is a NumPy + ml_dtypes restatement of the reference's CPU-runnable
("unfused") code path and of the arithmetic written inside its fused kernels.
It exists to check the CUDA library; nothing that ships may import it.  Only the
tests, the smoke check and the benchmark's CPU-baseline leg use it.

Parity status: pinned on outputs of the reference's own text.  JAX is not
installable where this oracle was written, so tests/golden/make_golden.py imports the
reference's source files unmodified over a NumPy stand-in for the `jax` names they
use (tests/jax_standin, with a NumPy interpreter for the Pallas kernels) and records
what the reference's public API returns for both of its texts; this module and its C
twin reproduce those vectors bit for bit (tests/test_golden.py).  Also pinned on every
exact known answer the reference's own tests hold (tests/test_oracle_pins.py).  What
the stand-in cannot show: XLA's own `pow` (bias corrections) and `ldexp` below
2**-119, and the code Triton generates for the kernels on a GPU.

Numerical contract (every function below keeps it):
  * strict IEEE fp32, one rounding per written operation, evaluated left to
    right as the reference writes it, no fused multiply-add;
  * true divisions (never reciprocal multiplies);
  * codes round with floor(x + 0.5); ECC rounds half away from zero;
  * casts to bf16 / fp16 are round-to-nearest-even with subnormals kept;
  * ldexp is an exact power-of-two scaling (correctly rounded when the result is
    subnormal).

Two conventions exist because the reference has two texts for the same step:
  UNFUSED  — the jnp code that runs on CPU  (adamw.py:356-423 + 463,
             lion.py:18-70, sgd.py:18-77)
  FUSED    — the body of the Pallas kernels  (adamw.py:45-145,
             momentum_kernel.py:38-112), evaluated with the same strict fp32
             rules (the GPU compiler's own contraction choices are not modelled).
They differ in how (1 - beta) is formed, in Lion's interpolation form, in the
guard applied to an all-zero group scale and in how AdamW hands back the param.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, NamedTuple, Optional, Sequence, Tuple, Union

import ml_dtypes
import numpy as np

F32 = np.float32
BF16 = np.dtype(ml_dtypes.bfloat16)
FP16 = np.dtype(np.float16)
FP32 = np.dtype(np.float32)

ECC_MAX = {np.dtype(np.int8): F32(127.0), np.dtype(np.int16): F32(32767.0)}
# compression.py:20-33 / utils.py:26-29
LP_CONSTANTS = {
    BF16: {"mantissa_bits": 7, "min_normal_exponent": -126},
    FP16: {"mantissa_bits": 10, "min_normal_exponent": -14},
}


class Quantized(NamedTuple):
    """values has the shape of the tensor, scales one fp16 per group (quantization.py:9-12)."""

    values: np.ndarray
    scales: np.ndarray


@dataclass(frozen=True)
class Convention:
    """Which of the reference's two texts a step follows."""

    name: str
    one_minus_in_f32: bool  # True: 1.0 - f32(beta) in fp32 (adamw.py:99-100); False: f32(1.0 - beta) (adamw.py:394-395)
    lion_lerp: bool  # True: mu + (1-b)(g-mu) (lion.py:50-52); False: b*mu + (1-b)*g (momentum_kernel.py:78-79)
    adam_bf16_delta: bool  # True: param + bf16(new - param) (adamw.py:411,463); False: store new_lp (adamw.py:134)
    scale_floor: bool  # True: max(absmax, 1e-12) (adamw.py:121,128); False: where(absmax > 0, absmax, 1) (quantization.py:41)


UNFUSED = Convention("unfused", one_minus_in_f32=False, lion_lerp=True, adam_bf16_delta=True, scale_floor=False)
FUSED = Convention("fused", one_minus_in_f32=True, lion_lerp=False, adam_bf16_delta=False, scale_floor=True)


def _f32(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32)


def one_minus(beta: float, conv: Convention) -> np.float32:
    """(1 - beta) as the chosen reference text forms it."""
    if conv.one_minus_in_f32:
        return F32(F32(1.0) - F32(beta))
    return F32(1.0 - float(beta))


# --------------------------------------------------------------------------
# quantization.py
# --------------------------------------------------------------------------


def _round_to_nearest(x: np.ndarray) -> np.ndarray:
    """floor(x + 0.5): ties go up (quantization.py:15-17)."""
    return np.floor(_f32(x) + F32(0.5))


def _pad_groups(x: np.ndarray, group_size: int) -> Tuple[np.ndarray, int]:
    """Row-major flatten, zero-pad the last group (quantization.py:20-26)."""
    flat = np.ravel(_f32(x))
    pad = (-flat.size) % group_size
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=np.float32)])
    return flat.reshape((-1, group_size)), pad


def _unpad_groups(x: np.ndarray, pad: int, shape) -> np.ndarray:
    flat = x.reshape((-1,))
    if pad:
        flat = flat[:-pad]
    return flat.reshape(shape)


def _safe_scales(scales: np.ndarray, conv: Convention) -> np.ndarray:
    if conv.scale_floor:
        return np.maximum(scales, F32(1e-12))
    return np.where(scales > 0, scales, F32(1.0)).astype(np.float32)


def quantize_momentum(x: np.ndarray, group_size: int = 32, conv: Convention = UNFUSED) -> Quantized:
    """int8 soft-sign codes with per-group absmax scales (quantization.py:37-46; kernel twin adamw.py:120-125)."""
    x = np.asarray(x)
    groups, pad = _pad_groups(x, group_size)
    scales = np.max(np.abs(groups), axis=1, keepdims=True)
    safe = _safe_scales(scales, conv)
    normalized = groups / safe
    transformed = (F32(2.0) * normalized) / (F32(1.0) + np.abs(normalized))
    quantized = _round_to_nearest(transformed * F32(127.0))
    values = _unpad_groups(np.clip(quantized, F32(-127.0), F32(127.0)), pad, x.shape).astype(np.int8)
    stored = safe if conv.scale_floor else scales
    return Quantized(values=values, scales=stored.reshape((-1,)).astype(np.float16))


def dequantize_momentum(q: Quantized, group_size: int = 32) -> np.ndarray:
    """Inverse soft-sign times the fp16 scale (quantization.py:49-56)."""
    groups, pad = _pad_groups(q.values, group_size)
    transformed = groups / F32(127.0)
    normalized = transformed / (F32(2.0) - np.abs(transformed))
    scales = q.scales.astype(np.float32).reshape((-1, 1))
    return _unpad_groups(normalized * scales, pad, q.values.shape)


def quantize_variance(x: np.ndarray, group_size: int = 32, conv: Convention = UNFUSED) -> Quantized:
    """uint8 codes of sqrt(x) with per-group max scales (quantization.py:59-68; kernel twin adamw.py:127-131)."""
    x = np.asarray(x)
    root = np.sqrt(_f32(x))
    groups, pad = _pad_groups(root, group_size)
    scales = np.max(groups, axis=1, keepdims=True)
    safe = _safe_scales(scales, conv)
    transformed = groups / safe
    quantized = _round_to_nearest(transformed * F32(255.0))
    values = _unpad_groups(np.clip(quantized, F32(0.0), F32(255.0)), pad, x.shape).astype(np.uint8)
    stored = safe if conv.scale_floor else scales
    return Quantized(values=values, scales=stored.reshape((-1,)).astype(np.float16))


def dequantize_variance(q: Quantized, group_size: int = 32) -> np.ndarray:
    """(code/255 * scale)^2 (quantization.py:71-77)."""
    groups, pad = _pad_groups(q.values, group_size)
    transformed = groups / F32(255.0)
    scales = q.scales.astype(np.float32).reshape((-1, 1))
    root = transformed * scales
    return _unpad_groups(root * root, pad, q.values.shape)


# --------------------------------------------------------------------------
# utils.py:499-557 and compression.py:39-121
# --------------------------------------------------------------------------


def _round_away_from_zero(x: np.ndarray) -> np.ndarray:
    """sign(x) * floor(|x| + 0.5) (utils.py:499-501)."""
    return np.sign(x) * np.floor(np.abs(x) + F32(0.5))


def log_half_ulp(x_lp: np.ndarray) -> np.ndarray:
    """Exponent of half an ULP of each low-precision value (utils.py:504-518)."""
    dt = np.dtype(x_lp.dtype)
    c = LP_CONSTANTS[dt]
    mant, emin = c["mantissa_bits"], c["min_normal_exponent"]
    bias = 1 - emin
    bits = np.abs(x_lp).view(np.uint16).astype(np.int32)
    exponent_bits = bits >> mant
    unbiased = np.where(exponent_bits == 0, np.int32(emin), exponent_bits - bias)
    return (unbiased - mant - 1).astype(np.int32)


def ecc_dtype_for(narrow_dtype, master_weight_bits: Optional[int]):
    """int8 / int16 / None (compression.py:39-54)."""
    if master_weight_bits not in (None, 24, 32):
        raise ValueError(f"master_weight_bits must be one of (None, 24, 32), got {master_weight_bits}")
    narrow_dtype = np.dtype(narrow_dtype)
    if master_weight_bits is None or narrow_dtype not in LP_CONSTANTS:
        return None
    nbytes = master_weight_bits // 8 - narrow_dtype.itemsize
    if nbytes <= 0:
        return None
    return np.dtype(np.int8) if nbytes == 1 else np.dtype(np.int16)


def split_leaf(theta, narrow_dtype=BF16, master_weight_bits: Optional[int] = 24):
    """fp32 -> (low-precision value, ECC or None) (compression.py:84-104, utils.py:539-557)."""
    theta = _f32(theta)
    narrow_dtype = np.dtype(narrow_dtype)
    lp = theta.astype(narrow_dtype)
    ecc_dt = ecc_dtype_for(narrow_dtype, master_weight_bits)
    if ecc_dt is None:
        return lp, None
    error = theta - lp.astype(np.float32)
    ls = log_half_ulp(lp)
    error_norm = np.ldexp(error, -ls).astype(np.float32)
    scaled = np.clip(error_norm, F32(-1.0), F32(1.0)) * ECC_MAX[ecc_dt]
    return lp, _round_away_from_zero(scaled).astype(ecc_dt)


def reconstruct_leaf(lp: np.ndarray, ecc: Optional[np.ndarray]) -> np.ndarray:
    """(low-precision value, ECC) -> fp32 (compression.py:107-121, utils.py:521-536)."""
    lp = np.asarray(lp)
    if ecc is None or np.dtype(lp.dtype) not in LP_CONSTANTS or np.dtype(ecc.dtype) not in ECC_MAX:
        return lp.astype(np.float32)
    ls = log_half_ulp(lp)
    correction = ecc.astype(np.float32) / ECC_MAX[np.dtype(ecc.dtype)]
    error = np.ldexp(correction, ls).astype(np.float32)
    return lp.astype(np.float32) + error


def use_ecc_leaf(param: np.ndarray, master_weight_bits: Optional[int]) -> bool:
    """utils.py:174-181."""
    if master_weight_bits is None:
        return False
    dt = np.dtype(param.dtype)
    if dt not in LP_CONSTANTS:
        return False
    return master_weight_bits > dt.itemsize * 8


# --------------------------------------------------------------------------
# scalar preparation (adamw.py:510,526-528; utils.py:277-284)
# --------------------------------------------------------------------------


def bias_corrections(b1: float, b2: float, count: int) -> Tuple[np.float32, np.float32]:
    """1 - f32(beta) ** f32(count), count being the post-increment step number.

    The reference evaluates the power with XLA's fp32 pow; here it is evaluated in
    float64 and rounded once, which is the correctly rounded value.  A last-place
    difference of the live pow from this is a documented, permitted deviation.
    """
    c = float(count)
    p1 = F32(float(F32(b1)) ** c)
    p2 = F32(float(F32(b2)) ** c)
    return F32(F32(1.0) - p1), F32(F32(1.0) - p2)


# --------------------------------------------------------------------------
# per-leaf steps
# --------------------------------------------------------------------------

State = Union[Quantized, np.ndarray]


class AdamLeaf(NamedTuple):
    param: np.ndarray
    ecc: Optional[np.ndarray]
    mu: State
    nu: State


class MomentumLeaf(NamedTuple):
    param: np.ndarray
    ecc: Optional[np.ndarray]
    mu: Optional[State]


def _materialize_m(mu: State, group_size: int) -> np.ndarray:
    return dequantize_momentum(mu, group_size) if isinstance(mu, Quantized) else _f32(mu)


def _materialize_v(nu: State, group_size: int) -> np.ndarray:
    return dequantize_variance(nu, group_size) if isinstance(nu, Quantized) else _f32(nu)


def _bf16_style_sub(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """a - b between two low-precision arrays: computed in fp32, rounded to the arrays' dtype."""
    return (a.astype(np.float32) - b.astype(np.float32)).astype(a.dtype)


def _bf16_style_add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    return (a.astype(np.float32) + b.astype(np.float32)).astype(a.dtype)


def adam_leaf(
    grad,
    param: np.ndarray,
    ecc: Optional[np.ndarray],
    mu: State,
    nu: State,
    *,
    lr,
    b1: float,
    b2: float,
    eps: float,
    weight_decay: float,
    decoupled_weight_decay: bool,
    bias_correction1,
    bias_correction2,
    quantize: bool = True,
    group_size: int = 32,
    master_weight_bits: Optional[int] = 24,
    conv: Convention = UNFUSED,
) -> AdamLeaf:
    """One Adam/AdamW step on one leaf (adamw.py:356-423 and :463; kernel text adamw.py:76-131)."""
    g = _f32(grad)
    lr = F32(lr)
    b1f, b2f, epsf, wdf = F32(b1), F32(b2), F32(eps), F32(weight_decay)
    bc1, bc2 = F32(bias_correction1), F32(bias_correction2)
    use_ecc = use_ecc_leaf(param, master_weight_bits)
    theta = reconstruct_leaf(param, ecc) if use_ecc else param.astype(np.float32)
    m = _materialize_m(mu, group_size)
    v = _materialize_v(nu, group_size)

    if not decoupled_weight_decay and (weight_decay or conv is FUSED):
        g = g + wdf * theta
    m = b1f * m + one_minus(b1, conv) * g
    v = b2f * v + one_minus(b2, conv) * (g * g)
    if decoupled_weight_decay and (weight_decay or conv is FUSED):
        theta = theta * (F32(1.0) - lr * wdf)
    new_theta = theta - ((lr / bc1) * m) / (np.sqrt(v) / np.sqrt(bc2) + epsf)

    if use_ecc:
        new_lp, new_ecc = split_leaf(new_theta, param.dtype, master_weight_bits)
    else:
        new_lp, new_ecc = new_theta.astype(param.dtype), None
    if conv.adam_bf16_delta:
        update = _bf16_style_sub(new_lp, param)
        new_param = _bf16_style_add(param, update)
    else:
        new_param = new_lp
    mu_out = quantize_momentum(m, group_size, conv) if quantize else m
    nu_out = quantize_variance(v, group_size, conv) if quantize else v
    return AdamLeaf(new_param, new_ecc, mu_out, nu_out)


def lion_leaf(
    grad,
    param: np.ndarray,
    ecc: Optional[np.ndarray],
    mu: State,
    *,
    lr,
    b1: float,
    b2: float,
    weight_decay: float,
    quantize: bool = True,
    group_size: int = 32,
    master_weight_bits: Optional[int] = 24,
    conv: Convention = UNFUSED,
) -> MomentumLeaf:
    """One Lion step on one leaf (lion.py:18-70; kernel text momentum_kernel.py:74-103 with do_lion)."""
    g = _f32(grad)
    lr = F32(lr)
    wdf = F32(weight_decay)
    use_ecc = use_ecc_leaf(param, master_weight_bits)
    theta = reconstruct_leaf(param, ecc) if use_ecc else param.astype(np.float32)
    m = _materialize_m(mu, group_size)

    if conv.lion_lerp:
        if weight_decay:
            theta = theta * (F32(1.0) - lr * wdf)
        update = np.sign(m + one_minus(b1, conv) * (g - m))
        new_theta = theta - lr * update
        m = m + one_minus(b2, conv) * (g - m)
    else:
        update = np.sign(F32(b1) * m + one_minus(b1, conv) * g)
        m = F32(b2) * m + one_minus(b2, conv) * g
        theta = theta * (F32(1.0) - lr * wdf)
        new_theta = theta - lr * update

    if use_ecc:
        new_lp, new_ecc = split_leaf(new_theta, param.dtype, master_weight_bits)
    else:
        new_lp, new_ecc = new_theta.astype(param.dtype), None
    mu_out = quantize_momentum(m, group_size, conv) if quantize else m
    return MomentumLeaf(new_lp, new_ecc, mu_out)


def sgd_leaf(
    grad,
    param: np.ndarray,
    ecc: Optional[np.ndarray],
    mu: Optional[State],
    *,
    lr,
    momentum: float,
    dampening: float,
    weight_decay: float,
    nesterov: bool,
    decoupled_weight_decay: bool,
    quantize: bool = True,
    group_size: int = 32,
    master_weight_bits: Optional[int] = 24,
    conv: Convention = UNFUSED,
) -> MomentumLeaf:
    """One SGD/SGDW step on one leaf (sgd.py:18-77; kernel text momentum_kernel.py:74-103).

    momentum == 0 keeps no momentum buffer (mu is None) and steps along the gradient.
    """
    g = _f32(grad)
    lr = F32(lr)
    wdf = F32(weight_decay)
    use_ecc = use_ecc_leaf(param, master_weight_bits)
    theta = reconstruct_leaf(param, ecc) if use_ecc else param.astype(np.float32)

    if not decoupled_weight_decay and (weight_decay or conv is FUSED):
        g = g + wdf * theta
    if momentum > 0.0:
        if mu is None:
            m = g
        else:
            m = F32(momentum) * _materialize_m(mu, group_size) + F32(1.0 - dampening) * g
        direction = g + F32(momentum) * m if nesterov else m
    else:
        m = None
        direction = g
    if decoupled_weight_decay and (weight_decay or conv is FUSED):
        theta = theta * (F32(1.0) - lr * wdf)
    new_theta = theta - lr * direction

    if use_ecc:
        new_lp, new_ecc = split_leaf(new_theta, param.dtype, master_weight_bits)
    else:
        new_lp, new_ecc = new_theta.astype(param.dtype), None
    if m is None:
        mu_out = None
    else:
        mu_out = quantize_momentum(m, group_size, conv) if quantize else m
    return MomentumLeaf(new_lp, new_ecc, mu_out)


# --------------------------------------------------------------------------
# state initialisation (utils.py:287-306, 337-358)
# --------------------------------------------------------------------------


def init_adam_leaf(param: np.ndarray, group_size: int = 32, quantize: bool = True, master_weight_bits: Optional[int] = 24):
    zeros = np.zeros(param.shape, dtype=np.float32)
    mu = quantize_momentum(zeros, group_size) if quantize else zeros
    nu = quantize_variance(zeros, group_size) if quantize else zeros.copy()
    ecc = None
    if use_ecc_leaf(param, master_weight_bits):
        ecc = np.zeros(param.shape, dtype=np.int8 if master_weight_bits == 24 else np.int16)
    return mu, nu, ecc


def init_momentum_leaf(
    param: np.ndarray,
    group_size: int = 32,
    quantize: bool = True,
    master_weight_bits: Optional[int] = 24,
    use_momentum: bool = True,
):
    mu = None
    if use_momentum:
        zeros = np.zeros(param.shape, dtype=np.float32)
        mu = quantize_momentum(zeros, group_size) if quantize else zeros
    ecc = None
    if use_ecc_leaf(param, master_weight_bits):
        ecc = np.zeros(param.shape, dtype=np.int8 if master_weight_bits == 24 else np.int16)
    return mu, ecc


# ---- global-norm gradient clipping in front of the step ------------------------------------------
#
# The reference's GPT-2 recipe chains optax.clip_by_global_norm before tx.step
# (examples/train_gpt2_pretrain.py:56-70).  optax is a third-party dependency of the examples
# (unpinned, not vendored); its published algorithm is
#     g_norm  = sqrt(sum over leaves of sum(|g|^2))
#     trigger = g_norm < max_norm
#     g      <- g if trigger else (g / g_norm.astype(g.dtype)) * max_norm
# with every operation carried out in the leaf's dtype (XLA evaluates bf16 / fp16 element-wise
# operations in fp32 and rounds the result).  The order in which XLA sums the squares is not
# specified, so the norm itself is "parity unpinned": this restatement takes squares exactly,
# sums them in float64 and rounds the square root to fp32; the element-wise part is exact given
# the norm.


def global_sq_norm(grads: Sequence[np.ndarray]) -> float:
    return float(sum(np.sum(np.asarray(g, dtype=np.float64) ** 2) for g in grads))


def clip_by_global_norm(grads: Sequence[np.ndarray], max_norm: float, sq_norm: Optional[float] = None) -> List[np.ndarray]:
    """Clipped copies of `grads`.  `sq_norm` overrides the sum of squares (to feed the value a device computed)."""
    if sq_norm is None:
        sq_norm = global_sq_norm(grads)
    norm = np.float32(np.sqrt(np.float64(sq_norm)))
    if norm < np.float32(max_norm):
        return [np.array(g, copy=True) for g in grads]
    out = []
    for g in grads:
        dt = g.dtype
        n_g = np.float32(norm.astype(dt))
        m_g = np.float32(np.float32(max_norm).astype(dt))
        q = (g.astype(np.float32) / n_g).astype(np.float32).astype(dt)
        out.append((q.astype(np.float32) * m_g).astype(np.float32).astype(dt))
    return out
