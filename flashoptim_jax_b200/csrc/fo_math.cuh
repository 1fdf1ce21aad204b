// Device arithmetic of the optimizer step: strict fp32, one IEEE rounding per written
// operation, never contracted into FMA (the __f*_rn intrinsics are exempt from contraction).
//
// Two families live here:
//   ieee::  the formulas exactly as the reference writes them, on the plain IEEE
//           operations (division, square root, ldexp).  Slow, obviously right.
//   fast::  shortcuts that give the same bits with fewer instructions: divisions by a
//           constant or by a per-group scale through one correctly rounded reciprocal and
//           an FMA residual correction (Markstein), power-of-two scaling through exponent
//           bit arithmetic, square root through one MUFU.RSQ and an FMA correction.  Each
//           shortcut has a guarded range outside which it falls back to ieee::, and each
//           is compared with ieee:: on the device by fo_selftest (exhaustively where the
//           input space allows).
// The step kernels use fast:: unless FO_NAIVE_MATH is defined.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/flashoptim_b200.h"

#define FO_DEVI __device__ __forceinline__

namespace fo {

FO_DEVI float fmul(float a, float b) { return __fmul_rn(a, b); }
FO_DEVI float fadd(float a, float b) { return __fadd_rn(a, b); }
FO_DEVI float fsub(float a, float b) { return __fsub_rn(a, b); }
FO_DEVI float fdiv(float a, float b) { return __fdiv_rn(a, b); }
FO_DEVI float fsqrt(float a) { return __fsqrt_rn(a); }

// ---- 16-bit parameter formats ------------------------------------------------------------
// mantissa bits / min normal exponent as in flashoptim_jax/utils.py:26-29.
template <int PDT>
struct Lp;
template <>
struct Lp<FO_BF16> {
  static constexpr int MANT = 7, EMIN = -126, BIAS = 127;
  static FO_DEVI float to_f32(uint32_t b) { return __uint_as_float(b << 16); }
  static FO_DEVI uint32_t from_f32(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
};
template <>
struct Lp<FO_F16> {
  static constexpr int MANT = 10, EMIN = -14, BIAS = 15;
  static FO_DEVI float to_f32(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)b)); }
  static FO_DEVI uint32_t from_f32(float f) { return __half_as_ushort(__float2half_rn(f)); }
};

template <int ECC_BITS>
struct Ecc {
  static constexpr float MAX = ECC_BITS == 8 ? 127.0f : 32767.0f;
  // 1/MAX rounded to nearest: 0x3C010204 = RN(1/127), 0x38000100 = RN(1/32767)
  static constexpr uint32_t RCP_BITS = ECC_BITS == 8 ? 0x3C010204u : 0x38000100u;
};

// exponent of half an ULP of a 16-bit value (flashoptim_jax/utils.py:504-518)
template <int PDT>
FO_DEVI int log_half_ulp(uint32_t bits) {
  using L = Lp<PDT>;
  int eb = (int)((bits & 0x7FFFu) >> L::MANT);
  int e = eb == 0 ? L::EMIN : eb - L::BIAS;
  return e - L::MANT - 1;
}

// ===========================================================================================
namespace ieee {

// flashoptim_jax/quantization.py:49-56 without the scale: (q/127) / (2 - |q/127|)
FO_DEVI float deq_m_norm(int q) {
  float t = fdiv((float)q, 127.0f);
  return fdiv(t, fsub(2.0f, fabsf(t)));
}
// flashoptim_jax/quantization.py:74: q/255
FO_DEVI float deq_v_norm(int q) { return fdiv((float)q, 255.0f); }

// flashoptim_jax/utils.py:521-536
template <int PDT, int ECC_BITS>
FO_DEVI float reconstruct(uint32_t bits, int ecc) {
  float corr = fdiv((float)ecc, Ecc<ECC_BITS>::MAX);
  float err = ldexpf(corr, log_half_ulp<PDT>(bits));
  return fadd(Lp<PDT>::to_f32(bits), err);
}

// flashoptim_jax/utils.py:539-557 (+ :499-501)
template <int PDT, int ECC_BITS>
FO_DEVI void split(float theta, uint32_t& bits, int& ecc) {
  bits = Lp<PDT>::from_f32(theta);
  float err = fsub(theta, Lp<PDT>::to_f32(bits));
  float en = ldexpf(err, -log_half_ulp<PDT>(bits));
  float c = fminf(fmaxf(en, -1.0f), 1.0f);
  float s = fmul(c, Ecc<ECC_BITS>::MAX);
  float r = floorf(fadd(fabsf(s), 0.5f));
  ecc = s > 0.0f ? (int)r : (s < 0.0f ? -(int)r : 0);
}

FO_DEVI float safe_scale(float a, bool floor_mode) {
  if (floor_mode) return fmaxf(a, 1e-12f);
  return a > 0.0f ? a : 1.0f;
}
// flashoptim_jax/quantization.py:42-45
FO_DEVI int quant_m(float x, float safe) {
  float n = fdiv(x, safe);
  float t = fdiv(fmul(2.0f, n), fadd(1.0f, fabsf(n)));
  float q = floorf(fadd(fmul(t, 127.0f), 0.5f));
  return (int)fminf(fmaxf(q, -127.0f), 127.0f);
}
// flashoptim_jax/quantization.py:65-67 (root = sqrt(nu) already taken)
FO_DEVI int quant_v(float root, float safe) {
  float t = fdiv(root, safe);
  float q = floorf(fadd(fmul(t, 255.0f), 0.5f));
  return (int)fminf(fmaxf(q, 0.0f), 255.0f);
}

}  // namespace ieee

// ===========================================================================================
namespace fast {

// a / b given y = RN(1/b): product, exact residual, one correction.
FO_DEVI float div_by_rcp(float a, float b, float y) {
  float q0 = fmul(a, y);
  float r = __fmaf_rn(-b, q0, a);
  return __fmaf_rn(r, y, q0);
}

// integer-valued x in [-MAX, MAX] divided by the ECC range
template <int ECC_BITS>
FO_DEVI float ecc_fraction(int ecc) {
  return div_by_rcp((float)ecc, Ecc<ECC_BITS>::MAX, __uint_as_float(Ecc<ECC_BITS>::RCP_BITS));
}

// 2^(log_half_ulp) as a float, from the exponent field of the 16-bit value.
// bf16: field = eb - 8 (needs eb >= 9 to be a normal float); fp16: field = eb + 101, always normal.
template <int PDT>
FO_DEVI float half_ulp(uint32_t bits) {
  using L = Lp<PDT>;
  int eb = (int)((bits & 0x7FFFu) >> L::MANT);
  eb = max(eb, 1);
  int field = eb - L::BIAS - L::MANT - 1 + 127;
  uint32_t sb = field >= 1 ? ((uint32_t)field << 23) : (1u << (22 + field));  // subnormal powers of two for tiny bf16
  return __uint_as_float(sb);
}

template <int PDT, int ECC_BITS>
FO_DEVI float reconstruct(uint32_t bits, int ecc) {
  // one multiplication by an exact power of two (normal or subnormal) rounds exactly as ldexp does
  float err = fmul(ecc_fraction<ECC_BITS>(ecc), half_ulp<PDT>(bits));
  return fadd(Lp<PDT>::to_f32(bits), err);
}

template <int PDT, int ECC_BITS>
FO_DEVI void split(float theta, uint32_t& bits, int& ecc) {
  using L = Lp<PDT>;
  bits = L::from_f32(theta);
  float err = fsub(theta, L::to_f32(bits));
  int eb = max((int)((bits & 0x7FFFu) >> L::MANT), 1);
  int field = 127 - (eb - L::BIAS - L::MANT - 1);  // exponent field of 2^(-log_half_ulp)
  float en;
  if (field <= 254) {
    en = fmul(err, __uint_as_float((uint32_t)field << 23));
  } else {
    // |theta| < 2^-118 (bf16 only): 2^(-ls) overflows a float, scale in two exact steps
    en = fmul(fmul(err, __uint_as_float(254u << 23)), __uint_as_float((uint32_t)(field - 127) << 23));
  }
  float c = fminf(fmaxf(en, -1.0f), 1.0f);
  float s = fmul(c, Ecc<ECC_BITS>::MAX);
  // sign(s)*floor(|s|+0.5) == trunc(s + copysign(0.5, s))
  ecc = __float2int_rz(fadd(s, copysignf(0.5f, s)));
}

// sqrt through MUFU.RSQ and one FMA correction; values the approximation cannot take
// (zero, tiny, huge, inf, nan) go to the IEEE instruction.
FO_DEVI float sqrt_rn(float v) {
  if (!(v >= 1.0e-30f && v <= 1.0e30f)) return v == 0.0f ? v : fsqrt(v);
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(v));
  float r = fmul(v, y);
  float h = fmul(0.5f, y);
  float e = __fmaf_rn(-r, r, v);
  return __fmaf_rn(e, h, r);
}

// code of the soft-sign transform: floor(127 * (2n / (1 + |n|)) + 0.5) for |n| <= 1
FO_DEVI int softsign_code(float n) {
  float d = fadd(1.0f, fabsf(n));
  float a = fadd(n, n);
  float y0;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y0) : "f"(d));
  float e = __fmaf_rn(-d, y0, 1.0f);
  float y = __fmaf_rn(e, y0, y0);
  float q0 = fmul(a, y);
  float r = __fmaf_rn(-d, q0, a);
  float t = __fmaf_rn(r, y, q0);
  return __float2int_rd(fadd(fmul(t, 127.0f), 0.5f));
}

// per-group quantizer state: the scale guard, its reciprocal and whether the shortcut is safe
struct GroupScale {
  float safe, rcp;
  bool tame;
};
FO_DEVI GroupScale group_scale(float absmax, bool floor_mode) {
  GroupScale g;
  g.safe = ieee::safe_scale(absmax, floor_mode);
  g.tame = g.safe >= 1.0e-30f && g.safe <= 1.0e30f;
  g.rcp = __frcp_rn(g.safe);
  return g;
}
FO_DEVI int quant_m(float x, const GroupScale& g) {
  if (!g.tame) return ieee::quant_m(x, g.safe);
  return softsign_code(div_by_rcp(x, g.safe, g.rcp));
}
FO_DEVI int quant_v(float root, const GroupScale& g) {
  if (!g.tame) return ieee::quant_v(root, g.safe);
  float t = div_by_rcp(root, g.safe, g.rcp);
  return __float2int_rd(fadd(fmul(t, 255.0f), 0.5f));
}

}  // namespace fast

#ifdef FO_NAIVE_MATH
namespace M = ieee;
#else
namespace M = fast;
#endif

}  // namespace fo
