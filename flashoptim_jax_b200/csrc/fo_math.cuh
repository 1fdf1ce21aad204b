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

// RN(1/s) for s in [1e-30, 1e30]: MUFU.RCP and FO_RCP_STEPS correction steps, no range
// checks.  Compared with the IEEE reciprocal over every float of that range by fo_selftest.
#ifndef FO_RCP_STEPS
#define FO_RCP_STEPS 1
#endif
template <int STEPS>
FO_DEVI float rcp_steps(float s) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(s));
#pragma unroll
  for (int k = 0; k < STEPS; ++k) {
    float e = __fmaf_rn(-s, y, 1.0f);
    y = __fmaf_rn(e, y, y);
  }
  return y;
}
FO_DEVI float rcp_rn(float s) {
#if FO_RCP_STEPS == 0
  return __frcp_rn(s);
#else
  return rcp_steps<FO_RCP_STEPS>(s);
#endif
}

// integer-valued x in [-MAX, MAX] divided by the ECC range
template <int ECC_BITS>
FO_DEVI float ecc_fraction_f(float x) {
  return div_by_rcp(x, Ecc<ECC_BITS>::MAX, __uint_as_float(Ecc<ECC_BITS>::RCP_BITS));
}
template <int ECC_BITS>
FO_DEVI float ecc_fraction(int ecc) {
  return ecc_fraction_f<ECC_BITS>((float)ecc);
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

// sign(s)*floor(|s|+0.5) for |s| <= 32767, as an integer: trunc(s + copysign(0.5, s))
FO_DEVI int round_half_away(float s) { return __float2int_rz(fadd(s, copysignf(0.5f, s))); }

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
  ecc = round_half_away(fmul(c, Ecc<ECC_BITS>::MAX));
}

// ---- the same two conversions for values already known to be "ordinary" -------------------
// Given the fp32 image lpf of a 16-bit value with |lpf| >= kOrdinaryMin<PDT>: 2^ls and 2^-ls
// by exponent-field arithmetic.  fp16 has no small-value exception once the field is clamped
// to the smallest normal half (zero and subnormal halves use the min normal exponent).
template <int PDT>
struct Ordinary;
template <>
struct Ordinary<FO_BF16> {
  static constexpr float kMin = 7.8886091e-31f;  // 2^-100: below it 2^ls, 2^-ls or MAX*2^-ls stops being a normal float
  static FO_DEVI uint32_t ebits(float lpf) { return __float_as_uint(lpf) & 0x7F800000u; }
  static FO_DEVI float ulp_half(uint32_t eb) { return __uint_as_float(eb - (8u << 23)); }
  static FO_DEVI float ulp_half_inv(uint32_t eb) { return __uint_as_float((262u << 23) - eb); }
};
template <>
struct Ordinary<FO_F16> {
  static constexpr float kMin = 0.0f;
  static FO_DEVI uint32_t ebits(float lpf) { return max(__float_as_uint(lpf) & 0x7F800000u, 113u << 23); }
  static FO_DEVI float ulp_half(uint32_t eb) { return __uint_as_float(eb - (11u << 23)); }
  static FO_DEVI float ulp_half_inv(uint32_t eb) { return __uint_as_float((265u << 23) - eb); }
};

template <int PDT, int ECC_BITS>
FO_DEVI float reconstruct_ordinary(float lpf, float ecc_as_float) {
  const uint32_t eb = Ordinary<PDT>::ebits(lpf);
  return fadd(lpf, fmul(ecc_fraction_f<ECC_BITS>(ecc_as_float), Ordinary<PDT>::ulp_half(eb)));
}
// lpf is RN_lp(theta) already converted back to fp32
template <int PDT, int ECC_BITS>
FO_DEVI int ecc_ordinary(float theta, float lpf) {
  const uint32_t eb = Ordinary<PDT>::ebits(lpf);
  float en = fmul(fsub(theta, lpf), Ordinary<PDT>::ulp_half_inv(eb));
  float a = fminf(fabsf(en), 1.0f);
  float s = copysignf(fmul(a, Ecc<ECC_BITS>::MAX), en);
  return round_half_away(s);
}

// sqrt through MUFU.RSQ and one FMA correction, for 1e-30 <= v < inf
FO_DEVI float sqrt_core(float v) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(v));
  float r = fmul(v, y);
  float h = fmul(0.5f, y);
  float e = __fmaf_rn(-r, r, v);
  return __fmaf_rn(e, h, r);
}
FO_DEVI float sqrt_rn(float v) {
  if (!(v >= 1.0e-30f)) return fsqrt(v);
  return sqrt_core(v);
}

// floor(y) for |y| < 2^22 as the low bits of a float: adding 1.5*2^23 rounding down leaves
// 0x400000 + floor(y) in the mantissa, so the low byte is floor(y) in two's complement.
FO_DEVI uint32_t floor_bits(float y) { return __float_as_uint(__fadd_rd(y, 12582912.0f)); }

// soft-sign transform 2n / (1 + |n|) for |n| <= 1 through MUFU.RCP, one Newton step and a
// residual correction; only the resulting int8 code has to match the IEEE division.
FO_DEVI float softsign_t(float n) {
  float d = fadd(1.0f, fabsf(n));
  float a = fadd(n, n);
  float y = rcp_steps<1>(d);
  float q0 = fmul(a, y);
  float r = __fmaf_rn(-d, q0, a);
  return __fmaf_rn(r, y, q0);
}
// low byte = floor(127 t + 0.5) in two's complement
FO_DEVI uint32_t softsign_code_bits(float n) { return floor_bits(fadd(fmul(softsign_t(n), 127.0f), 0.5f)); }
FO_DEVI int softsign_code(float n) { return (int)(signed char)(softsign_code_bits(n) & 0xFFu); }

// per-group quantizer state: the scale guard, its reciprocal and whether the shortcut is safe
struct GroupScale {
  float safe, rcp;
  bool tame;
};
FO_DEVI GroupScale group_scale(float absmax, bool floor_mode) {
  GroupScale g;
  g.tame = absmax >= 1.0e-12f && absmax <= 1.0e30f;  // above both guards' thresholds: safe == absmax
  g.safe = g.tame ? absmax : ieee::safe_scale(absmax, floor_mode);
  g.rcp = g.tame ? rcp_rn(absmax) : 0.0f;
  return g;
}
FO_DEVI int quant_m(float x, const GroupScale& g) {
  if (!g.tame) return ieee::quant_m(x, g.safe);
  return softsign_code(div_by_rcp(x, g.safe, g.rcp));
}
FO_DEVI uint32_t quant_v_bits(float root, float safe, float rcp) {
  return floor_bits(fadd(fmul(div_by_rcp(root, safe, rcp), 255.0f), 0.5f));
}
FO_DEVI int quant_v(float root, const GroupScale& g) {
  if (!g.tame) return ieee::quant_v(root, g.safe);
  return (int)(quant_v_bits(root, g.safe, g.rcp) & 0xFFu);
}

}  // namespace fast

// ===========================================================================================
// fast2: the same shortcuts on pairs of elements with the sm_100 packed fp32x2 instructions
// (add / mul / fma .f32x2: two independent IEEE operations per issue slot).  One pair is two
// neighbouring elements of a leaf.  Every function here has a scalar twin above with the
// same operation sequence per component, so results are bit-identical to fast:: and hence
// to ieee::; fo_selftest sweeps these packed forms.
namespace fast2 {

using f2 = float2;
FO_DEVI f2 mk(float a, float b) { return make_float2(a, b); }
FO_DEVI f2 sp(float a) { return make_float2(a, a); }
// Inline PTX with explicit rounding modifiers: an operation that names its rounding mode is
// never merged into an fma.  (The __fmul2_rn / __fadd2_rn intrinsics were observed to be
// contracted into fma.f32x2 even under -fmad=false, which changes last bits.)
FO_DEVI unsigned long long as_b64(f2 a) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a.x), "f"(a.y));
  return r;
}
FO_DEVI f2 as_f2(unsigned long long r) {
  f2 a;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a.x), "=f"(a.y) : "l"(r));
  return a;
}
FO_DEVI f2 mul2(f2 a, f2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(as_b64(a)), "l"(as_b64(b)));
  return as_f2(d);
}
FO_DEVI f2 add2(f2 a, f2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(as_b64(a)), "l"(as_b64(b)));
  return as_f2(d);
}
FO_DEVI f2 fma2(f2 a, f2 b, f2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(as_b64(a)), "l"(as_b64(b)), "l"(as_b64(c)));
  return as_f2(d);
}
// x + y where x and/or y are themselves products.  The assembler was observed to contract
// mul.rn.f32x2 followed by add.rn.f32x2 into one fma.f32x2 (and to simplify x*1 first), which
// changes last bits.  Writing the sum as x*one + y with `one` a run-time 1.0f it cannot see
// through keeps both roundings: a product of three factors is not an fma, and neither is an
// fma whose addend is a product.  RN(x*1 + y) == RN(x + y).
FO_DEVI f2 sum2(f2 x, f2 y, f2 one) { return fma2(x, one, y); }
FO_DEVI f2 add2_rd(f2 a, f2 b) {
  unsigned long long d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(as_b64(a)), "l"(as_b64(b)));
  return as_f2(d);
}

FO_DEVI float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
FO_DEVI float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed operations take no negated operands, and a packed negation is a whole instruction.
// The sequences below therefore carry signs through their intermediate values (rounding to
// nearest is symmetric: RN(-x) == -RN(x)), so that every residual a - b*q is formed as an fma
// of operands that already have the right signs.  Scalar negations feeding a special-function
// unit are free (source modifier).

// a / b given nb = -b and y = RN(1/b)
FO_DEVI f2 div_by_rcp2(f2 a, f2 nb, f2 y) {
  f2 q0 = mul2(a, y);
  f2 r = fma2(nb, q0, a);
  return fma2(r, y, q0);
}
// a / b given na = -a, b and ny = -RN(1/b)
FO_DEVI f2 div_negnum_by_rcp2(f2 na, f2 b, f2 ny) {
  f2 q0 = mul2(na, ny);      // a*y
  f2 nr = fma2(b, q0, na);   // b*q0 - a = -(a - b*q0)
  return fma2(nr, ny, q0);   // q0 + (a - b*q0)*y
}

// -RN(1/d) per component for d in [1e-30, 1e30]
FO_DEVI f2 neg_rcp2(f2 d) {
  f2 ny0 = mk(rcp_approx(-d.x), rcp_approx(-d.y));
  f2 e = fma2(d, ny0, sp(1.0f));  // 1 - d*y0
  return fma2(e, ny0, ny0);       // -(y0 + e*y0)
}

// RN(-a/d) per component, proven: y = RN(1/d) (checked exhaustively), first correction
// gives a faithful quotient, the second the correctly rounded one (Markstein).  Needs
// d in [1e-12, 2^47], |a| in [2^-70, 2^60] (so |a/d| stays a normal number and both residuals are exact).
FO_DEVI f2 neg_div2(f2 a, f2 d) {
  f2 ny = neg_rcp2(d);
  f2 q = mul2(a, ny);        // -a*y
  f2 nr = fma2(d, q, a);     // a + d*q = -((-a) - d*q)
  q = fma2(nr, ny, q);
  nr = fma2(d, q, a);
  return fma2(nr, ny, q);
}

// -sqrt(v) per component given nv = -v, for 1e-30 <= v < inf
FO_DEVI f2 neg_sqrt_core2(f2 nv) {
  f2 y = mk(rsqrt_approx(-nv.x), rsqrt_approx(-nv.y));
  f2 nr = mul2(nv, y);        // -r, r = v*y
  f2 h = mul2(y, sp(0.5f));
  f2 ne = fma2(nr, nr, nv);   // r*r - v
  return fma2(ne, h, nr);     // -(r + (v - r*r)*h)
}

// power-of-two scales folded into the ECC constants: the fraction comes out pre-multiplied by
// 2^-(MANT+1), so 2^log_half_ulp is just the exponent field of the stored value
template <int PDT, int ECC_BITS>
struct EccConst {
  static constexpr float kFold = PDT == FO_BF16 ? 256.0f : 2048.0f;           // 2^(MANT+1)
  // 1/MAX as an unevaluated sum hi + lo of two floats, both times 2^-(MANT+1) (exact scalings).
  // 1/127 and 1/32767 have periodic binary expansions, so lo is hi shifted down by 28 resp. 30 bits.
  static FO_DEVI float rcp_hi() { return __uint_as_float(Ecc<ECC_BITS>::RCP_BITS) * (1.0f / kFold); }
  static FO_DEVI float rcp_lo() { return rcp_hi() * (ECC_BITS == 8 ? 3.7252902984619140625e-9f : 9.31322574615478515625e-10f); }
};
template <int PDT>
FO_DEVI uint32_t exp_field(float lpf) {
  uint32_t eb = __float_as_uint(lpf) & 0x7F800000u;
  if constexpr (PDT == FO_F16) eb = max(eb, 113u << 23);  // zero / subnormal halves use the min normal exponent
  return eb;
}
// master weight from (stored value as fp32, ECC as fp32) for ordinary values (see fast::Ordinary)
template <int PDT, int ECC_BITS>
FO_DEVI f2 reconstruct_ordinary2(f2 lpf, f2 ef, f2 one) {
  using K = EccConst<PDT, ECC_BITS>;
  // RN(e / MAX) for every integer e of the ECC type: e*hi + RN(e*lo) carries the quotient to
  // about 2^-48, which no e/MAX comes that close to a rounding boundary without being exact
  // (all 2^ECC_BITS values are compared with the IEEE division by the self-test)
  f2 fr = fma2(ef, sp(K::rcp_hi()), mul2(ef, sp(K::rcp_lo())));
  f2 sc = mk(__uint_as_float(exp_field<PDT>(lpf.x)), __uint_as_float(exp_field<PDT>(lpf.y)));
  return sum2(mul2(fr, sc), lpf, one);
}
// 2^(1 - exponent of lpf) as float bits: the inverted exponent field (one logic operation)
template <int PDT>
FO_DEVI uint32_t inv_exp_field(float lpf) {
  uint32_t ib = ~__float_as_uint(lpf) & 0x7F800000u;
  if constexpr (PDT == FO_F16) ib = min(ib, 142u << 23);  // zero / subnormal halves use the min normal exponent
  return ib;
}
// ECC of theta given lpf = RN_lp(theta) as fp32, for kMin <= |lpf| <= 1e38 (see fast::Ordinary):
// err * 2^-log_half_ulp * MAX, |.| <= MAX without clipping because |err| is at most half an ULP of lpf
template <int PDT, int ECC_BITS>
FO_DEVI void ecc_ordinary2(f2 theta, f2 lpf, int& e0, int& e1) {
  constexpr float kC = Ecc<ECC_BITS>::MAX * (PDT == FO_BF16 ? 128.0f : 1024.0f);  // MAX * 2^MANT, exact
  f2 err = fma2(lpf, sp(-1.0f), theta);
  f2 sc = mk(__uint_as_float(inv_exp_field<PDT>(lpf.x)), __uint_as_float(inv_exp_field<PDT>(lpf.y)));
  f2 s = mul2(mul2(err, sc), sp(kC));  // the first product is exact (a power of two, no underflow: err is a multiple of theta's ULP)
  f2 y = add2(s, mk(copysignf(0.5f, s.x), copysignf(0.5f, s.y)));  // round half away from zero ...
  e0 = __float2int_rz(y.x);                                        // ... by truncation
  e1 = __float2int_rz(y.y);
}

// RN(c/255) for the codes c in bytes b and b+1 of w (flashoptim_jax/quantization.py:74), without a
// table: the byte goes into the mantissa of 2^23, which is then subtracted; c*hi + RN(c*lo) with
// hi + lo = 1/255 to 2^-48 equals RN(c/255) for all 256 codes (compared with the IEEE division
// by the self-test).
FO_DEVI f2 codes_over_255(uint32_t w, int b) {
  f2 cf = add2(mk(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (uint32_t)b)),
                  __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (uint32_t)(b + 1)))),
               sp(-8388608.0f));
  return fma2(cf, sp(__uint_as_float(0x3B808081u)), mul2(cf, sp(__uint_as_float(0xAF7EFEFFu))));
}

// bits whose low byte is floor(127 * 2n/(1+|n|) + 0.5), |n| <= 1
FO_DEVI void softsign_code_bits2(f2 n, f2 one, uint32_t& c0, uint32_t& c1) {
  f2 d = add2(mk(fabsf(n.x), fabsf(n.y)), sp(1.0f));
  f2 ny = neg_rcp2(d);
  f2 nq0 = mul2(n, ny);
  f2 r = fma2(d, nq0, n);                      // n - d*q0
  f2 nq = fma2(r, ny, nq0);                    // -n/(1+|n|); 2n/(1+|n|) * 127 == nq * -254 exactly
  f2 c = sum2(mul2(nq, sp(-254.0f)), sp(0.5f), one);
  f2 fl = add2_rd(c, sp(12582912.0f));
  c0 = __float_as_uint(fl.x);
  c1 = __float_as_uint(fl.y);
}
// bits whose low byte is floor(255 * root/av + 0.5); nroot = -root, nrcp = -RN(1/av)
FO_DEVI void quant_v_bits2(f2 nroot, f2 av, f2 nrcp, f2 one, uint32_t& c0, uint32_t& c1) {
  f2 t = div_negnum_by_rcp2(nroot, av, nrcp);
  f2 c = sum2(mul2(t, sp(255.0f)), sp(0.5f), one);
  f2 fl = add2_rd(c, sp(12582912.0f));
  c0 = __float_as_uint(fl.x);
  c1 = __float_as_uint(fl.y);
}

}  // namespace fast2

}  // namespace fo
