/*
 * CPU oracle, C restatement (TEST INFRASTRUCTURE ONLY — never linked into the product).
 *
 * Same arithmetic as oracle/flashoptim_oracle.py, written as scalar loops over
 * quantization groups so that multi-gigabyte leaves finish in seconds and so that
 * the benchmark has a multi-threaded CPU baseline.  It is validated bit-for-bit
 * against the NumPy oracle by the CPU test-suite, and it reproduces bit for bit the
 * golden vectors that tests/golden/make_golden.py records from the reference's own
 * source files (imported unmodified over a NumPy stand-in for jax; JAX itself is not
 * installable where this was written).
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp).
 * Every fp32 operation below is a single IEEE operation; -ffp-contract=off keeps
 * the compiler from fusing a*b+c.
 *
 * Reference lines restated (paths inside the reference project):
 *   flashoptim_jax/quantization.py:15-77     codecs
 *   flashoptim_jax/utils.py:499-557          ECC split / reconstruct
 *   flashoptim_jax/adamw.py:356-423,463      unfused Adam/AdamW leaf
 *   flashoptim_jax/adamw.py:76-131           fused kernel text
 *   flashoptim_jax/lion.py:18-70             unfused Lion leaf
 *   flashoptim_jax/sgd.py:18-77              unfused SGD leaf
 *   flashoptim_jax/momentum_kernel.py:74-103 fused Lion/SGD kernel text
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORC_F32 = 0, ORC_BF16 = 1, ORC_F16 = 2 };
enum { ORC_ADAM = 0, ORC_LION = 1, ORC_SGD = 2 };
enum { ORC_STATE_QUANT = 0, ORC_STATE_FULL = 1, ORC_STATE_NONE = 2 };
enum {
  ORC_FLAG_DECOUPLED = 1,   /* AdamW / SGDW / Lion: theta *= 1 - lr*wd */
  ORC_FLAG_NESTEROV = 2,
  ORC_FLAG_LION_LERP = 4,   /* lion.py:50-52 form */
  ORC_FLAG_LP_DELTA = 8,    /* adamw.py:411,463: param + lp(new - param) */
  ORC_FLAG_SCALE_FLOOR = 16 /* adamw.py:121: max(absmax, 1e-12) */
};

typedef struct {
  float lr, wd;
  float b1, b2;             /* Adam betas | Lion b1,b2 | SGD: b1 = momentum, b2 unused */
  float omb1, omb2;         /* (1-b1), (1-b2) as the caller's convention forms them | SGD: omb1 = 1 - dampening */
  float eps, bc1, bc2;
} OrcHyper;

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0) {
    /* zero or subnormal: value = m * 2^-24, exact in fp32 */
    float v = (float)m * 5.9604644775390625e-08f;
    return u2f(f2u(v) | sign);
  }
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}
static inline uint16_t f32_to_f16(float f) {
  uint32_t u = f2u(f);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  u &= 0x7FFFFFFFu;
  if (u > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
  if (u >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536 (65520..65536 handled by carry below) */
  if (u < 0x38800000u) {
    /* below the smallest normal half: let the FPU round to a multiple of 2^-24 */
    float a = u2f(u) + 0.5f; /* 0.5f has ulp 2^-24 in [0.5,1) */
    return (uint16_t)(sign | (uint16_t)(f2u(a) - 0x3F000000u));
  }
  uint32_t odd = (u >> 13) & 1u;
  u += 0xC8000FFFu; /* rebias exponent by -112 and add rounding bias 0xFFF */
  u += odd;
  return (uint16_t)(sign | (uint16_t)(u >> 13));
}

static inline float load_fp(const void* p, int dt, uint64_t i) {
  if (dt == ORC_F32) return ((const float*)p)[i];
  if (dt == ORC_BF16) return bf16_to_f32(((const uint16_t*)p)[i]);
  return f16_to_f32(((const uint16_t*)p)[i]);
}

/* exponent of half an ULP of a low-precision value (utils.py:504-518) */
static inline int log_half_ulp(uint16_t bits, int dt) {
  int mant = dt == ORC_BF16 ? 7 : 10;
  int emin = dt == ORC_BF16 ? -126 : -14;
  int eb = (bits & 0x7FFF) >> mant;
  int e = eb == 0 ? emin : eb - (1 - emin);
  return e - mant - 1;
}

/* utils.py:521-536 */
static inline float reconstruct_one(uint16_t lpbits, int pdt, int ecc, float ecc_max) {
  float lp = pdt == ORC_BF16 ? bf16_to_f32(lpbits) : f16_to_f32(lpbits);
  float corr = (float)ecc / ecc_max;
  float err = ldexpf(corr, log_half_ulp(lpbits, pdt));
  return lp + err;
}

/* utils.py:539-557 */
static inline void split_one(float theta, int pdt, float ecc_max, uint16_t* lp_out, int* ecc_out) {
  uint16_t lpb = pdt == ORC_BF16 ? f32_to_bf16(theta) : f32_to_f16(theta);
  float lp = pdt == ORC_BF16 ? bf16_to_f32(lpb) : f16_to_f32(lpb);
  float err = theta - lp;
  float en = ldexpf(err, -log_half_ulp(lpb, pdt));
  float c = en < -1.0f ? -1.0f : (en > 1.0f ? 1.0f : en);
  float s = c * ecc_max;
  float r = floorf(fabsf(s) + 0.5f);
  *lp_out = lpb;
  *ecc_out = s > 0.0f ? (int)r : (s < 0.0f ? -(int)r : 0);
}

static inline float deq_m(int q, float scale) {
  float t = (float)q / 127.0f;
  float nrm = t / (2.0f - fabsf(t));
  return nrm * scale;
}
static inline float deq_v(int q, float scale) {
  float t = (float)q / 255.0f;
  float s = t * scale;
  return s * s;
}
static inline float safe_scale(float a, int flags) {
  if (flags & ORC_FLAG_SCALE_FLOOR) return a > 1e-12f ? a : 1e-12f;
  return a > 0.0f ? a : 1.0f;
}
static inline int quant_m(float x, float safe) {
  float nrm = x / safe;
  float t = (2.0f * nrm) / (1.0f + fabsf(nrm));
  float q = floorf(t * 127.0f + 0.5f);
  q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
  return (int)q;
}
static inline int quant_v(float root, float safe) {
  float t = root / safe;
  float q = floorf(t * 255.0f + 0.5f);
  q = q < 0.0f ? 0.0f : (q > 255.0f ? 255.0f : q);
  return (int)q;
}
static inline float signf(float x) { return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x); }

/* ---- standalone codecs (group-parallel) --------------------------------- */

int orc_quantize_momentum(const float* x, int8_t* values, uint16_t* scales, uint64_t n, int g, int flags) {
  int64_t G = (int64_t)((n + g - 1) / g);
#pragma omp parallel for schedule(static)
  for (int64_t gi = 0; gi < G; ++gi) {
    uint64_t lo = (uint64_t)gi * g, hi = lo + g < n ? lo + g : n;
    float a = 0.0f;
    for (uint64_t i = lo; i < hi; ++i) a = fmaxf(a, fabsf(x[i]));
    float safe = safe_scale(a, flags);
    for (uint64_t i = lo; i < hi; ++i) values[i] = (int8_t)quant_m(x[i], safe);
    scales[gi] = f32_to_f16(a);
  }
  return 0;
}
int orc_dequantize_momentum(const int8_t* values, const uint16_t* scales, float* out, uint64_t n, int g) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = deq_m(values[i], f16_to_f32(scales[i / g]));
  return 0;
}
int orc_quantize_variance(const float* x, uint8_t* values, uint16_t* scales, uint64_t n, int g, int flags) {
  int64_t G = (int64_t)((n + g - 1) / g);
#pragma omp parallel for schedule(static)
  for (int64_t gi = 0; gi < G; ++gi) {
    uint64_t lo = (uint64_t)gi * g, hi = lo + g < n ? lo + g : n;
    float a = 0.0f;
    for (uint64_t i = lo; i < hi; ++i) a = fmaxf(a, sqrtf(x[i]));
    float safe = safe_scale(a, flags);
    for (uint64_t i = lo; i < hi; ++i) values[i] = (uint8_t)quant_v(sqrtf(x[i]), safe);
    scales[gi] = f32_to_f16(a);
  }
  return 0;
}
int orc_dequantize_variance(const uint8_t* values, const uint16_t* scales, float* out, uint64_t n, int g) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = deq_v(values[i], f16_to_f32(scales[i / g]));
  return 0;
}
int orc_split(const float* theta, uint16_t* lp, void* ecc, int pdt, int ecc_bits, uint64_t n) {
  float ecc_max = ecc_bits == 8 ? 127.0f : 32767.0f;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    if (ecc_bits == 0) {
      lp[i] = pdt == ORC_BF16 ? f32_to_bf16(theta[i]) : f32_to_f16(theta[i]);
      continue;
    }
    int e;
    split_one(theta[i], pdt, ecc_max, &lp[i], &e);
    if (ecc_bits == 8) ((int8_t*)ecc)[i] = (int8_t)e; else ((int16_t*)ecc)[i] = (int16_t)e;
  }
  return 0;
}
int orc_reconstruct(const uint16_t* lp, const void* ecc, float* theta, int pdt, int ecc_bits, uint64_t n) {
  float ecc_max = ecc_bits == 8 ? 127.0f : 32767.0f;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    if (ecc_bits == 0) { theta[i] = pdt == ORC_BF16 ? bf16_to_f32(lp[i]) : f16_to_f32(lp[i]); continue; }
    int e = ecc_bits == 8 ? (int)((const int8_t*)ecc)[i] : (int)((const int16_t*)ecc)[i];
    theta[i] = reconstruct_one(lp[i], pdt, e, ecc_max);
  }
  return 0;
}

/* ---- fused-in-place leaf step -------------------------------------------- */

#define ORC_MAX_GROUP 1024

/*
 * One optimizer step over one leaf, in place.  mu/nu are int8/uint8 codes with fp16
 * scales (state == QUANT), fp32 arrays (FULL) or absent (NONE, SGD without momentum).
 * ecc_bits 0 means the leaf carries no ECC (ecc may be NULL).  Returns 0, or -1 on
 * an unsupported argument.
 */
int orc_step_leaf(int opt, const void* grad, int gdt, void* param, int pdt, void* ecc, int ecc_bits,
                  void* mu, uint16_t* mu_scales, void* nu, uint16_t* nu_scales, int state,
                  uint64_t n, int g, const OrcHyper* hp, int flags) {
  if (g <= 0 || g > ORC_MAX_GROUP) return -1;
  if (pdt == ORC_F32 && ecc_bits != 0) return -1;
  if (state != ORC_STATE_QUANT) g = 32; /* grouping is irrelevant without codes */
  const OrcHyper h = *hp;
  const float ecc_max = ecc_bits == 8 ? 127.0f : 32767.0f;
  const float decay = 1.0f - h.lr * h.wd;
  const float lr_bc1 = h.lr / h.bc1;
  const float sqrt_bc2 = sqrtf(h.bc2);
  int64_t G = (int64_t)((n + g - 1) / g);
#pragma omp parallel for schedule(static)
  for (int64_t gi = 0; gi < G; ++gi) {
    uint64_t lo = (uint64_t)gi * g, hi = lo + g < n ? lo + g : n;
    float mbuf[ORC_MAX_GROUP], rbuf[ORC_MAX_GROUP];
    float msc = 0.0f, vsc = 0.0f;
    if (state == ORC_STATE_QUANT) {
      msc = f16_to_f32(mu_scales[gi]);
      if (opt == ORC_ADAM) vsc = f16_to_f32(nu_scales[gi]);
    }
    float m_abs = 0.0f, r_max = 0.0f;
    for (uint64_t i = lo; i < hi; ++i) {
      float gr = load_fp(grad, gdt, i);
      uint16_t lpb = 0;
      float theta;
      if (pdt == ORC_F32) theta = ((float*)param)[i];
      else {
        lpb = ((uint16_t*)param)[i];
        if (ecc_bits) {
          int e = ecc_bits == 8 ? (int)((int8_t*)ecc)[i] : (int)((int16_t*)ecc)[i];
          theta = reconstruct_one(lpb, pdt, e, ecc_max);
        } else theta = pdt == ORC_BF16 ? bf16_to_f32(lpb) : f16_to_f32(lpb);
      }
      float m = 0.0f, v = 0.0f, root = 0.0f;
      if (state == ORC_STATE_QUANT) {
        m = deq_m(((int8_t*)mu)[i], msc);
        if (opt == ORC_ADAM) v = deq_v(((uint8_t*)nu)[i], vsc);
      } else if (state == ORC_STATE_FULL) {
        m = ((float*)mu)[i];
        if (opt == ORC_ADAM) v = ((float*)nu)[i];
      }
      float nt;
      if (opt == ORC_ADAM) {
        if (!(flags & ORC_FLAG_DECOUPLED)) gr = gr + h.wd * theta;
        m = h.b1 * m + h.omb1 * gr;
        v = h.b2 * v + h.omb2 * (gr * gr);
        if (flags & ORC_FLAG_DECOUPLED) theta = theta * decay;
        root = sqrtf(v);
        nt = theta - (lr_bc1 * m) / (root / sqrt_bc2 + h.eps);
      } else if (opt == ORC_LION) {
        float upd;
        if (flags & ORC_FLAG_LION_LERP) {
          float d = gr - m;
          upd = signf(m + h.omb1 * d);
          m = m + h.omb2 * d;
        } else {
          upd = signf(h.b1 * m + h.omb1 * gr);
          m = h.b2 * m + h.omb2 * gr;
        }
        theta = theta * decay;
        nt = theta - h.lr * upd;
      } else {
        if (!(flags & ORC_FLAG_DECOUPLED)) gr = gr + h.wd * theta;
        float dir = gr;
        if (state != ORC_STATE_NONE) {
          m = h.b1 * m + h.omb1 * gr;
          dir = (flags & ORC_FLAG_NESTEROV) ? gr + h.b1 * m : m;
        }
        if (flags & ORC_FLAG_DECOUPLED) theta = theta * decay;
        nt = theta - h.lr * dir;
      }
      /* write param (+ECC) */
      if (pdt == ORC_F32) {
        if (flags & ORC_FLAG_LP_DELTA) {
          float oldf = ((float*)param)[i];
          float d = nt - oldf;
          nt = oldf + d;
        }
        ((float*)param)[i] = nt;
      } else {
        uint16_t nlp;
        if (ecc_bits) {
          int e;
          split_one(nt, pdt, ecc_max, &nlp, &e);
          if (ecc_bits == 8) ((int8_t*)ecc)[i] = (int8_t)e; else ((int16_t*)ecc)[i] = (int16_t)e;
        } else nlp = pdt == ORC_BF16 ? f32_to_bf16(nt) : f32_to_f16(nt);
        if (flags & ORC_FLAG_LP_DELTA) {
          float oldf = pdt == ORC_BF16 ? bf16_to_f32(lpb) : f16_to_f32(lpb);
          float newf = pdt == ORC_BF16 ? bf16_to_f32(nlp) : f16_to_f32(nlp);
          float d = newf - oldf;
          uint16_t db = pdt == ORC_BF16 ? f32_to_bf16(d) : f32_to_f16(d);
          float df = pdt == ORC_BF16 ? bf16_to_f32(db) : f16_to_f32(db);
          float s = oldf + df;
          nlp = pdt == ORC_BF16 ? f32_to_bf16(s) : f32_to_f16(s);
        }
        ((uint16_t*)param)[i] = nlp;
      }
      /* state */
      if (state == ORC_STATE_FULL) {
        ((float*)mu)[i] = m;
        if (opt == ORC_ADAM) ((float*)nu)[i] = v;
      } else if (state == ORC_STATE_QUANT) {
        mbuf[i - lo] = m;
        m_abs = fmaxf(m_abs, fabsf(m));
        if (opt == ORC_ADAM) { rbuf[i - lo] = root; r_max = fmaxf(r_max, root); }
      }
    }
    if (state == ORC_STATE_QUANT) {
      float ms = safe_scale(m_abs, flags);
      for (uint64_t i = lo; i < hi; ++i) ((int8_t*)mu)[i] = (int8_t)quant_m(mbuf[i - lo], ms);
      mu_scales[gi] = f32_to_f16(m_abs);
      if (opt == ORC_ADAM) {
        float vs = safe_scale(r_max, flags);
        for (uint64_t i = lo; i < hi; ++i) ((uint8_t*)nu)[i] = (uint8_t)quant_v(rbuf[i - lo], vs);
        nu_scales[gi] = f32_to_f16(r_max);
      }
    }
  }
  return 0;
}

int orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}
