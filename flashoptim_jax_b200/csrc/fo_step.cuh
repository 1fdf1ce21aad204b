// Multi-tensor fused optimizer step for sm_100a.
//
// One launch walks a table of pytree leaves.  The leaves are cut into chunks of 2048
// elements; a persistent grid of blocks strides over the chunk list.  Inside a chunk a
// thread owns 8 consecutive elements, so every warp-wide access is a run of 256
// consecutive elements: 16 B per lane for the 2-byte streams (grad, param, int16 ECC), 8 B
// per lane for the 1-byte streams (int8/uint8 codes, int8 ECC).  A 32-element quantization
// group is 4 adjacent lanes; its absmax is two xor-shuffles.  Everything between load and
// store lives in registers: reconstruct the fp32 master weight, dequantize the moments,
// apply the update, split the weight back, requantize with fresh group scales.  All arrays
// are updated in place; a group is read and written by the same 4 lanes only.
//
// Two code paths produce the same bits:
//   hot   full, 16-byte-aligned chunks under ordinary hyper-parameters: vector accesses and
//         the fast:: arithmetic of fo_math.cuh, with per-piece checks that send unusual
//         values (|param| < 2^-118, second moment < 1e-30, group scale outside
//         [1e-12, 1e30]) to the IEEE formulation;
//   cold  everything else (leaf tails, unaligned leaves, eps or bias correction outside the
//         range the shortcut division is proven for): scalar guarded accesses and ieee::
//         arithmetic only.
//
// The arithmetic follows flashoptim_jax/adamw.py:76-131 and
// flashoptim_jax/momentum_kernel.py:62-103 operation by operation (see fo_math.cuh).
#pragma once

#include <cuda_runtime.h>

#include "fo_math.cuh"

namespace fo {

#ifndef FO_THREADS
#define FO_THREADS 256
#endif
#ifndef FO_MIN_BLOCKS
#define FO_MIN_BLOCKS 3
#endif
constexpr int kThreads = FO_THREADS;
constexpr int kPiece = 8;
constexpr int kChunk = kThreads * kPiece;      // elements per chunk
constexpr int kMaxLeaves = 320;                // leaves per launch (kernel-parameter table)
constexpr int kGenericTile = 1024;             // slots per block of the any-group-size kernel
constexpr uint32_t kFlagTameAdam = 1u << 31;   // internal: sqrt(nu)/sqrt(bc2) may use the reciprocal shortcut

struct DevLeaf {
  const void* grad;
  void* param;
  void* ecc;
  void* mu;
  void* mu_scales;
  void* nu;
  void* nu_scales;
  unsigned long long n;
};

struct DevHyper {
  float lr, wd, b1, b2, omb1, omb2, eps, bc1, bc2;
  // derived on the host with the same IEEE fp32 operations the kernel would use
  float decay, lr_bc1, sqrt_bc2, rcp_sqrt_bc2;
  uint32_t flags;
  const float* dyn;  // optional device {lr, bc1, bc2}
};

struct StepParams {
  DevLeaf leaf[kMaxLeaves];
  uint32_t first_block[kMaxLeaves + 1];  // first chunk of each leaf; [n_leaves] = total chunks
  uint8_t hyper_of[kMaxLeaves];
  uint8_t aligned[kMaxLeaves];
  DevHyper hyper[FO_MAX_HYPERS];
  int32_t n_leaves;
  int32_t grad_dtype;
  int32_t group_size;
  int32_t pad;
};

// true when the quotient sqrt(nu)/sqrt(bc2) may be formed as div_by_rcp without changing
// (quotient + eps): for sqrt(nu) >= 2^-100 the shortcut is exact, below it the quotient is
// under half an ULP of eps either way.
__host__ __device__ inline bool adam_is_tame(float eps, float sqrt_bc2) {
  return eps >= 1.0e-12f && eps <= 1.0e12f && sqrt_bc2 >= 1.52587890625e-05f && sqrt_bc2 <= 2.0f;
}

struct Hyp {
  float lr, wd, b1, b2, omb1, omb2, eps;
  float decay, lr_bc1, sqrt_bc2, rcp_sqrt_bc2;
  uint32_t flags;
};

template <int OPT>
FO_DEVI Hyp load_hyper(const DevHyper& d) {
  Hyp h;
  h.lr = d.lr; h.wd = d.wd; h.b1 = d.b1; h.b2 = d.b2; h.omb1 = d.omb1; h.omb2 = d.omb2; h.eps = d.eps;
  h.decay = d.decay; h.lr_bc1 = d.lr_bc1; h.sqrt_bc2 = d.sqrt_bc2; h.rcp_sqrt_bc2 = d.rcp_sqrt_bc2;
  h.flags = d.flags;
  if (d.dyn != nullptr) {
    float lr = d.dyn[0];
    h.lr = lr;
    h.decay = fsub(1.0f, fmul(lr, d.wd));
    if constexpr (OPT == FO_OPT_ADAM) {
      h.lr_bc1 = fdiv(lr, d.dyn[1]);
      h.sqrt_bc2 = fsqrt(d.dyn[2]);
      h.rcp_sqrt_bc2 = __frcp_rn(h.sqrt_bc2);
      h.flags = (d.flags & ~kFlagTameAdam) | (adam_is_tame(d.eps, h.sqrt_bc2) ? kFlagTameAdam : 0u);
    }
  }
  return h;
}

FO_DEVI float sign_of(float x) { return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x); }

// ============================================================================================
// cold path: one element at a time, IEEE arithmetic only
// ============================================================================================

template <int OPT, int STATE>
FO_DEVI void update_element_ieee(const Hyp& h, float g, float& theta, float& m, float& v, float& root) {
  if constexpr (OPT == FO_OPT_ADAM) {
    // flashoptim_jax/adamw.py:95-106
    if (!(h.flags & FO_FLAG_DECOUPLED_WD)) g = fadd(g, fmul(h.wd, theta));
    m = fadd(fmul(h.b1, m), fmul(h.omb1, g));
    v = fadd(fmul(h.b2, v), fmul(h.omb2, fmul(g, g)));
    if (h.flags & FO_FLAG_DECOUPLED_WD) theta = fmul(theta, h.decay);
    root = fsqrt(v);
    theta = fsub(theta, fdiv(fmul(h.lr_bc1, m), fadd(fdiv(root, h.sqrt_bc2), h.eps)));
  } else if constexpr (OPT == FO_OPT_LION) {
    // flashoptim_jax/momentum_kernel.py:77-79 or flashoptim_jax/lion.py:50-52
    float upd;
    if (h.flags & FO_FLAG_LION_LERP) {
      float d = fsub(g, m);
      upd = sign_of(fadd(m, fmul(h.omb1, d)));
      m = fadd(m, fmul(h.omb2, d));
    } else {
      upd = sign_of(fadd(fmul(h.b1, m), fmul(h.omb1, g)));
      m = fadd(fmul(h.b2, m), fmul(h.omb2, g));
    }
    theta = fsub(fmul(theta, h.decay), fmul(h.lr, upd));
  } else {
    // flashoptim_jax/momentum_kernel.py:74-75,80-86; flashoptim_jax/sgd.py:45-63
    if (!(h.flags & FO_FLAG_DECOUPLED_WD)) g = fadd(g, fmul(h.wd, theta));
    float dir = g;
    if constexpr (STATE != FO_STATE_NONE) {
      m = fadd(fmul(h.b1, m), fmul(h.omb1, g));
      dir = (h.flags & FO_FLAG_NESTEROV) ? fadd(g, fmul(h.b1, m)) : m;
    }
    if (h.flags & FO_FLAG_DECOUPLED_WD) theta = fmul(theta, h.decay);
    theta = fsub(theta, fmul(h.lr, dir));
  }
}

// master weight -> stored form; old_bits is the stored param before the step, used only by
// the CPU-path convention that hands back param + lp(new - param) (adamw.py:411,415,463)
template <int PDT, int ECC_BITS>
FO_DEVI void store_form_ieee(uint32_t flags, float theta, uint32_t old_bits, uint32_t& new_bits, int& ecc) {
  using L = Lp<PDT>;
  if constexpr (ECC_BITS != 0) {
    ieee::split<PDT, ECC_BITS>(theta, new_bits, ecc);
  } else {
    new_bits = L::from_f32(theta);
    ecc = 0;
  }
  if (flags & FO_FLAG_LP_DELTA) {
    float oldf = L::to_f32(old_bits);
    float d = L::to_f32(L::from_f32(fsub(L::to_f32(new_bits), oldf)));
    new_bits = L::from_f32(fadd(oldf, d));
  }
}

template <int PDT, int ECC_BITS>
FO_DEVI float master_of_ieee(uint32_t bits, int ecc) {
  if constexpr (ECC_BITS == 0) {
    return Lp<PDT>::to_f32(bits);
  } else {
    return ieee::reconstruct<PDT, ECC_BITS>(bits, ecc);
  }
}

FO_DEVI float load_grad(const void* grad, int gdt, unsigned long long i) {
  if (gdt == FO_F32) return ((const float*)grad)[i];
  if (gdt == FO_BF16) return Lp<FO_BF16>::to_f32(((const unsigned short*)grad)[i]);
  return Lp<FO_F16>::to_f32(((const unsigned short*)grad)[i]);
}

// One chunk, any alignment, any length: thread t owns elements base + 8t .. base + 8t + 7,
// out-of-range elements count as zeros (flashoptim_jax/quantization.py:20-26).
template <int OPT, int PDT, int ECC_BITS, int STATE>
__device__ __noinline__ void cold_chunk(const DevLeaf& L, const Hyp& h, int gdt, unsigned long long base,
                                        const float* lut_m, const float* lut_v) {
  const unsigned long long n = L.n;
  const unsigned long long i0 = base + (unsigned long long)threadIdx.x * kPiece;
  const unsigned long long gi = i0 >> 5;
  const bool live = i0 < n;
  float m[8], root[8];
  float msc = 0.0f, vsc = 0.0f;
  if constexpr (STATE == FO_STATE_QUANT) {
    if (live) {
      msc = __half2float(((const __half*)L.mu_scales)[gi]);
      if constexpr (OPT == FO_OPT_ADAM) vsc = __half2float(((const __half*)L.nu_scales)[gi]);
    }
  }
#pragma unroll 1
  for (int j = 0; j < 8; ++j) {
    const unsigned long long i = i0 + j;
    m[j] = 0.0f; root[j] = 0.0f;
    if (i < n) {
      const float g = load_grad(L.grad, gdt, i);
      float theta, old_f32 = 0.0f;
      uint32_t pb = 0;
      if constexpr (PDT == FO_F32) {
        theta = ((const float*)L.param)[i];
        old_f32 = theta;
      } else {
        pb = ((const unsigned short*)L.param)[i];
        int e = 0;
        if constexpr (ECC_BITS == 16) e = ((const short*)L.ecc)[i];
        if constexpr (ECC_BITS == 8) e = ((const signed char*)L.ecc)[i];
        theta = master_of_ieee<PDT, ECC_BITS>(pb, e);
      }
      float mm = 0.0f, vv = 0.0f, rr = 0.0f;
      if constexpr (STATE == FO_STATE_QUANT) {
        mm = fmul(lut_m[((const unsigned char*)L.mu)[i]], msc);
        if constexpr (OPT == FO_OPT_ADAM) {
          float s = fmul(lut_v[((const unsigned char*)L.nu)[i]], vsc);
          vv = fmul(s, s);
        }
      } else if constexpr (STATE == FO_STATE_FULL) {
        mm = ((const float*)L.mu)[i];
        if constexpr (OPT == FO_OPT_ADAM) vv = ((const float*)L.nu)[i];
      }
      update_element_ieee<OPT, STATE>(h, g, theta, mm, vv, rr);
      if constexpr (PDT == FO_F32) {
        if (h.flags & FO_FLAG_LP_DELTA) theta = fadd(old_f32, fsub(theta, old_f32));
        ((float*)L.param)[i] = theta;
      } else {
        uint32_t nb;
        int e;
        store_form_ieee<PDT, ECC_BITS>(h.flags, theta, pb, nb, e);
        ((unsigned short*)L.param)[i] = (unsigned short)nb;
        if constexpr (ECC_BITS == 16) ((short*)L.ecc)[i] = (short)e;
        if constexpr (ECC_BITS == 8) ((signed char*)L.ecc)[i] = (signed char)e;
      }
      if constexpr (STATE == FO_STATE_FULL) {
        ((float*)L.mu)[i] = mm;
        if constexpr (OPT == FO_OPT_ADAM) ((float*)L.nu)[i] = vv;
      }
      m[j] = mm; root[j] = rr;
    }
  }
  if constexpr (STATE == FO_STATE_QUANT) {
    const bool floor_mode = (h.flags & FO_FLAG_SCALE_FLOOR) != 0;
    const bool writer = (threadIdx.x & 3) == 0 && live;
    float am = 0.0f, av = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { am = fmaxf(am, fabsf(m[j])); av = fmaxf(av, root[j]); }
    am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 2));
    const float sm = ieee::safe_scale(am, floor_mode);
#pragma unroll 1
    for (int j = 0; j < 8; ++j)
      if (i0 + j < n) ((signed char*)L.mu)[i0 + j] = (signed char)ieee::quant_m(m[j], sm);
    if (writer) ((__half*)L.mu_scales)[gi] = __float2half_rn(am);
    if constexpr (OPT == FO_OPT_ADAM) {
      av = fmaxf(av, __shfl_xor_sync(0xFFFFFFFFu, av, 1));
      av = fmaxf(av, __shfl_xor_sync(0xFFFFFFFFu, av, 2));
      const float sv = ieee::safe_scale(av, floor_mode);
#pragma unroll 1
      for (int j = 0; j < 8; ++j)
        if (i0 + j < n) ((unsigned char*)L.nu)[i0 + j] = (unsigned char)ieee::quant_v(root[j], sv);
      if (writer) ((__half*)L.nu_scales)[gi] = __float2half_rn(av);
    }
  }
}

// ============================================================================================
// hot path: one full aligned chunk, vector accesses, fast:: arithmetic
// ============================================================================================

// two 16-bit values of a packed word as fp32, and back
template <int PDT>
FO_DEVI void unpack2(uint32_t w, float& lo, float& hi) {
  if constexpr (PDT == FO_BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x; hi = f.y;
  }
}
template <int PDT>
FO_DEVI uint32_t pack2(float lo, float hi) {
  if constexpr (PDT == FO_BF16) {
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
  } else {
    __half2 b = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
  }
}

// per-element IEEE conversions kept out of line: they only run for unusual values
template <int PDT, int ECC_BITS>
__device__ __noinline__ float reconstruct_slow(uint32_t bits, int e) {
  return ieee::reconstruct<PDT, ECC_BITS>(bits, e);
}
template <int PDT, int ECC_BITS>
__device__ __noinline__ int ecc_slow(float theta) {
  uint32_t bits;
  int e;
  ieee::split<PDT, ECC_BITS>(theta, bits, e);
  return e;
}

FO_DEVI float min8(const float (&x)[8]) {
  return fminf(fminf(fminf(x[0], x[1]), fminf(x[2], x[3])), fminf(fminf(x[4], x[5]), fminf(x[6], x[7])));
}
FO_DEVI float minabs8(const float (&x)[8]) {
  return fminf(fminf(fminf(fabsf(x[0]), fabsf(x[1])), fminf(fabsf(x[2]), fabsf(x[3]))),
               fminf(fminf(fabsf(x[4]), fabsf(x[5])), fminf(fabsf(x[6]), fabsf(x[7]))));
}
FO_DEVI float maxabs8(const float (&x)[8]) {
  return fmaxf(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))),
               fmaxf(fmaxf(fabsf(x[4]), fabsf(x[5])), fmaxf(fabsf(x[6]), fabsf(x[7]))));
}
FO_DEVI float group_max(float a) {
  a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, 1));
  return fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, 2));
}
// low bytes of four words -> one word
FO_DEVI uint32_t pack_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
FO_DEVI uint32_t pack_halves(uint32_t lo, uint32_t hi) { return __byte_perm(lo, hi, 0x5410); }

template <int OPT, int PDT, int ECC_BITS, int STATE>
FO_DEVI void hot_chunk(const DevLeaf& L, const Hyp& h, const int gdt, const unsigned long long base,
                       const float* lut_m, const float* lut_v) {
  const unsigned long long i0 = base + (unsigned long long)threadIdx.x * kPiece;
  const unsigned long long gi = i0 >> 5;

  // ---- loads (all issued before the first use) ----------------------------------------------
  uint4 pw = make_uint4(0, 0, 0, 0), ew4 = make_uint4(0, 0, 0, 0);
  uint2 ew2 = make_uint2(0, 0), mq = make_uint2(0, 0), vq = make_uint2(0, 0);
  float4 fa[2], ma[2], va[2];
  float msc = 0.0f, vsc = 0.0f;
  if constexpr (PDT == FO_F32) {
    fa[0] = __ldcs((const float4*)((const float*)L.param + i0));
    fa[1] = __ldcs((const float4*)((const float*)L.param + i0) + 1);
  } else {
    pw = __ldcs((const uint4*)((const unsigned short*)L.param + i0));
  }
  if constexpr (ECC_BITS == 16) ew4 = __ldcs((const uint4*)((const short*)L.ecc + i0));
  if constexpr (ECC_BITS == 8) ew2 = __ldcs((const uint2*)((const signed char*)L.ecc + i0));
  if constexpr (STATE == FO_STATE_QUANT) {
    mq = __ldcs((const uint2*)((const unsigned char*)L.mu + i0));
    msc = __half2float(((const __half*)L.mu_scales)[gi]);
    if constexpr (OPT == FO_OPT_ADAM) {
      vq = __ldcs((const uint2*)((const unsigned char*)L.nu + i0));
      vsc = __half2float(((const __half*)L.nu_scales)[gi]);
    }
  } else if constexpr (STATE == FO_STATE_FULL) {
    ma[0] = __ldcs((const float4*)((const float*)L.mu + i0));
    ma[1] = __ldcs((const float4*)((const float*)L.mu + i0) + 1);
    if constexpr (OPT == FO_OPT_ADAM) {
      va[0] = __ldcs((const float4*)((const float*)L.nu + i0));
      va[1] = __ldcs((const float4*)((const float*)L.nu + i0) + 1);
    }
  }
  float g[8];
  if (gdt == FO_F32) {
    const float4 a = __ldcs((const float4*)((const float*)L.grad + i0));
    const float4 b = __ldcs((const float4*)((const float*)L.grad + i0) + 1);
    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
  } else {
    const uint4 w = __ldcs((const uint4*)((const unsigned short*)L.grad + i0));
    if (gdt == FO_BF16) {
      unpack2<FO_BF16>(w.x, g[0], g[1]); unpack2<FO_BF16>(w.y, g[2], g[3]);
      unpack2<FO_BF16>(w.z, g[4], g[5]); unpack2<FO_BF16>(w.w, g[6], g[7]);
    } else {
      unpack2<FO_F16>(w.x, g[0], g[1]); unpack2<FO_F16>(w.y, g[2], g[3]);
      unpack2<FO_F16>(w.z, g[4], g[5]); unpack2<FO_F16>(w.w, g[6], g[7]);
    }
  }

  // ---- master weight ---------------------------------------------------------------------------
  float theta[8], old_lp[8];
  if constexpr (PDT == FO_F32) {
    theta[0] = fa[0].x; theta[1] = fa[0].y; theta[2] = fa[0].z; theta[3] = fa[0].w;
    theta[4] = fa[1].x; theta[5] = fa[1].y; theta[6] = fa[1].z; theta[7] = fa[1].w;
#pragma unroll
    for (int j = 0; j < 8; ++j) old_lp[j] = theta[j];
  } else {
    unpack2<PDT>(pw.x, old_lp[0], old_lp[1]); unpack2<PDT>(pw.y, old_lp[2], old_lp[3]);
    unpack2<PDT>(pw.z, old_lp[4], old_lp[5]); unpack2<PDT>(pw.w, old_lp[6], old_lp[7]);
    if constexpr (ECC_BITS == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) theta[j] = old_lp[j];
    } else {
      int e[8];
      if constexpr (ECC_BITS == 16) {
        const uint32_t w[4] = {ew4.x, ew4.y, ew4.z, ew4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { e[2 * k] = (int)(short)(w[k] & 0xFFFFu); e[2 * k + 1] = (int)w[k] >> 16; }
      } else {
        const uint32_t w[2] = {ew2.x, ew2.y};
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = (int)(signed char)((w[k >> 2] >> (8 * (k & 3))) & 0xFFu);
      }
      bool ordinary = true;
      if constexpr (PDT == FO_BF16) ordinary = minabs8(old_lp) >= fast::Ordinary<PDT>::kMin;
      if (ordinary) {
#pragma unroll
        for (int j = 0; j < 8; ++j) theta[j] = fast::reconstruct_ordinary<PDT, ECC_BITS>(old_lp[j], (float)e[j]);
      } else {
        const uint32_t w[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
        for (int j = 0; j < 8; ++j)
          theta[j] = reconstruct_slow<PDT, ECC_BITS>((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu, e[j]);
      }
    }
  }

  // ---- moments -----------------------------------------------------------------------------------
  float m[8], v[8], root[8];
  if constexpr (STATE == FO_STATE_QUANT) {
    const uint32_t mw[2] = {mq.x, mq.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) m[j] = fmul(lut_m[(mw[j >> 2] >> (8 * (j & 3))) & 0xFFu], msc);   // quantization.py:52-55
    if constexpr (OPT == FO_OPT_ADAM) {
      const uint32_t vw[2] = {vq.x, vq.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float s = fmul(lut_v[(vw[j >> 2] >> (8 * (j & 3))) & 0xFFu], vsc);                   // quantization.py:74-77
        v[j] = fmul(s, s);
      }
    }
  } else if constexpr (STATE == FO_STATE_FULL) {
    m[0] = ma[0].x; m[1] = ma[0].y; m[2] = ma[0].z; m[3] = ma[0].w; m[4] = ma[1].x; m[5] = ma[1].y; m[6] = ma[1].z; m[7] = ma[1].w;
    if constexpr (OPT == FO_OPT_ADAM) {
      v[0] = va[0].x; v[1] = va[0].y; v[2] = va[0].z; v[3] = va[0].w; v[4] = va[1].x; v[5] = va[1].y; v[6] = va[1].z; v[7] = va[1].w;
    }
  }

  // ---- update --------------------------------------------------------------------------------------
  const bool decoupled = (h.flags & FO_FLAG_DECOUPLED_WD) != 0;
  if constexpr (OPT == FO_OPT_ADAM) {
    // flashoptim_jax/adamw.py:95-106
    if (!decoupled) {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = fadd(g[j], fmul(h.wd, theta[j]));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      m[j] = fadd(fmul(h.b1, m[j]), fmul(h.omb1, g[j]));
      v[j] = fadd(fmul(h.b2, v[j]), fmul(h.omb2, fmul(g[j], g[j])));
    }
    if (decoupled) {
#pragma unroll
      for (int j = 0; j < 8; ++j) theta[j] = fmul(theta[j], h.decay);
    }
    if (min8(v) >= 1.0e-30f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) root[j] = fast::sqrt_core(v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) root[j] = fsqrt(v[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float quo = fast::div_by_rcp(root[j], h.sqrt_bc2, h.rcp_sqrt_bc2);
      theta[j] = fsub(theta[j], fdiv(fmul(h.lr_bc1, m[j]), fadd(quo, h.eps)));
    }
  } else if constexpr (OPT == FO_OPT_LION) {
    // flashoptim_jax/momentum_kernel.py:77-79 or flashoptim_jax/lion.py:50-52
    float upd[8];
    if (h.flags & FO_FLAG_LION_LERP) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = fsub(g[j], m[j]);
        upd[j] = sign_of(fadd(m[j], fmul(h.omb1, d)));
        m[j] = fadd(m[j], fmul(h.omb2, d));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        upd[j] = sign_of(fadd(fmul(h.b1, m[j]), fmul(h.omb1, g[j])));
        m[j] = fadd(fmul(h.b2, m[j]), fmul(h.omb2, g[j]));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) theta[j] = fsub(fmul(theta[j], h.decay), fmul(h.lr, upd[j]));
  } else {
    // flashoptim_jax/momentum_kernel.py:74-75,80-86; flashoptim_jax/sgd.py:45-63
    if (!decoupled) {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = fadd(g[j], fmul(h.wd, theta[j]));
    }
    float dir[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) dir[j] = g[j];
    if constexpr (STATE != FO_STATE_NONE) {
#pragma unroll
      for (int j = 0; j < 8; ++j) m[j] = fadd(fmul(h.b1, m[j]), fmul(h.omb1, g[j]));
      if (h.flags & FO_FLAG_NESTEROV) {
#pragma unroll
        for (int j = 0; j < 8; ++j) dir[j] = fadd(g[j], fmul(h.b1, m[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) dir[j] = m[j];
      }
    }
    if (decoupled) {
#pragma unroll
      for (int j = 0; j < 8; ++j) theta[j] = fmul(theta[j], h.decay);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) theta[j] = fsub(theta[j], fmul(h.lr, dir[j]));
  }

  // ---- parameter (+ECC) back ---------------------------------------------------------------------
  if constexpr (PDT == FO_F32) {
    if (h.flags & FO_FLAG_LP_DELTA) {
#pragma unroll
      for (int j = 0; j < 8; ++j) theta[j] = fadd(old_lp[j], fsub(theta[j], old_lp[j]));
    }
    __stcs((float4*)((float*)L.param + i0), make_float4(theta[0], theta[1], theta[2], theta[3]));
    __stcs((float4*)((float*)L.param + i0) + 1, make_float4(theta[4], theta[5], theta[6], theta[7]));
  } else {
    uint32_t nw[4];
    float new_lp[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      nw[k] = pack2<PDT>(theta[2 * k], theta[2 * k + 1]);
      unpack2<PDT>(nw[k], new_lp[2 * k], new_lp[2 * k + 1]);
    }
    if constexpr (ECC_BITS != 0) {
      int ne[8];
      bool ordinary = true;
      if constexpr (PDT == FO_BF16) ordinary = minabs8(new_lp) >= fast::Ordinary<PDT>::kMin;
      if (ordinary) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ne[j] = fast::ecc_ordinary<PDT, ECC_BITS>(theta[j], new_lp[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) ne[j] = ecc_slow<PDT, ECC_BITS>(theta[j]);
      }
      if constexpr (ECC_BITS == 16) {
        uint4 o;
        o.x = pack_halves(ne[0], ne[1]); o.y = pack_halves(ne[2], ne[3]);
        o.z = pack_halves(ne[4], ne[5]); o.w = pack_halves(ne[6], ne[7]);
        __stcs((uint4*)((short*)L.ecc + i0), o);
      } else {
        uint2 o;
        o.x = pack_bytes(ne[0], ne[1], ne[2], ne[3]);
        o.y = pack_bytes(ne[4], ne[5], ne[6], ne[7]);
        __stcs((uint2*)((signed char*)L.ecc + i0), o);
      }
    }
    if (h.flags & FO_FLAG_LP_DELTA) {
      // adamw.py:411,415,463: param + lp(new_lp - param), both roundings to the param dtype
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float d0, d1;
        unpack2<PDT>(pack2<PDT>(fsub(new_lp[2 * k], old_lp[2 * k]), fsub(new_lp[2 * k + 1], old_lp[2 * k + 1])), d0, d1);
        nw[k] = pack2<PDT>(fadd(old_lp[2 * k], d0), fadd(old_lp[2 * k + 1], d1));
      }
    }
    __stcs((uint4*)((unsigned short*)L.param + i0), make_uint4(nw[0], nw[1], nw[2], nw[3]));
  }

  // ---- moments back ------------------------------------------------------------------------------
  if constexpr (STATE == FO_STATE_FULL) {
    __stcs((float4*)((float*)L.mu + i0), make_float4(m[0], m[1], m[2], m[3]));
    __stcs((float4*)((float*)L.mu + i0) + 1, make_float4(m[4], m[5], m[6], m[7]));
    if constexpr (OPT == FO_OPT_ADAM) {
      __stcs((float4*)((float*)L.nu + i0), make_float4(v[0], v[1], v[2], v[3]));
      __stcs((float4*)((float*)L.nu + i0) + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
  } else if constexpr (STATE == FO_STATE_QUANT) {
    const bool floor_mode = (h.flags & FO_FLAG_SCALE_FLOOR) != 0;
    const bool writer = (threadIdx.x & 3) == 0;
    {
      const float am = group_max(maxabs8(m));
      uint32_t q[8];
      if (am >= 1.0e-12f && am <= 1.0e30f) {
        const float rcp = fast::rcp_rn(am);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = fast::softsign_code_bits(fast::div_by_rcp(m[j], am, rcp));
      } else {
        const float safe = ieee::safe_scale(am, floor_mode);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = (uint32_t)ieee::quant_m(m[j], safe);
      }
      uint2 o;
      o.x = pack_bytes(q[0], q[1], q[2], q[3]);
      o.y = pack_bytes(q[4], q[5], q[6], q[7]);
      __stcs((uint2*)((signed char*)L.mu + i0), o);
      if (writer) ((__half*)L.mu_scales)[gi] = __float2half_rn(am);
    }
    if constexpr (OPT == FO_OPT_ADAM) {
      const float av = group_max(maxabs8(root));
      uint32_t q[8];
      if (av >= 1.0e-12f && av <= 1.0e30f) {
        const float rcp = fast::rcp_rn(av);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = fast::quant_v_bits(root[j], av, rcp);
      } else {
        const float safe = ieee::safe_scale(av, floor_mode);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = (uint32_t)ieee::quant_v(root[j], safe);
      }
      uint2 o;
      o.x = pack_bytes(q[0], q[1], q[2], q[3]);
      o.y = pack_bytes(q[4], q[5], q[6], q[7]);
      __stcs((uint2*)((unsigned char*)L.nu + i0), o);
      if (writer) ((__half*)L.nu_scales)[gi] = __float2half_rn(av);
    }
  }
}

// exact dequantization tables, one entry per code byte (built once per block)
FO_DEVI void build_luts(float* lut_m, float* lut_v) {
  for (int b = threadIdx.x; b < 256; b += blockDim.x) {
    lut_m[b] = ieee::deq_m_norm((int)(signed char)b);
    lut_v[b] = ieee::deq_v_norm(b);
  }
  __syncthreads();
}

template <int OPT, int PDT, int ECC_BITS, int STATE>
__global__ void __launch_bounds__(kThreads, FO_MIN_BLOCKS) step_kernel(const __grid_constant__ StepParams p) {
  __shared__ float lut_m[256], lut_v[256];
  if constexpr (STATE == FO_STATE_QUANT) build_luts(lut_m, lut_v);
  const uint32_t total = p.first_block[p.n_leaves];
  int l = 0;
  int l_loaded = -1;
  Hyp h;
  bool hot_ok = false;
  for (uint32_t c = blockIdx.x; c < total; c += gridDim.x) {
    while (c >= p.first_block[l + 1]) ++l;
    if (l != l_loaded) {
      h = load_hyper<OPT>(p.hyper[p.hyper_of[l]]);
      l_loaded = l;
      hot_ok = p.aligned[l] != 0;
#ifdef FO_NAIVE_MATH
      hot_ok = false;
#endif
      if constexpr (OPT == FO_OPT_ADAM) hot_ok = hot_ok && (h.flags & kFlagTameAdam) != 0;
    }
    const DevLeaf& L = p.leaf[l];
    const unsigned long long base = (unsigned long long)(c - p.first_block[l]) * kChunk;
    if (hot_ok && base + kChunk <= L.n) hot_chunk<OPT, PDT, ECC_BITS, STATE>(L, h, p.grad_dtype, base, lut_m, lut_v);
    else cold_chunk<OPT, PDT, ECC_BITS, STATE>(L, h, p.grad_dtype, base, lut_m, lut_v);
  }
}

// ---- any group size (1..1024): one block per tile of whole groups, group maxima through
// shared-memory atomics on the (non-negative) float bit patterns; IEEE arithmetic only ------
template <int OPT, int PDT, int ECC_BITS>
__global__ void __launch_bounds__(256) step_kernel_generic(const __grid_constant__ StepParams p) {
  __shared__ float lut_m[256], lut_v[256];
  __shared__ unsigned int smax_m[kGenericTile], smax_v[kGenericTile];
  build_luts(lut_m, lut_v);
  int lo = 0, hi = p.n_leaves;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (p.first_block[mid] <= blockIdx.x) lo = mid; else hi = mid;
  }
  const int l = lo;
  const DevLeaf& L = p.leaf[l];
  const Hyp h = load_hyper<OPT>(p.hyper[p.hyper_of[l]]);
  const int G = p.group_size;
  const int groups_per_tile = max(1, kGenericTile / G);
  const int tile = groups_per_tile * G;
  const unsigned long long n = L.n;
  const unsigned long long base = (unsigned long long)(blockIdx.x - p.first_block[l]) * tile;
  for (int i = threadIdx.x; i < groups_per_tile; i += 256) { smax_m[i] = 0u; smax_v[i] = 0u; }
  __syncthreads();
  constexpr int kPer = kGenericTile / 256;
  float m[kPer], root[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int li = threadIdx.x + k * 256;
    const unsigned long long i = base + li;
    m[k] = 0.0f; root[k] = 0.0f;
    if (li < tile && i < n) {
      const unsigned long long gi = i / G;
      const float g = load_grad(L.grad, p.grad_dtype, i);
      float theta, old_f32 = 0.0f;
      uint32_t pb = 0;
      if constexpr (PDT == FO_F32) {
        theta = ((const float*)L.param)[i];
        old_f32 = theta;
      } else {
        pb = ((const unsigned short*)L.param)[i];
        int e = 0;
        if constexpr (ECC_BITS == 16) e = ((const short*)L.ecc)[i];
        if constexpr (ECC_BITS == 8) e = ((const signed char*)L.ecc)[i];
        theta = master_of_ieee<PDT, ECC_BITS>(pb, e);
      }
      float mm = fmul(lut_m[((const unsigned char*)L.mu)[i]], __half2float(((const __half*)L.mu_scales)[gi]));
      float vv = 0.0f, rr = 0.0f;
      if constexpr (OPT == FO_OPT_ADAM) {
        float s = fmul(lut_v[((const unsigned char*)L.nu)[i]], __half2float(((const __half*)L.nu_scales)[gi]));
        vv = fmul(s, s);
      }
      update_element_ieee<OPT, FO_STATE_QUANT>(h, g, theta, mm, vv, rr);
      if constexpr (PDT == FO_F32) {
        if (h.flags & FO_FLAG_LP_DELTA) theta = fadd(old_f32, fsub(theta, old_f32));
        ((float*)L.param)[i] = theta;
      } else {
        uint32_t nb;
        int e;
        store_form_ieee<PDT, ECC_BITS>(h.flags, theta, pb, nb, e);
        ((unsigned short*)L.param)[i] = (unsigned short)nb;
        if constexpr (ECC_BITS == 16) ((short*)L.ecc)[i] = (short)e;
        if constexpr (ECC_BITS == 8) ((signed char*)L.ecc)[i] = (signed char)e;
      }
      m[k] = mm; root[k] = rr;
      atomicMax(&smax_m[li / G], __float_as_uint(fabsf(mm)));
      if constexpr (OPT == FO_OPT_ADAM) atomicMax(&smax_v[li / G], __float_as_uint(rr));
    }
  }
  __syncthreads();
  const bool floor_mode = (h.flags & FO_FLAG_SCALE_FLOOR) != 0;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int li = threadIdx.x + k * 256;
    const unsigned long long i = base + li;
    if (li < tile && i < n) {
      const float am = __uint_as_float(smax_m[li / G]);
      ((signed char*)L.mu)[i] = (signed char)ieee::quant_m(m[k], ieee::safe_scale(am, floor_mode));
      if (li % G == 0) ((__half*)L.mu_scales)[i / G] = __float2half_rn(am);
      if constexpr (OPT == FO_OPT_ADAM) {
        const float av = __uint_as_float(smax_v[li / G]);
        ((unsigned char*)L.nu)[i] = (unsigned char)ieee::quant_v(root[k], ieee::safe_scale(av, floor_mode));
        if (li % G == 0) ((__half*)L.nu_scales)[i / G] = __float2half_rn(av);
      }
    }
  }
}

// elements one block iteration covers, as the host must assume when it builds first_block[]
inline unsigned long long chunk_elems(int group_size, bool generic) {
  if (generic) return (unsigned long long)(kGenericTile / group_size > 0 ? kGenericTile / group_size : 1) * group_size;
  return (unsigned long long)kChunk;
}

// grid of the persistent kernel: resident blocks per SM x SMs of the current device
struct LaunchInfo {
  unsigned int total_chunks;
  int sm_count;
};
using LaunchFn = cudaError_t (*)(const StepParams&, const LaunchInfo&, cudaStream_t);

template <int OPT, int PDT, int ECC_BITS, int STATE>
cudaError_t launch_step(const StepParams& p, const LaunchInfo& info, cudaStream_t s) {
  unsigned int grid = (unsigned int)info.sm_count * FO_MIN_BLOCKS;
  if (grid > info.total_chunks) grid = info.total_chunks;
  step_kernel<OPT, PDT, ECC_BITS, STATE><<<grid, kThreads, 0, s>>>(p);
  return cudaGetLastError();
}
template <int OPT, int PDT, int ECC_BITS>
cudaError_t launch_step_generic(const StepParams& p, const LaunchInfo& info, cudaStream_t s) {
  step_kernel_generic<OPT, PDT, ECC_BITS><<<info.total_chunks, 256, 0, s>>>(p);
  return cudaGetLastError();
}

// lookups implemented by the instantiation units (fo_step_inst.cu, one per slice);
// each returns nullptr for a (param dtype, ecc width) pair that does not exist
#define FO_DECLARE_LOOKUP(name) LaunchFn name(int pdt, int ecc_bits);
FO_DECLARE_LOOKUP(lookup_adam_quant) FO_DECLARE_LOOKUP(lookup_adam_full) FO_DECLARE_LOOKUP(lookup_adam_generic)
FO_DECLARE_LOOKUP(lookup_lion_quant) FO_DECLARE_LOOKUP(lookup_lion_full) FO_DECLARE_LOOKUP(lookup_lion_generic)
FO_DECLARE_LOOKUP(lookup_sgd_quant) FO_DECLARE_LOOKUP(lookup_sgd_full) FO_DECLARE_LOOKUP(lookup_sgd_generic)
FO_DECLARE_LOOKUP(lookup_sgd_none)
#undef FO_DECLARE_LOOKUP

}  // namespace fo
