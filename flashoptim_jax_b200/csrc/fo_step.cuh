// Multi-tensor fused optimizer step for sm_100a.
//
// One launch walks a table of pytree leaves.  A block owns one contiguous chunk of one
// leaf; a thread owns PIECES pieces of 8 consecutive elements (piece p of thread t starts
// at chunk + p*2048 + t*8), so every warp-wide access is a run of 256 consecutive
// elements: 16 B per lane for the 2-byte streams (grad, param, int16 ECC), 8 B per lane
// for the 1-byte streams (int8/uint8 codes, int8 ECC).  A 32-element quantization group
// is 4 adjacent lanes of one piece; its absmax is two xor-shuffles.  Everything between
// load and store lives in registers: reconstruct the fp32 master weight, dequantize the
// moments, apply the update, split the weight back, requantize with fresh group scales.
// All arrays are updated in place; a group is read and written by the same 4 lanes only.
//
// The arithmetic follows flashoptim_jax/adamw.py:76-131 and
// flashoptim_jax/momentum_kernel.py:62-103 operation by operation (see fo_math.cuh).
#pragma once

#include <cuda_runtime.h>

#include "fo_math.cuh"

namespace fo {

constexpr int kThreads = 256;
constexpr int kPiece = 8;
constexpr int kPieceSpan = kThreads * kPiece;  // 2048 elements covered by one piece of a block
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
  uint32_t first_block[kMaxLeaves + 1];
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

#ifdef FO_NAIVE_MATH
FO_DEVI float step_sqrt(float v) { return fsqrt(v); }
struct GroupScale { float safe; };
FO_DEVI GroupScale step_group_scale(float a, bool floor_mode) { return GroupScale{ieee::safe_scale(a, floor_mode)}; }
FO_DEVI int step_quant_m(float x, const GroupScale& g) { return ieee::quant_m(x, g.safe); }
FO_DEVI int step_quant_v(float r, const GroupScale& g) { return ieee::quant_v(r, g.safe); }
#else
FO_DEVI float step_sqrt(float v) { return fast::sqrt_rn(v); }
using GroupScale = fast::GroupScale;
FO_DEVI GroupScale step_group_scale(float a, bool floor_mode) { return fast::group_scale(a, floor_mode); }
FO_DEVI int step_quant_m(float x, const GroupScale& g) { return fast::quant_m(x, g); }
FO_DEVI int step_quant_v(float r, const GroupScale& g) { return fast::quant_v(r, g); }
#endif

// One element of the update.  In: grad, master weight, moments.  Out: new master weight,
// new moments; root = sqrt(new nu) (Adam), reused by the variance quantizer.
template <int OPT, int STATE>
FO_DEVI void update_element(const Hyp& h, float g, float& theta, float& m, float& v, float& root) {
  if constexpr (OPT == FO_OPT_ADAM) {
    // flashoptim_jax/adamw.py:95-106
    if (!(h.flags & FO_FLAG_DECOUPLED_WD)) g = fadd(g, fmul(h.wd, theta));
    m = fadd(fmul(h.b1, m), fmul(h.omb1, g));
    v = fadd(fmul(h.b2, v), fmul(h.omb2, fmul(g, g)));
    if (h.flags & FO_FLAG_DECOUPLED_WD) theta = fmul(theta, h.decay);
    root = step_sqrt(v);
    float quo;
#ifndef FO_NAIVE_MATH
    if (h.flags & kFlagTameAdam) quo = fast::div_by_rcp(root, h.sqrt_bc2, h.rcp_sqrt_bc2);
    else
#endif
      quo = fdiv(root, h.sqrt_bc2);
    theta = fsub(theta, fdiv(fmul(h.lr_bc1, m), fadd(quo, h.eps)));
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

// master weight -> stored form.  old_bits/old_f32 is the stored param before the step, used
// only by the CPU-path convention that hands back param + lp(new - param).
template <int PDT, int ECC_BITS>
FO_DEVI void store_form(const Hyp& h, float theta, uint32_t old_bits, uint32_t& new_bits, int& ecc) {
  using L = Lp<PDT>;
  if constexpr (ECC_BITS != 0) {
#ifdef FO_NAIVE_MATH
    ieee::split<PDT, ECC_BITS>(theta, new_bits, ecc);
#else
    fast::split<PDT, ECC_BITS>(theta, new_bits, ecc);
#endif
  } else {
    new_bits = L::from_f32(theta);
    ecc = 0;
  }
  if (h.flags & FO_FLAG_LP_DELTA) {
    float oldf = L::to_f32(old_bits);
    float d = L::to_f32(L::from_f32(fsub(L::to_f32(new_bits), oldf)));
    new_bits = L::from_f32(fadd(oldf, d));
  }
}

template <int PDT, int ECC_BITS>
FO_DEVI float master_of(uint32_t bits, int ecc) {
  if constexpr (ECC_BITS == 0) {
    return Lp<PDT>::to_f32(bits);
  } else {
#ifdef FO_NAIVE_MATH
    return ieee::reconstruct<PDT, ECC_BITS>(bits, ecc);
#else
    return fast::reconstruct<PDT, ECC_BITS>(bits, ecc);
#endif
  }
}

// ---- register-level loads / stores of one 8-element piece --------------------------------

template <bool VEC>
FO_DEVI void load_f32x8(const void* base, unsigned long long i0, unsigned long long n, float (&out)[8]) {
  const float* p = (const float*)base + i0;
  if constexpr (VEC) {
    float4 a = __ldcs((const float4*)p), b = __ldcs((const float4*)p + 1);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = (i0 + j < n) ? p[j] : 0.0f;
  }
}
template <bool VEC>
FO_DEVI void store_f32x8(void* base, unsigned long long i0, unsigned long long n, const float (&v)[8]) {
  float* p = (float*)base + i0;
  if constexpr (VEC) {
    __stcs((float4*)p, make_float4(v[0], v[1], v[2], v[3]));
    __stcs((float4*)p + 1, make_float4(v[4], v[5], v[6], v[7]));
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i0 + j < n) p[j] = v[j];
  }
}
// eight 16-bit patterns, zero-extended
template <bool VEC>
FO_DEVI void load_u16x8(const void* base, unsigned long long i0, unsigned long long n, uint32_t (&out)[8]) {
  const unsigned short* p = (const unsigned short*)base + i0;
  if constexpr (VEC) {
    uint4 w = __ldcs((const uint4*)p);
    out[0] = w.x & 0xFFFFu; out[1] = w.x >> 16; out[2] = w.y & 0xFFFFu; out[3] = w.y >> 16;
    out[4] = w.z & 0xFFFFu; out[5] = w.z >> 16; out[6] = w.w & 0xFFFFu; out[7] = w.w >> 16;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = (i0 + j < n) ? (uint32_t)p[j] : 0u;
  }
}
template <bool VEC>
FO_DEVI void store_u16x8(void* base, unsigned long long i0, unsigned long long n, const uint32_t (&v)[8]) {
  unsigned short* p = (unsigned short*)base + i0;
  if constexpr (VEC) {
    uint4 w;
    w.x = (v[0] & 0xFFFFu) | (v[1] << 16); w.y = (v[2] & 0xFFFFu) | (v[3] << 16);
    w.z = (v[4] & 0xFFFFu) | (v[5] << 16); w.w = (v[6] & 0xFFFFu) | (v[7] << 16);
    __stcs((uint4*)p, w);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i0 + j < n) p[j] = (unsigned short)v[j];
  }
}
// eight bytes, zero-extended
template <bool VEC>
FO_DEVI void load_u8x8(const void* base, unsigned long long i0, unsigned long long n, uint32_t (&out)[8]) {
  const unsigned char* p = (const unsigned char*)base + i0;
  if constexpr (VEC) {
    uint2 w = __ldcs((const uint2*)p);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[j] = (w.x >> (8 * j)) & 0xFFu;
      out[4 + j] = (w.y >> (8 * j)) & 0xFFu;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = (i0 + j < n) ? (uint32_t)p[j] : 0u;
  }
}
template <bool VEC>
FO_DEVI void store_u8x8(void* base, unsigned long long i0, unsigned long long n, const uint32_t (&v)[8]) {
  unsigned char* p = (unsigned char*)base + i0;
  if constexpr (VEC) {
    uint2 w;
    w.x = (v[0] & 0xFFu) | ((v[1] & 0xFFu) << 8) | ((v[2] & 0xFFu) << 16) | (v[3] << 24);
    w.y = (v[4] & 0xFFu) | ((v[5] & 0xFFu) << 8) | ((v[6] & 0xFFu) << 16) | (v[7] << 24);
    __stcs((uint2*)p, w);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i0 + j < n) p[j] = (unsigned char)v[j];
  }
}

template <bool VEC>
FO_DEVI void load_grad8(const void* base, int gdt, unsigned long long i0, unsigned long long n, float (&g)[8]) {
  if (gdt == FO_F32) {
    load_f32x8<VEC>(base, i0, n, g);
  } else {
    uint32_t b[8];
    load_u16x8<VEC>(base, i0, n, b);
    if (gdt == FO_BF16) {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = Lp<FO_BF16>::to_f32(b[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = Lp<FO_F16>::to_f32(b[j]);
    }
  }
}

// everything a thread holds for one piece between load and compute
template <int PDT, int ECC_BITS, int STATE, int OPT>
struct Piece {
  uint32_t pb[8];   // 16-bit param patterns (PDT != F32)
  float pf[8];      // fp32 params (PDT == F32)
  uint32_t eb[8];   // raw ECC patterns, sign-extended later
  uint32_t mq[8];   // mu codes (raw bytes)  | QUANT
  uint32_t vq[8];   // nu codes              | QUANT
  float mf[8];      // fp32 mu               | FULL
  float vf[8];      // fp32 nu               | FULL
  float msc, vsc;   // fp16 group scales as fp32
};

template <int OPT, int PDT, int ECC_BITS, int STATE, bool VEC>
FO_DEVI void load_piece(const DevLeaf& L, unsigned long long i0, Piece<PDT, ECC_BITS, STATE, OPT>& r) {
  const unsigned long long n = L.n;
  if constexpr (PDT == FO_F32) load_f32x8<VEC>(L.param, i0, n, r.pf);
  else load_u16x8<VEC>(L.param, i0, n, r.pb);
  if constexpr (ECC_BITS == 16) load_u16x8<VEC>(L.ecc, i0, n, r.eb);
  if constexpr (ECC_BITS == 8) load_u8x8<VEC>(L.ecc, i0, n, r.eb);
  if constexpr (STATE == FO_STATE_QUANT) {
    load_u8x8<VEC>(L.mu, i0, n, r.mq);
    const bool live = VEC || i0 < n;
    const unsigned long long gi = i0 >> 5;
    r.msc = live ? __half2float(((const __half*)L.mu_scales)[gi]) : 0.0f;
    if constexpr (OPT == FO_OPT_ADAM) {
      load_u8x8<VEC>(L.nu, i0, n, r.vq);
      r.vsc = live ? __half2float(((const __half*)L.nu_scales)[gi]) : 0.0f;
    }
  } else if constexpr (STATE == FO_STATE_FULL) {
    load_f32x8<VEC>(L.mu, i0, n, r.mf);
    if constexpr (OPT == FO_OPT_ADAM) load_f32x8<VEC>(L.nu, i0, n, r.vf);
  }
}

template <int OPT, int PDT, int ECC_BITS, int STATE, bool VEC>
FO_DEVI void finish_piece(const DevLeaf& L, const Hyp& h, unsigned long long i0, Piece<PDT, ECC_BITS, STATE, OPT>& r,
                          const float (&g)[8], const float* lut_m, const float* lut_v) {
  const unsigned long long n = L.n;
  float theta[8], m[8], v[8], root[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if constexpr (PDT == FO_F32) theta[j] = r.pf[j];
    else {
      int e = ECC_BITS == 16 ? (int)(short)r.eb[j] : (int)(signed char)r.eb[j];
      theta[j] = master_of<PDT, ECC_BITS>(r.pb[j], e);
    }
    m[j] = 0.0f; v[j] = 0.0f; root[j] = 0.0f;
    if constexpr (STATE == FO_STATE_QUANT) {
      m[j] = fmul(lut_m[r.mq[j]], r.msc);                       // quantization.py:52-55
      if constexpr (OPT == FO_OPT_ADAM) {
        float s = fmul(lut_v[r.vq[j]], r.vsc);                  // quantization.py:74-77
        v[j] = fmul(s, s);
      }
    } else if constexpr (STATE == FO_STATE_FULL) {
      m[j] = r.mf[j];
      if constexpr (OPT == FO_OPT_ADAM) v[j] = r.vf[j];
    }
    update_element<OPT, STATE>(h, g[j], theta[j], m[j], v[j], root[j]);
  }

  // parameter (+ECC) back
  if constexpr (PDT == FO_F32) {
    if (h.flags & FO_FLAG_LP_DELTA) {
#pragma unroll
      for (int j = 0; j < 8; ++j) theta[j] = fadd(r.pf[j], fsub(theta[j], r.pf[j]));
    }
    store_f32x8<VEC>(L.param, i0, n, theta);
  } else {
    uint32_t nb[8], ne[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int e;
      store_form<PDT, ECC_BITS>(h, theta[j], r.pb[j], nb[j], e);
      ne[j] = (uint32_t)e;
    }
    store_u16x8<VEC>(L.param, i0, n, nb);
    if constexpr (ECC_BITS == 16) store_u16x8<VEC>(L.ecc, i0, n, ne);
    if constexpr (ECC_BITS == 8) store_u8x8<VEC>(L.ecc, i0, n, ne);
  }

  // moments back
  if constexpr (STATE == FO_STATE_FULL) {
    store_f32x8<VEC>(L.mu, i0, n, m);
    if constexpr (OPT == FO_OPT_ADAM) store_f32x8<VEC>(L.nu, i0, n, v);
  } else if constexpr (STATE == FO_STATE_QUANT) {
    const bool floor_mode = (h.flags & FO_FLAG_SCALE_FLOOR) != 0;
    const bool writer = (threadIdx.x & 3) == 0 && (VEC || i0 < n);
    const unsigned long long gi = i0 >> 5;
    float am = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(m[j]));
    am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 2));
    GroupScale gm = step_group_scale(am, floor_mode);
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = (uint32_t)step_quant_m(m[j], gm);
    store_u8x8<VEC>(L.mu, i0, n, q);
    if (writer) ((__half*)L.mu_scales)[gi] = __float2half_rn(am);
    if constexpr (OPT == FO_OPT_ADAM) {
      float av = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) av = fmaxf(av, root[j]);
      av = fmaxf(av, __shfl_xor_sync(0xFFFFFFFFu, av, 1));
      av = fmaxf(av, __shfl_xor_sync(0xFFFFFFFFu, av, 2));
      GroupScale gv = step_group_scale(av, floor_mode);
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = (uint32_t)step_quant_v(root[j], gv);
      store_u8x8<VEC>(L.nu, i0, n, q);
      if (writer) ((__half*)L.nu_scales)[gi] = __float2half_rn(av);
    }
  }
}

FO_DEVI int find_leaf(const StepParams& p, uint32_t bid) {
  int lo = 0, hi = p.n_leaves;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (p.first_block[mid] <= bid) lo = mid; else hi = mid;
  }
  return lo;
}

// exact dequantization tables, one entry per code byte (built once per block)
FO_DEVI void build_luts(float* lut_m, float* lut_v) {
  int b = threadIdx.x;
  if (b < 256) {
    lut_m[b] = ieee::deq_m_norm((int)(signed char)b);
    lut_v[b] = ieee::deq_v_norm(b);
  }
  __syncthreads();
}

template <int OPT, int PDT, int ECC_BITS, int STATE, int PIECES, bool VEC>
FO_DEVI void run_chunk(const StepParams& p, const DevLeaf& L, const Hyp& h, unsigned long long base,
                       const float* lut_m, const float* lut_v) {
  Piece<PDT, ECC_BITS, STATE, OPT> r[PIECES];
  float g[PIECES][8];
#pragma unroll
  for (int k = 0; k < PIECES; ++k)
    load_piece<OPT, PDT, ECC_BITS, STATE, VEC>(L, base + (unsigned long long)k * kPieceSpan + threadIdx.x * kPiece, r[k]);
#pragma unroll
  for (int k = 0; k < PIECES; ++k)
    load_grad8<VEC>(L.grad, p.grad_dtype, base + (unsigned long long)k * kPieceSpan + threadIdx.x * kPiece, L.n, g[k]);
#pragma unroll
  for (int k = 0; k < PIECES; ++k)
    finish_piece<OPT, PDT, ECC_BITS, STATE, VEC>(L, h, base + (unsigned long long)k * kPieceSpan + threadIdx.x * kPiece,
                                                 r[k], g[k], lut_m, lut_v);
}

template <int OPT, int PDT, int ECC_BITS, int STATE, int PIECES>
__global__ void __launch_bounds__(kThreads) step_kernel(const __grid_constant__ StepParams p) {
  __shared__ float lut_m[256], lut_v[256];
  if constexpr (STATE == FO_STATE_QUANT) build_luts(lut_m, lut_v);
  const int l = find_leaf(p, blockIdx.x);
  const DevLeaf& L = p.leaf[l];
  const Hyp h = load_hyper<OPT>(p.hyper[p.hyper_of[l]]);
  constexpr unsigned long long kChunk = (unsigned long long)PIECES * kPieceSpan;
  const unsigned long long base = (unsigned long long)(blockIdx.x - p.first_block[l]) * kChunk;
  if (p.aligned[l] && base + kChunk <= L.n)
    run_chunk<OPT, PDT, ECC_BITS, STATE, PIECES, true>(p, L, h, base, lut_m, lut_v);
  else
    run_chunk<OPT, PDT, ECC_BITS, STATE, PIECES, false>(p, L, h, base, lut_m, lut_v);
}

// ---- any group size (1..1024): one block per tile of whole groups, group maxima through
// shared-memory atomics on the (non-negative) float bit patterns --------------------------
template <int OPT, int PDT, int ECC_BITS>
__global__ void __launch_bounds__(kThreads) step_kernel_generic(const __grid_constant__ StepParams p) {
  __shared__ float lut_m[256], lut_v[256];
  __shared__ unsigned int smax_m[kGenericTile], smax_v[kGenericTile];
  build_luts(lut_m, lut_v);
  const int l = find_leaf(p, blockIdx.x);
  const DevLeaf& L = p.leaf[l];
  const Hyp h = load_hyper<OPT>(p.hyper[p.hyper_of[l]]);
  const int G = p.group_size;
  const int groups_per_tile = max(1, kGenericTile / G);
  const int tile = groups_per_tile * G;
  const unsigned long long n = L.n;
  const unsigned long long base = (unsigned long long)(blockIdx.x - p.first_block[l]) * tile;
  for (int i = threadIdx.x; i < groups_per_tile; i += kThreads) { smax_m[i] = 0u; smax_v[i] = 0u; }
  __syncthreads();
  constexpr int kPer = kGenericTile / kThreads;
  float m[kPer], root[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int li = threadIdx.x + k * kThreads;
    const unsigned long long i = base + li;
    m[k] = 0.0f; root[k] = 0.0f;
    if (li < tile && i < n) {
      const unsigned long long gi = i / G;
      float g = p.grad_dtype == FO_F32 ? ((const float*)L.grad)[i]
              : p.grad_dtype == FO_BF16 ? Lp<FO_BF16>::to_f32(((const unsigned short*)L.grad)[i])
                                        : Lp<FO_F16>::to_f32(((const unsigned short*)L.grad)[i]);
      float theta; uint32_t pb = 0;
      if constexpr (PDT == FO_F32) theta = ((const float*)L.param)[i];
      else {
        pb = ((const unsigned short*)L.param)[i];
        int e = ECC_BITS == 16 ? (int)((const short*)L.ecc)[i] : ECC_BITS == 8 ? (int)((const signed char*)L.ecc)[i] : 0;
        theta = master_of<PDT, ECC_BITS>(pb, e);
      }
      const float old_f32 = theta;
      float mm = fmul(lut_m[((const unsigned char*)L.mu)[i]], __half2float(((const __half*)L.mu_scales)[gi]));
      float vv = 0.0f, rr = 0.0f;
      if constexpr (OPT == FO_OPT_ADAM) {
        float s = fmul(lut_v[((const unsigned char*)L.nu)[i]], __half2float(((const __half*)L.nu_scales)[gi]));
        vv = fmul(s, s);
      }
      update_element<OPT, FO_STATE_QUANT>(h, g, theta, mm, vv, rr);
      if constexpr (PDT == FO_F32) {
        if (h.flags & FO_FLAG_LP_DELTA) theta = fadd(old_f32, fsub(theta, old_f32));
        ((float*)L.param)[i] = theta;
      } else {
        uint32_t nb; int e;
        store_form<PDT, ECC_BITS>(h, theta, pb, nb, e);
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
    const int li = threadIdx.x + k * kThreads;
    const unsigned long long i = base + li;
    if (li < tile && i < n) {
      const float am = __uint_as_float(smax_m[li / G]);
      ((signed char*)L.mu)[i] = (signed char)step_quant_m(m[k], step_group_scale(am, floor_mode));
      if (li % G == 0) ((__half*)L.mu_scales)[i / G] = __float2half_rn(am);
      if constexpr (OPT == FO_OPT_ADAM) {
        const float av = __uint_as_float(smax_v[li / G]);
        ((unsigned char*)L.nu)[i] = (unsigned char)step_quant_v(root[k], step_group_scale(av, floor_mode));
        if (li % G == 0) ((__half*)L.nu_scales)[i / G] = __float2half_rn(av);
      }
    }
  }
}

// elements one block covers, as the host must assume when it builds first_block[]
constexpr int kPiecesDefault = 2;
inline unsigned long long chunk_elems(int state, int group_size, bool generic) {
  (void)state;
  if (generic) return (unsigned long long)(kGenericTile / group_size > 0 ? kGenericTile / group_size : 1) * group_size;
  return (unsigned long long)kPiecesDefault * kPieceSpan;
}

using LaunchFn = cudaError_t (*)(const StepParams&, unsigned int grid, cudaStream_t);

template <int OPT, int PDT, int ECC_BITS, int STATE>
cudaError_t launch_step(const StepParams& p, unsigned int grid, cudaStream_t s) {
  step_kernel<OPT, PDT, ECC_BITS, STATE, kPiecesDefault><<<grid, kThreads, 0, s>>>(p);
  return cudaGetLastError();
}
template <int OPT, int PDT, int ECC_BITS>
cudaError_t launch_step_generic(const StepParams& p, unsigned int grid, cudaStream_t s) {
  step_kernel_generic<OPT, PDT, ECC_BITS><<<grid, kThreads, 0, s>>>(p);
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
