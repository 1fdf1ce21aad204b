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

#include <atomic>

#include "fo_math.cuh"

namespace fo {

// Tuning (measured on B200): 256-thread blocks; Adam's working set wants 128 registers
// (2 resident blocks per SM), Lion / SGD fit 3 blocks.
#ifndef FO_THREADS
#define FO_THREADS 256
#endif
#ifndef FO_MIN_BLOCKS_ADAM
#define FO_MIN_BLOCKS_ADAM 2
#endif
#ifndef FO_MIN_BLOCKS_MOMENTUM
#define FO_MIN_BLOCKS_MOMENTUM 3
#endif
#ifndef FO_MAX_STAGES
#define FO_MAX_STAGES 3
#endif
#ifndef FO_LUT_COPIES
#define FO_LUT_COPIES 8
#endif
constexpr int kThreads = FO_THREADS;
constexpr int min_blocks(int opt) { return opt == FO_OPT_ADAM ? FO_MIN_BLOCKS_ADAM : FO_MIN_BLOCKS_MOMENTUM; }
constexpr int kPiece = 8;
constexpr int kLutCopies = FO_LUT_COPIES;                 // copies of the momentum dequantization table in shared memory
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

// Replicas of the parameter arrays on peer GPUs (ZeRO-1 all-gather folded into the step): every
// updated parameter vector is also stored `delta[r]` bytes away from its local address, i.e. at the
// same element of peer r's replica.  Plain stores through peer-mapped memory; no waiting on peers.
constexpr int kMaxPeers = 7;
// Reduce-scatter folded into the step: the gradient of an element is the mean over this rank's
// value and the values `gdelta[r]` bytes away (the same element of peer r's gradient buffer):
// fp32 sum in the order own, peer 0, peer 1, ..., divided by the number of ranks, rounded once to
// the gradient dtype.  Plain loads through peer-mapped memory.
struct Peers {
  int n;              // replicas that receive the parameter stores
  int ng;             // peers whose gradients are read
  long long delta[kMaxPeers];
  long long gdelta[kMaxPeers];
  float neg_ranks;    // -(ng + 1)
  float rcp_ranks;    // RN(1 / (ng + 1))
  int ranks_pow2;     // the division by the rank count is exact for every input
  int pad;
  // NVLink-switch forms of the two exchanges (0 = off; the point-to-point tables above stay valid
  // and serve the ragged ends): byte distance from a local address to the multicast address of
  // the same element.  A multicast store reaches every rank's replica, this one's included; a
  // multicast load-reduce returns the sum over all ranks' gradients, added up in the switch in
  // fp32 and rounded to the gradient dtype.
  long long mc_pdelta;
  long long mc_gdelta;
};

FO_DEVI uint4 multicast_sum(const void* p, const int gdt) {
  uint4 v;
  if (gdt == FO_BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
FO_DEVI void multicast_store(void* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <typename T>
FO_DEVI void store_to_peers(const Peers& peers, T* local, const T& v) {
  for (int r = 0; r < peers.n; ++r) *reinterpret_cast<T*>(reinterpret_cast<char*>(local) + peers.delta[r]) = v;
}

struct StepParams {
  DevLeaf leaf[kMaxLeaves];
  uint32_t first_block[kMaxLeaves + 1];  // first chunk of each leaf; [n_leaves] = total chunks
  uint8_t hyper_of[kMaxLeaves];
  uint8_t aligned[kMaxLeaves];
  DevHyper hyper[FO_MAX_HYPERS];
  int32_t n_leaves;
  int32_t grad_dtype;
  int32_t group_size;
  float one;  // 1.0f the compiler cannot see through (see fast2::sum2)
  int32_t stages;  // shared-memory stages of the copy pipeline (2..8), set by the launcher
  Peers peers;
  const double* sq_norm;  // device: sum of squares of all gradients of the step (nullptr: no clipping)
  float max_norm;
  uint32_t run_chunks;  // consecutive chunks a block takes at a time (set by the launcher)
};

// true when the quotient sqrt(nu)/sqrt(bc2) may be formed as div_by_rcp without changing
// (quotient + eps): for sqrt(nu) >= 2^-100 the shortcut is exact, below it the quotient is
// under half an ULP of eps either way.
__host__ __device__ inline bool adam_is_tame(float eps, float sqrt_bc2) {
  return eps >= 1.0e-12f && eps <= 1.0f && sqrt_bc2 >= 1.52587890625e-05f && sqrt_bc2 <= 2.0f;
}

struct Hyp {
  float lr, wd, b1, b2, omb1, omb2, eps;
  float decay, lr_bc1, sqrt_bc2, rcp_sqrt_bc2;
  float m_lo, m_hi;  // Adam: first moments between these keep the update's numerator lr/bc1 * m inside [2^-70, 2^60]
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
  h.m_lo = 0.0f; h.m_hi = 0.0f;
  if constexpr (OPT == FO_OPT_ADAM) {
    // quotients nudged two places inwards, so that m >= m_lo implies RN(|lr_bc1| * m) >= 2^-70 and
    // m <= m_hi implies RN(|lr_bc1| * m) <= 2^60; lr = 0 gives m_lo = inf (everything takes the IEEE repairs)
    const float lrb = fabsf(h.lr_bc1);
    h.m_lo = fmul(fdiv(8.4703295e-22f, lrb), 1.0000005f);
    h.m_hi = fmul(fdiv(1.1529215e18f, lrb), 0.9999995f);
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
// fp32 value rounded to the gradient dtype and back
FO_DEVI float round_to_grad_dtype(float x, int gdt) {
  if (gdt == FO_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  if (gdt == FO_F16) return __half2float(__float2half_rn(x));
  return x;
}
// Global-norm clipping folded into the step (optax.clip_by_global_norm as the reference's GPT-2
// recipe chains it in front of the optimizer, examples/train_gpt2_pretrain.py:56-70):
//   norm = sqrt(sum of squares);  keep g if norm < max_norm, else g <- (g / norm.astype(g.dtype)) * max_norm
// with the division and the product each rounded to the gradient dtype.
struct Clip {
  bool active;   // norm >= max_norm (or NaN): gradients are rescaled
  bool div_ok;   // the reciprocal shortcut is exact for this divisor
  float n_g;     // norm rounded to the gradient dtype
  float rcp_n;   // RN(1 / n_g)
  float m_g;     // max_norm rounded to the gradient dtype
};
FO_DEVI Clip load_clip(const double* sq_norm, float max_norm, int gdt) {
  Clip c;
  c.active = false; c.div_ok = true; c.n_g = 1.0f; c.rcp_n = 1.0f; c.m_g = 1.0f;
  if (sq_norm == nullptr) return c;
  const float norm = (float)sqrt(*sq_norm);
  c.active = !(norm < max_norm);
  c.n_g = round_to_grad_dtype(norm, gdt);
  c.m_g = round_to_grad_dtype(max_norm, gdt);
  c.rcp_n = __frcp_rn(c.n_g);
  // Markstein's correction needs a correctly rounded reciprocal of a divisor whose mantissa is not all ones
  c.div_ok = (__float_as_uint(c.n_g) & 0x7FFFFFu) != 0x7FFFFFu && c.n_g >= 9.5367432e-7f && c.n_g <= 1048576.0f;  // [2^-20, 2^20]
  return c;
}
FO_DEVI float clip_ieee(float g, const Clip& c, int gdt) {
  if (!c.active) return g;
  return round_to_grad_dtype(fmul(round_to_grad_dtype(fdiv(g, c.n_g), gdt), c.m_g), gdt);
}

// the gradient of element i: the local value, or the mean over the ranks (see Peers)
FO_DEVI float load_grad_mean(const void* grad, int gdt, unsigned long long i, const Peers& peers) {
  float g = load_grad(grad, gdt, i);
  if (peers.ng == 0) return g;
  for (int r = 0; r < peers.ng; ++r) g = fadd(g, load_grad((const char*)grad + peers.gdelta[r], gdt, i));
  return round_to_grad_dtype(fdiv(g, -peers.neg_ranks), gdt);
}

// One chunk, any alignment, any length: thread t owns elements base + 8t .. base + 8t + 7,
// out-of-range elements count as zeros (flashoptim_jax/quantization.py:20-26).
template <int OPT, int PDT, int ECC_BITS, int STATE>
__device__ __noinline__ void cold_chunk(const DevLeaf& L, const Hyp& h, int gdt, unsigned long long base,
                                        const float* lut_m, const float* lut_v, const Peers& peers, const Clip& clip) {
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
      const float g = clip_ieee(load_grad_mean(L.grad, gdt, i, peers), clip, gdt);
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
        store_to_peers(peers, (float*)L.param + i, theta);
      } else {
        uint32_t nb;
        int e;
        store_form_ieee<PDT, ECC_BITS>(h.flags, theta, pb, nb, e);
        ((unsigned short*)L.param)[i] = (unsigned short)nb;
        store_to_peers(peers, (unsigned short*)L.param + i, (unsigned short)nb);
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

FO_DEVI float group_max(float a) {
  a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, 1));
  return fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, 2));
}
// low bytes of four words -> one word
FO_DEVI uint32_t pack_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
FO_DEVI uint32_t pack_halves(uint32_t lo, uint32_t hi) { return __byte_perm(lo, hi, 0x5410); }

// 3-input min / max (one instruction on sm_100)
FO_DEVI float min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
FO_DEVI float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Per-lane repairs of the second-chance path (REPAIR = true below), kept out of line: they run only
// for lanes that hold a value outside the range a shortcut is proven for (zeros, subnormals, huge
// values) and redo that stage with IEEE operations.
template <int PDT, int ECC_BITS>
__device__ __noinline__ float repair_master(uint32_t bits, int e) {
  return ieee::reconstruct<PDT, ECC_BITS>(bits, e);
}
template <int PDT, int ECC_BITS>
__device__ __noinline__ int repair_ecc(float theta) {
  uint32_t bits;
  int e;
  ieee::split<PDT, ECC_BITS>(theta, bits, e);
  return e;
}
// root = sqrt(v); returns theta - (lr_bc1 * m) / (root / sqrt_bc2 + eps)   (adamw.py:104-106)
static __device__ __noinline__ float repair_adam(float v, float m, float theta, float lr_bc1, float sqrt_bc2, float eps, float& root) {
  root = fsqrt(v);
  return fsub(theta, fdiv(fmul(lr_bc1, m), fadd(fdiv(root, sqrt_bc2), eps)));
}
static __device__ __noinline__ uint32_t repair_code_m(float x, float safe) { return (uint32_t)ieee::quant_m(x, safe); }
static __device__ __noinline__ uint32_t repair_code_v(float r, float safe) { return (uint32_t)ieee::quant_v(r, safe); }

// what one thread loads for one chunk: its 8 elements of every stream, still packed
template <int OPT, int PDT, int ECC_BITS, int STATE>
struct Raw {
  uint4 g0, g1;        // grad: 8 x 16-bit in g0, or 8 x fp32 in g0,g1
  uint4 p0, p1;        // param: 8 x 16-bit in p0, or 8 x fp32 in p0,p1
  uint4 e;             // ECC: 8 x int16 in e, or 8 x int8 in e.x,e.y
  uint2 mq, vq;        // codes
  __half msc, vsc;     // group scales
  uint4 m0, m1, v0, v1;  // fp32 moments (FULL)
};

template <int OPT, int PDT, int ECC_BITS, int STATE>
FO_DEVI void hot_load(const DevLeaf& L, const int gdt, const uint32_t i0, Raw<OPT, PDT, ECC_BITS, STATE>& r) {
  if constexpr (PDT == FO_F32) {
    r.p0 = __ldcs((const uint4*)((const float*)L.param + i0));
    r.p1 = __ldcs((const uint4*)((const float*)L.param + i0) + 1);
  } else {
    r.p0 = __ldcs((const uint4*)((const unsigned short*)L.param + i0));
  }
  if constexpr (ECC_BITS == 16) r.e = __ldcs((const uint4*)((const short*)L.ecc + i0));
  if constexpr (ECC_BITS == 8) {
    const uint2 t = __ldcs((const uint2*)((const signed char*)L.ecc + i0));
    r.e.x = t.x; r.e.y = t.y;
  }
  if constexpr (STATE == FO_STATE_QUANT) {
    r.mq = __ldcs((const uint2*)((const unsigned char*)L.mu + i0));
    r.msc = ((const __half*)L.mu_scales)[i0 >> 5];
    if constexpr (OPT == FO_OPT_ADAM) {
      r.vq = __ldcs((const uint2*)((const unsigned char*)L.nu + i0));
      r.vsc = ((const __half*)L.nu_scales)[i0 >> 5];
    }
  } else if constexpr (STATE == FO_STATE_FULL) {
    r.m0 = __ldcs((const uint4*)((const float*)L.mu + i0));
    r.m1 = __ldcs((const uint4*)((const float*)L.mu + i0) + 1);
    if constexpr (OPT == FO_OPT_ADAM) {
      r.v0 = __ldcs((const uint4*)((const float*)L.nu + i0));
      r.v1 = __ldcs((const uint4*)((const float*)L.nu + i0) + 1);
    }
  }
  if (gdt == FO_F32) {
    r.g0 = __ldcs((const uint4*)((const float*)L.grad + i0));
    r.g1 = __ldcs((const uint4*)((const float*)L.grad + i0) + 1);
  } else {
    r.g0 = __ldcs((const uint4*)((const unsigned short*)L.grad + i0));
  }
}

// ---- shared-memory staging of the streams (asynchronous copies) ---------------------------------
// Every thread copies its own eight elements of every stream of a later chunk into a slot of
// shared memory that only it reads back, so the pipeline needs no barrier: the thread waits for
// its own copy groups.  Several chunks are in flight per thread at no cost in registers.
// A 32-byte stream (fp32) is kept as two planes of 16 bytes per thread, so that the 128-bit
// reads of a warp fall on consecutive banks.
template <int OPT, int PDT, int ECC_BITS, int STATE>
struct Stage {
  static constexpr int kParam = PDT == FO_F32 ? 32 : 16;  // bytes per thread and stage
  static constexpr int kEcc = ECC_BITS == 16 ? 16 : (ECC_BITS == 8 ? 8 : 0);
  static constexpr int kMu = STATE == FO_STATE_QUANT ? 8 : (STATE == FO_STATE_FULL ? 32 : 0);
  static constexpr int kNu = OPT == FO_OPT_ADAM ? kMu : 0;
  static constexpr int kOffEcc = kParam * kThreads;       // byte offsets of the streams inside a stage
  static constexpr int kOffMu = kOffEcc + kEcc * kThreads;
  static constexpr int kOffNu = kOffMu + kMu * kThreads;
  static constexpr int kOffGrad = kOffNu + kNu * kThreads;
  // the gradient comes last: this rank's piece, then one piece per peer whose gradients are averaged in
  __host__ __device__ static constexpr int grad_bytes(int gdt) { return (gdt == FO_F32 ? 32 : 16) * kThreads; }
  __host__ __device__ static constexpr int bytes(int gdt, int grad_peers) { return kOffGrad + grad_bytes(gdt) * (1 + grad_peers); }
};
constexpr int kMaxStages = FO_MAX_STAGES;   // local streams: deeper brings nothing (measured 2 = 3 = 4)
#ifndef FO_PLAIN_STAGES
#define FO_PLAIN_STAGES 3
#endif
constexpr int kPlainStages = FO_PLAIN_STAGES;  // stages (= unroll factor) of the kernel without peer or clipping code
#ifndef FO_MAX_STAGES_PEERS
#define FO_MAX_STAGES_PEERS 8
#endif
constexpr int kMaxStagesPeers = FO_MAX_STAGES_PEERS;  // gradients read from peers over NVLink: several times the latency to cover
constexpr int kSwitchBatch = 4;  // multicast load-reduces a thread keeps in flight
FO_DEVI void copy_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// for the two halves of a 32-byte piece: each copy uses half of every 32-byte sector it touches,
// so the line is kept in L1 for the other half
FO_DEVI void copy_async16_l1(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
FO_DEVI void copy_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
FO_DEVI void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
FO_DEVI void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
FO_DEVI uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
  return v;
}
FO_DEVI uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory");
  return v;
}

// start the copies of this thread's piece at element i0 of every stream into the stage at
// shared address st (the group scales are not staged: they are two bytes per 32 elements)
template <int OPT, int PDT, int ECC_BITS, int STATE>
FO_DEVI void stage_fill(const DevLeaf& L, const int gdt, const uint32_t i0, const uint32_t st, const Peers& peers, const int ng,
                        const bool with_grad = true) {
  using S = Stage<OPT, PDT, ECC_BITS, STATE>;
  const uint32_t t16 = threadIdx.x * 16u, t8 = threadIdx.x * 8u;
  if constexpr (PDT == FO_F32) {
    copy_async16_l1(st + t16, (const float*)L.param + i0);
    copy_async16_l1(st + 16u * kThreads + t16, (const float*)L.param + i0 + 4);
  } else {
    copy_async16(st + t16, (const unsigned short*)L.param + i0);
  }
  if constexpr (ECC_BITS == 16) copy_async16(st + S::kOffEcc + t16, (const short*)L.ecc + i0);
  if constexpr (ECC_BITS == 8) copy_async8(st + S::kOffEcc + t8, (const signed char*)L.ecc + i0);
  if constexpr (STATE == FO_STATE_QUANT) {
    copy_async8(st + S::kOffMu + t8, (const unsigned char*)L.mu + i0);
    if constexpr (OPT == FO_OPT_ADAM) copy_async8(st + S::kOffNu + t8, (const unsigned char*)L.nu + i0);
  } else if constexpr (STATE == FO_STATE_FULL) {
    copy_async16_l1(st + S::kOffMu + t16, (const float*)L.mu + i0);
    copy_async16_l1(st + S::kOffMu + 16u * kThreads + t16, (const float*)L.mu + i0 + 4);
    if constexpr (OPT == FO_OPT_ADAM) {
      copy_async16_l1(st + S::kOffNu + t16, (const float*)L.nu + i0);
      copy_async16_l1(st + S::kOffNu + 16u * kThreads + t16, (const float*)L.nu + i0 + 4);
    }
  }
  if (!with_grad) return;  // the gradients arrive as sums from the switch (see the ring in step_kernel)
  uint32_t gs = st + S::kOffGrad;
  if (gdt == FO_F32) {
    copy_async16_l1(gs + t16, (const float*)L.grad + i0);
    copy_async16_l1(gs + 16u * kThreads + t16, (const float*)L.grad + i0 + 4);
  } else {
    copy_async16(gs + t16, (const unsigned short*)L.grad + i0);
  }
  for (int r = 0; r < ng; ++r) {  // the peers' pieces follow this rank's
    const char* g = (const char*)L.grad + peers.gdelta[r];
    gs += (uint32_t)S::grad_bytes(gdt);
    if (gdt == FO_F32) {
      copy_async16_l1(gs + t16, (const float*)g + i0);
      copy_async16_l1(gs + 16u * kThreads + t16, (const float*)g + i0 + 4);
    } else {
      copy_async16(gs + t16, (const unsigned short*)g + i0);
    }
  }
}

// read this thread's piece back from a stage whose copies have completed
template <int OPT, int PDT, int ECC_BITS, int STATE>
FO_DEVI void stage_read(const int gdt, const uint32_t st, Raw<OPT, PDT, ECC_BITS, STATE>& r) {
  using S = Stage<OPT, PDT, ECC_BITS, STATE>;
  const uint32_t t16 = threadIdx.x * 16u, t8 = threadIdx.x * 8u;
  r.p0 = lds128(st + t16);
  if constexpr (PDT == FO_F32) r.p1 = lds128(st + 16u * kThreads + t16);
  if constexpr (ECC_BITS == 16) r.e = lds128(st + S::kOffEcc + t16);
  if constexpr (ECC_BITS == 8) {
    const uint2 t = lds64(st + S::kOffEcc + t8);
    r.e.x = t.x; r.e.y = t.y;
  }
  if constexpr (STATE == FO_STATE_QUANT) {
    r.mq = lds64(st + S::kOffMu + t8);
    if constexpr (OPT == FO_OPT_ADAM) r.vq = lds64(st + S::kOffNu + t8);
  } else if constexpr (STATE == FO_STATE_FULL) {
    r.m0 = lds128(st + S::kOffMu + t16);
    r.m1 = lds128(st + S::kOffMu + 16u * kThreads + t16);
    if constexpr (OPT == FO_OPT_ADAM) {
      r.v0 = lds128(st + S::kOffNu + t16);
      r.v1 = lds128(st + S::kOffNu + 16u * kThreads + t16);
    }
  }
  r.g0 = lds128(st + S::kOffGrad + t16);
  if (gdt == FO_F32) r.g1 = lds128(st + S::kOffGrad + 16u * kThreads + t16);
}

// what survives of a chunk's loads once they are unpacked: fp32 pairs ready for the update
// (pair k holds elements 2k and 2k+1 of the thread's piece)
struct Unpacked {
  float2 g[4];
  float2 theta[4];    // master weight
  float2 m[4], v[4];
};

FO_DEVI void pairs_of(const uint4& a, const uint4& b, float2 (&o)[4]) {
  o[0] = make_float2(__uint_as_float(a.x), __uint_as_float(a.y));
  o[1] = make_float2(__uint_as_float(a.z), __uint_as_float(a.w));
  o[2] = make_float2(__uint_as_float(b.x), __uint_as_float(b.y));
  o[3] = make_float2(__uint_as_float(b.z), __uint_as_float(b.w));
}
template <int DT>
FO_DEVI void pairs_of16(const uint4& w, float2 (&o)[4]) {
  unpack2<DT>(w.x, o[0].x, o[0].y); unpack2<DT>(w.y, o[1].x, o[1].y);
  unpack2<DT>(w.z, o[2].x, o[2].y); unpack2<DT>(w.w, o[3].x, o[3].y);
}
FO_DEVI float min8(const float2 (&x)[4]) {
  return min3(min3(x[0].x, x[0].y, x[1].x), min3(x[1].y, x[2].x, x[2].y), fminf(x[3].x, x[3].y));
}
FO_DEVI float max8(const float2 (&x)[4]) {
  return max3(max3(x[0].x, x[0].y, x[1].x), max3(x[1].y, x[2].x, x[2].y), fmaxf(x[3].x, x[3].y));
}
FO_DEVI float minabs8(const float2 (&x)[4]) {
  return min3(min3(fabsf(x[0].x), fabsf(x[0].y), fabsf(x[1].x)), min3(fabsf(x[1].y), fabsf(x[2].x), fabsf(x[2].y)),
              fminf(fabsf(x[3].x), fabsf(x[3].y)));
}
FO_DEVI float maxabs8(const float2 (&x)[4]) {
  return max3(max3(fabsf(x[0].x), fabsf(x[0].y), fabsf(x[1].x)), max3(fabsf(x[1].y), fabsf(x[2].x), fabsf(x[2].y)),
              fmaxf(fabsf(x[3].x), fabsf(x[3].y)));
}
// byte k of a word as an index
FO_DEVI uint32_t byte_of(uint32_t w, int k) { return __byte_perm(w, 0u, 0x4440u | (uint32_t)k); }

// Addresses of the eight elements a thread owns in the current chunk, one per stream.  Inside a run
// of consecutive chunks they advance by compile-time constants, so a later chunk's address is this
// one plus an immediate.
struct Piece {
  const char* grad;
  char* param;
  char* ecc;
  char* mu;
  char* nu;
  char* msc;  // the group's scale (four lanes share one)
  char* vsc;
};
template <int PDT, int ECC_BITS, int STATE>
FO_DEVI Piece piece_at(const DevLeaf& L, const int gdt, const uint32_t i0) {
  Piece a;
  a.grad = (const char*)L.grad + (size_t)i0 * (gdt == FO_F32 ? 4u : 2u);
  a.param = (char*)L.param + (size_t)i0 * (PDT == FO_F32 ? 4u : 2u);
  a.ecc = (char*)L.ecc + (size_t)i0 * (ECC_BITS == 16 ? 2u : 1u);
  a.mu = (char*)L.mu + (size_t)i0 * (STATE == FO_STATE_FULL ? 4u : 1u);
  a.nu = (char*)L.nu + (size_t)i0 * (STATE == FO_STATE_FULL ? 4u : 1u);
  a.msc = (char*)L.mu_scales + (size_t)(i0 >> 5) * 2u;
  a.vsc = (char*)L.nu_scales + (size_t)(i0 >> 5) * 2u;
  return a;
}

// master weights of a piece from the stored parameter words (p0, p1) and ECC words (e_in); same
// contract for REPAIR as hot_unpack
template <bool REPAIR, int PDT, int ECC_BITS>
FO_DEVI bool unpack_master(const uint4& p0, const uint4& p1, const uint4& e_in, const float2 one2, float2 (&theta)[4]) {
  using namespace fast2;
  bool rare = false;
  if constexpr (PDT == FO_F32) {
    pairs_of(p0, p1, theta);
  } else {
    float2 old_lp[4];  // stored param as fp32
    pairs_of16<PDT>(p0, old_lp);
    if constexpr (ECC_BITS == 0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) theta[k] = old_lp[k];
    } else {
      int e[8];
      // The ECC halves / bytes go to fp32 by conversions that name the 16- or 8-bit part of the word
      // (no sign extension first); the integers are needed by the repairs only.
      float ef[8];
      if constexpr (ECC_BITS == 16) {
        const uint32_t w[4] = {e_in.x, e_in.y, e_in.z, e_in.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.rn.f32.s16 %0, lo; cvt.rn.f32.s16 %1, hi;}"
              : "=f"(ef[2 * k]), "=f"(ef[2 * k + 1]) : "r"(w[k]));
          if constexpr (REPAIR) { e[2 * k] = (int)(short)(w[k] & 0xFFFFu); e[2 * k + 1] = (int)w[k] >> 16; }
        }
      } else {
        const uint32_t w[2] = {e_in.x, e_in.y};
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          asm("{.reg .b8 b0, b1, b2, b3; .reg .s16 t; mov.b32 {b0, b1, b2, b3}, %4;"
              " cvt.s16.s8 t, b0; cvt.rn.f32.s16 %0, t; cvt.s16.s8 t, b1; cvt.rn.f32.s16 %1, t;"
              " cvt.s16.s8 t, b2; cvt.rn.f32.s16 %2, t; cvt.s16.s8 t, b3; cvt.rn.f32.s16 %3, t;}"
              : "=f"(ef[4 * k]), "=f"(ef[4 * k + 1]), "=f"(ef[4 * k + 2]), "=f"(ef[4 * k + 3]) : "r"(w[k]));
        }
        if constexpr (REPAIR) {
#pragma unroll
          for (int k = 0; k < 8; ++k) e[k] = (int)(signed char)((w[k >> 2] >> (8 * (k & 3))) & 0xFFu);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)
        theta[k] = reconstruct_ordinary2<PDT, ECC_BITS>(old_lp[k], mk(ef[2 * k], ef[2 * k + 1]), one2);
      if constexpr (PDT == FO_BF16) {
        // a value too small for the exponent-field shortcut (zero included)
        if (!(minabs8(old_lp) >= fast::Ordinary<PDT>::kMin)) {
          rare = true;
          if constexpr (REPAIR) {
            const uint32_t w[4] = {p0.x, p0.y, p0.z, p0.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              theta[k].x = repair_master<PDT, ECC_BITS>(w[k] & 0xFFFFu, e[2 * k]);
              theta[k].y = repair_master<PDT, ECC_BITS>(w[k] >> 16, e[2 * k + 1]);
            }
          }
        }
      }
    }
  }

  return rare;
}

// updated master weights -> parameter words and ECC words; same contract for REPAIR as hot_unpack
template <bool REPAIR, int PDT, int ECC_BITS>
FO_DEVI bool stored_form(const float2 (&theta)[4], uint32_t (&nw)[4], uint4& ecc_out) {
  using namespace fast2;
  bool rare = false;
#pragma unroll
  for (int k = 0; k < 4; ++k) nw[k] = 0u;
  ecc_out = make_uint4(0, 0, 0, 0);
  if constexpr (PDT != FO_F32) {
    float2 new_lp[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      nw[k] = pack2<PDT>(theta[k].x, theta[k].y);
      unpack2<PDT>(nw[k], new_lp[k].x, new_lp[k].y);
    }
    if constexpr (ECC_BITS != 0) {
      int ne[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) ecc_ordinary2<PDT, ECC_BITS>(theta[k], new_lp[k], ne[2 * k], ne[2 * k + 1]);
      {
        // outside these the exponent-field shortcut does not hold (tiny bf16 values), or the
        // update overflowed the 16-bit range and the reference clips the ECC
        bool odd = !(maxabs8(new_lp) <= 1.0e38f);
        if constexpr (PDT == FO_BF16) odd = odd || !(minabs8(new_lp) >= fast::Ordinary<PDT>::kMin);
        if (odd) {
          rare = true;
          if constexpr (REPAIR) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              ne[2 * k] = repair_ecc<PDT, ECC_BITS>(theta[k].x);
              ne[2 * k + 1] = repair_ecc<PDT, ECC_BITS>(theta[k].y);
            }
          }
        }
      }
      if constexpr (ECC_BITS == 16) {
        ecc_out.x = pack_halves(ne[0], ne[1]); ecc_out.y = pack_halves(ne[2], ne[3]);
        ecc_out.z = pack_halves(ne[4], ne[5]); ecc_out.w = pack_halves(ne[6], ne[7]);
      } else {
        ecc_out.x = pack_bytes(ne[0], ne[1], ne[2], ne[3]);
        ecc_out.y = pack_bytes(ne[4], ne[5], ne[6], ne[7]);
      }
    }
  }

  return rare;
}

// A warp whose 256 gradients are +-0 and whose moment codes are all 0, the lasting state of rows that
// never see a gradient (embedding rows of tokens that do not occur): the new moments are exactly zero
// and so is the update term, so the step is the weight decay alone, the new codes and scales are
// zeros.  Everything is read again from memory (the first pass has overwritten its registers with the
// results of 0/0 arithmetic).
// Returns false when a parameter lies outside the range of the packed split (the caller then takes
// the repairing pass); nothing has been stored in that case.
template <int OPT, int PDT, int ECC_BITS>
__device__ __noinline__ bool zero_chunk(const uint32_t flags, const float wd, const float decay, const int gdt, const float one,
                                        const char* p_grad, char* p_param, char* p_ecc, char* p_mu, char* p_nu, char* p_msc, char* p_vsc) {
  // (addresses and scalars by value: a structure passed by reference would have to live in local memory)
  using namespace fast2;
  const float2 one2 = sp(one);
  struct { const char* grad; char* param; char* ecc; char* mu; char* nu; char* msc; char* vsc; } at = {p_grad, p_param, p_ecc, p_mu, p_nu, p_msc, p_vsc};
  struct { uint32_t flags; float wd, decay; } h = {flags, wd, decay};
  // the test, on what is in memory: gradients +-0, all codes 0 (then the moments are zero whatever the
  // scales say), and no weight decay folded into the gradient
  if ((h.flags & FO_FLAG_DECOUPLED_WD) == 0 && h.wd != 0.0f) return false;
  {
    const uint4 g0 = __ldcs((const uint4*)at.grad);
    uint32_t any = (g0.x | g0.y | g0.z | g0.w) & (gdt == FO_F32 ? 0x7FFFFFFFu : 0x7FFF7FFFu);
    if (gdt == FO_F32) {
      const uint4 g1 = __ldcs((const uint4*)at.grad + 1);
      any |= (g1.x | g1.y | g1.z | g1.w) & 0x7FFFFFFFu;
    }
    const uint2 mq = __ldcs((const uint2*)at.mu);
    any |= mq.x | mq.y;
    if constexpr (OPT == FO_OPT_ADAM) {
      const uint2 vq = __ldcs((const uint2*)at.nu);
      any |= vq.x | vq.y;
    }
    if (!__all_sync(0xFFFFFFFFu, any == 0u)) return false;
  }
  uint4 p0, p1 = make_uint4(0, 0, 0, 0), e = make_uint4(0, 0, 0, 0);
  p0 = __ldcs((const uint4*)at.param);
  if constexpr (PDT == FO_F32) p1 = __ldcs((const uint4*)at.param + 1);
  if constexpr (ECC_BITS == 16) e = __ldcs((const uint4*)at.ecc);
  if constexpr (ECC_BITS == 8) {
    const uint2 t = __ldcs((const uint2*)at.ecc);
    e.x = t.x; e.y = t.y;
  }
  float2 theta[4];
  bool rare = unpack_master<false, PDT, ECC_BITS>(p0, p1, e, one2, theta);
  if (OPT == FO_OPT_LION || (h.flags & FO_FLAG_DECOUPLED_WD) != 0) {
#pragma unroll
    for (int k = 0; k < 4; ++k) theta[k] = mul2(theta[k], sp(h.decay));
  }
  uint32_t nw[4];
  uint4 ecc_out;
  rare = stored_form<false, PDT, ECC_BITS>(theta, nw, ecc_out) || rare;
  if (__any_sync(0xFFFFFFFFu, rare)) return false;
  if constexpr (PDT == FO_F32) {
    __stcs((float4*)at.param, make_float4(theta[0].x, theta[0].y, theta[1].x, theta[1].y));
    __stcs((float4*)at.param + 1, make_float4(theta[2].x, theta[2].y, theta[3].x, theta[3].y));
  } else {
    __stcs((uint4*)at.param, make_uint4(nw[0], nw[1], nw[2], nw[3]));
    if constexpr (ECC_BITS == 16) __stcs((uint4*)at.ecc, ecc_out);
    if constexpr (ECC_BITS == 8) __stcs((uint2*)at.ecc, make_uint2(ecc_out.x, ecc_out.y));
  }
  __stcs((uint2*)at.mu, make_uint2(0u, 0u));
  *(__half*)at.msc = __float2half_rn(0.0f);
  if constexpr (OPT == FO_OPT_ADAM) {
    __stcs((uint2*)at.nu, make_uint2(0u, 0u));
    *(__half*)at.vsc = __float2half_rn(0.0f);
  }
  return true;
}

// REPAIR = false: straight-line code; returns true when a value lies outside a shortcut's proven
// range (the results are then not to be stored).  REPAIR = true: the affected lane redoes the stage
// with IEEE operations and the results are always good.
template <bool REPAIR, int OPT, int PDT, int ECC_BITS, int STATE>
FO_DEVI bool hot_unpack(const Raw<OPT, PDT, ECC_BITS, STATE>& r, const int gdt, const float* lut_mw, const float one, Unpacked& u) {
  using namespace fast2;
  const float2 one2 = sp(one);
  bool rare = false;
  if (gdt == FO_F32) pairs_of(r.g0, r.g1, u.g);
  else if (gdt == FO_BF16) pairs_of16<FO_BF16>(r.g0, u.g);
  else pairs_of16<FO_F16>(r.g0, u.g);

  rare = unpack_master<REPAIR, PDT, ECC_BITS>(r.p0, r.p1, r.e, one2, u.theta);

  if constexpr (STATE == FO_STATE_QUANT) {
    const float2 msc = sp(__half2float(r.msc));
    const uint32_t mw[2] = {r.mq.x, r.mq.y};
#pragma unroll
    for (int k = 0; k < 4; ++k)  // quantization.py:52-55
      u.m[k] = mul2(mk(lut_mw[byte_of(mw[k >> 1], 2 * (k & 1)) * kLutCopies], lut_mw[byte_of(mw[k >> 1], 2 * (k & 1) + 1) * kLutCopies]), msc);
    if constexpr (OPT == FO_OPT_ADAM) {
      const float2 vsc = sp(__half2float(r.vsc));
      const uint32_t vw[2] = {r.vq.x, r.vq.y};
#pragma unroll
      for (int k = 0; k < 4; ++k) {  // quantization.py:74-77
        const float2 nrm = codes_over_255(vw[k >> 1], 2 * (k & 1));
        const float2 s = mul2(nrm, vsc);
        u.v[k] = mul2(s, s);
      }
    }
  } else if constexpr (STATE == FO_STATE_FULL) {
    pairs_of(r.m0, r.m1, u.m);
    if constexpr (OPT == FO_OPT_ADAM) pairs_of(r.v0, r.v1, u.v);
  }
  return rare;
}

FO_DEVI void grad_pairs(const uint4& w0, const uint4& w1, const int gdt, float2 (&o)[4]) {
  if (gdt == FO_F32) pairs_of(w0, w1, o);
  else if (gdt == FO_BF16) pairs_of16<FO_BF16>(w0, o);
  else pairs_of16<FO_F16>(w0, o);
}

template <bool REPAIR>
FO_DEVI bool mean_of_sum(float2 (&g)[4], const int gdt, const Peers& peers);

// Reduce-scatter folded into the step (see Peers): g holds this rank's gradients on entry and the
// mean over the ranks, rounded to the gradient dtype, on return.  fetch(r, w0, w1) delivers the
// words of peer r's piece.  Same contract for REPAIR as hot_unpack.
template <bool REPAIR, typename Fetch>
FO_DEVI bool merge_peer_grads(float2 (&g)[4], const int gdt, const Peers& peers, Fetch fetch) {
  using namespace fast2;
  for (int r = 0; r < peers.ng; ++r) {
    uint4 w0, w1 = make_uint4(0u, 0u, 0u, 0u);
    fetch(r, w0, w1);
    float2 pg[4];
    grad_pairs(w0, w1, gdt, pg);
#pragma unroll
    for (int k = 0; k < 4; ++k) g[k] = add2(g[k], pg[k]);
  }
  return mean_of_sum<REPAIR>(g, gdt, peers);
}

// second half of the averaging: g holds the sum over the ranks on entry
template <bool REPAIR>
FO_DEVI bool mean_of_sum(float2 (&g)[4], const int gdt, const Peers& peers) {
  using namespace fast2;
  bool rare = false;
  float2 mean[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) mean[k] = div_by_rcp2(g[k], sp(peers.neg_ranks), sp(peers.rcp_ranks));
  // a rank count that is not a power of two: the residual of the reciprocal division underflows for tiny sums
  if (!peers.ranks_pow2 && !(minabs8(g) >= 7.8886091e-31f)) {
    rare = true;
    if constexpr (REPAIR) {
#pragma unroll
      for (int k = 0; k < 4; ++k) mean[k] = mk(fdiv(g[k].x, -peers.neg_ranks), fdiv(g[k].y, -peers.neg_ranks));
    }
  }
  if (gdt == FO_BF16) {
#pragma unroll
    for (int k = 0; k < 4; ++k) unpack2<FO_BF16>(pack2<FO_BF16>(mean[k].x, mean[k].y), g[k].x, g[k].y);
  } else if (gdt == FO_F16) {
#pragma unroll
    for (int k = 0; k < 4; ++k) unpack2<FO_F16>(pack2<FO_F16>(mean[k].x, mean[k].y), g[k].x, g[k].y);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) g[k] = mean[k];
  }
  return rare;
}

// Global-norm clipping of a piece (see Clip), for gradients already known to be rescaled.
// Same contract for REPAIR as hot_unpack.
template <bool REPAIR>
FO_DEVI bool clip_grads(float2 (&g)[4], const int gdt, const Clip& c) {
  using namespace fast2;
  // The reciprocal shortcut is exact for 2^-100 <= |g| <= 2^100, and for zeros up to their sign,
  // which is put back below.  Magnitude bits minus one, as unsigned: zero wraps to the top and passes.
  uint32_t lo = 0xFFFFFFFFu, hi = 0u;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t a = (__float_as_uint(g[k].x) & 0x7FFFFFFFu) - 1u, b = (__float_as_uint(g[k].y) & 0x7FFFFFFFu) - 1u;
    lo = min(lo, min(a, b));
    hi = max(hi, max(a + 1u, b + 1u));
  }
  const bool rare = !c.div_ok || lo < 0x0D800000u - 1u || hi > 0x71800000u;  // 2^-100, 2^100
  float2 q[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    q[k] = div_by_rcp2(g[k], sp(-c.n_g), sp(c.rcp_n));
    q[k] = mk(copysignf(q[k].x, g[k].x), copysignf(q[k].y, g[k].y));
  }
  if constexpr (REPAIR) {
    if (rare) {
#pragma unroll
      for (int k = 0; k < 4; ++k) q[k] = mk(fdiv(g[k].x, c.n_g), fdiv(g[k].y, c.n_g));
    }
  }
  if (gdt == FO_BF16) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      unpack2<FO_BF16>(pack2<FO_BF16>(q[k].x, q[k].y), q[k].x, q[k].y);
      q[k] = mul2(q[k], sp(c.m_g));
      unpack2<FO_BF16>(pack2<FO_BF16>(q[k].x, q[k].y), g[k].x, g[k].y);
    }
  } else if (gdt == FO_F16) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      unpack2<FO_F16>(pack2<FO_F16>(q[k].x, q[k].y), q[k].x, q[k].y);
      q[k] = mul2(q[k], sp(c.m_g));
      unpack2<FO_F16>(pack2<FO_F16>(q[k].x, q[k].y), g[k].x, g[k].y);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) g[k] = mul2(q[k], sp(c.m_g));
  }
  return rare;
}

FO_DEVI float sign_of(float x);

template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__device__ __noinline__ void warm_chunk(const DevLeaf& L, const Hyp& h, const int gdt, const uint32_t base,
                                        const float one, const float* lut_mw, const Peers& peers, const Clip* clip);

// Second half of a hot chunk: update, split, requantize, store.  Each stage runs its packed
// shortcut unconditionally.
// REPAIR = false (first pass): a value outside the range a shortcut is proven for only raises
// `rare`; nothing is stored until the end, and if any lane of the warp saw such a value the warp's
// 256 elements are redone from memory by warm_chunk, otherwise the results are written.
// REPAIR = true (warm_chunk): the lane that holds such a value (exact zeros are the common case:
// untouched rows, padding, zero gradients) redoes that stage with IEEE operations, then stores.
// The stored bits are those of the IEEE path in every case.
template <bool REPAIR, int OPT, int PDT, int ECC_BITS, int STATE, bool AUX, bool MASKED = false>
FO_DEVI void hot_finish(const DevLeaf& L, const Hyp& h, const int gdt, const uint32_t base, const Piece& at, const float one,
                        bool rare, Unpacked& u, const float* lut_mw, const Peers& peers, const Clip* clip,
                        const int n_valid = kPiece, const bool group_valid = true) {
  using namespace fast2;
  const float2 one2 = sp(one);
  float2 (&g)[4] = u.g;
  float2 (&theta)[4] = u.theta;
  float2 (&m)[4] = u.m;
  float2 (&v)[4] = u.v;
  float2 nroot[4];  // Adam: -sqrt(second moment)

  // ---- update --------------------------------------------------------------------------------------
  const bool decoupled = (h.flags & FO_FLAG_DECOUPLED_WD) != 0;
  float am_lane = 0.0f, av_lane = 1.0f;
  if constexpr (OPT == FO_OPT_ADAM) {
    // flashoptim_jax/adamw.py:95-106
    if (!decoupled) {
#pragma unroll
      for (int k = 0; k < 4; ++k) g[k] = sum2(mul2(sp(h.wd), theta[k]), g[k], one2);
    }
    // The second moment and its square root are carried negated (nv = -v, nroot = -sqrt(v)):
    // the signs then fall where the packed residual corrections need them (see fo_math.cuh).
    float2 nv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      m[k] = sum2(mul2(sp(h.b1), m[k]), mul2(sp(h.omb1), g[k]), one2);
      nv[k] = sum2(mul2(sp(-h.b2), v[k]), mul2(sp(-h.omb2), mul2(g[k], g[k])), one2);
    }
    if constexpr (STATE == FO_STATE_FULL) {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = mul2(nv[k], sp(-1.0f));  // stored as it is
    }
    if (decoupled) {
#pragma unroll
      for (int k = 0; k < 4; ++k) theta[k] = mul2(theta[k], sp(h.decay));
    }
    const float2 sq = sp(h.sqrt_bc2), nrsq = sp(-h.rcp_sqrt_bc2), eps = sp(h.eps), lrb1 = sp(h.lr_bc1);
    float2 tn[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      nroot[k] = neg_sqrt_core2(nv[k]);
      const float2 den = add2(div_negnum_by_rcp2(nroot[k], sq, nrsq), eps);
      tn[k] = sum2(neg_div2(mul2(lrb1, m[k]), den), theta[k], one2);  // theta - (lr/bc1 * m) / den
    }
    // Ranges in which the packed square root and division are exact: second moment >= 1e-30 with
    // sqrt <= 2^30 (so the denominator lies in [eps, 2^47]) and numerator magnitudes in [2^-70, 2^60].
    am_lane = maxabs8(m);
    av_lane = -min8(nroot);
    // (with quantized moments the largest square root is checked once per group below, after the
    // shuffles; the repairing pass needs the answer per lane)
    bool wild = !(max8(nv) <= -1.0e-30f) || !(minabs8(m) >= h.m_lo) || !(am_lane <= h.m_hi);
    if constexpr (REPAIR || STATE != FO_STATE_QUANT) wild = wild || !(av_lane <= 1.0737418e9f);
    if (wild) {
      rare = true;
      if constexpr (REPAIR) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float rx, ry;
          tn[k].x = repair_adam(-nv[k].x, m[k].x, theta[k].x, h.lr_bc1, h.sqrt_bc2, h.eps, rx);
          tn[k].y = repair_adam(-nv[k].y, m[k].y, theta[k].y, h.lr_bc1, h.sqrt_bc2, h.eps, ry);
          nroot[k] = mk(-rx, -ry);
        }
        av_lane = -min8(nroot);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) theta[k] = tn[k];
  } else if constexpr (OPT == FO_OPT_LION) {
    // flashoptim_jax/momentum_kernel.py:77-79 or flashoptim_jax/lion.py:50-52
    float2 upd[4];
    if (h.flags & FO_FLAG_LION_LERP) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 d = fma2(m[k], sp(-1.0f), g[k]);  // g - m
        const float2 c = sum2(mul2(sp(h.omb1), d), m[k], one2);
        upd[k] = mk(sign_of(c.x), sign_of(c.y));
        m[k] = sum2(mul2(sp(h.omb2), d), m[k], one2);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 c = sum2(mul2(sp(h.b1), m[k]), mul2(sp(h.omb1), g[k]), one2);
        upd[k] = mk(sign_of(c.x), sign_of(c.y));
        m[k] = sum2(mul2(sp(h.b2), m[k]), mul2(sp(h.omb2), g[k]), one2);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) theta[k] = sum2(mul2(theta[k], sp(h.decay)), mul2(sp(-h.lr), upd[k]), one2);  // theta*decay - lr*upd
    am_lane = maxabs8(m);
  } else {
    // flashoptim_jax/momentum_kernel.py:74-75,80-86; flashoptim_jax/sgd.py:45-63
    if (!decoupled) {
#pragma unroll
      for (int k = 0; k < 4; ++k) g[k] = sum2(mul2(sp(h.wd), theta[k]), g[k], one2);
    }
    if constexpr (STATE != FO_STATE_NONE) {
#pragma unroll
      for (int k = 0; k < 4; ++k) m[k] = sum2(mul2(sp(h.b1), m[k]), mul2(sp(h.omb1), g[k]), one2);
      if (h.flags & FO_FLAG_NESTEROV) {
#pragma unroll
        for (int k = 0; k < 4; ++k) g[k] = sum2(mul2(sp(h.b1), m[k]), g[k], one2);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) g[k] = m[k];
      }
      am_lane = maxabs8(m);
    }
    if (decoupled) {
#pragma unroll
      for (int k = 0; k < 4; ++k) theta[k] = mul2(theta[k], sp(h.decay));
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) theta[k] = sum2(mul2(sp(-h.lr), g[k]), theta[k], one2);  // theta - lr*dir
  }

  // ---- parameter (+ECC) in stored form --------------------------------------------------------------
  uint32_t nw[4];
  uint4 ecc_out;
  rare = stored_form<REPAIR, PDT, ECC_BITS>(theta, nw, ecc_out) || rare;

  // ---- moments in stored form ------------------------------------------------------------------------
  uint2 mq = make_uint2(0, 0), vq = make_uint2(0, 0);
  float am = 0.0f, av = 0.0f;
  if constexpr (STATE == FO_STATE_QUANT) {
    const bool floor_mode = (h.flags & FO_FLAG_SCALE_FLOOR) != 0;
    am = group_max(am_lane);
    uint32_t q[8];
    const float2 nam = sp(-am), rm2 = sp(fast::rcp_rn(am));
#pragma unroll
    for (int k = 0; k < 4; ++k) softsign_code_bits2(div_by_rcp2(m[k], nam, rm2), one2, q[2 * k], q[2 * k + 1]);
    if (!(am >= 1.0e-12f && am <= 1.0e30f)) {  // all-zero group, or a scale outside the reciprocal's range
      rare = true;
      if constexpr (REPAIR) {
        const float safe = ieee::safe_scale(am, floor_mode);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          q[2 * k] = repair_code_m(m[k].x, safe);
          q[2 * k + 1] = repair_code_m(m[k].y, safe);
        }
      }
    }
    mq.x = pack_bytes(q[0], q[1], q[2], q[3]);
    mq.y = pack_bytes(q[4], q[5], q[6], q[7]);
    if constexpr (OPT == FO_OPT_ADAM) {
      av = group_max(av_lane);
      const float2 av2 = sp(av), nrv2 = sp(-fast::rcp_rn(av));
#pragma unroll
      for (int k = 0; k < 4; ++k) quant_v_bits2(nroot[k], av2, nrv2, one2, q[2 * k], q[2 * k + 1]);
      if (!(av >= 1.0e-12f && av <= 1.0737418e9f)) {  // 2^30: also the limit of the packed Adam division
        rare = true;
        if constexpr (REPAIR) {
          const float safe = ieee::safe_scale(av, floor_mode);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            q[2 * k] = repair_code_v(-nroot[k].x, safe);
            q[2 * k + 1] = repair_code_v(-nroot[k].y, safe);
          }
        }
      }
      vq.x = pack_bytes(q[0], q[1], q[2], q[3]);
      vq.y = pack_bytes(q[4], q[5], q[6], q[7]);
    }
  }

  // ---- first pass: one decision per warp -----------------------------------------------------------------
  (void)rare;
  if constexpr (!REPAIR) {
    if (__any_sync(0xFFFFFFFFu, rare)) {
      if constexpr (OPT == FO_OPT_ADAM && STATE == FO_STATE_QUANT && !AUX) {
        // no new first moment of the warp differs from zero: look whether the whole piece is at rest
        if (__all_sync(0xFFFFFFFFu, am_lane == 0.0f) && zero_chunk<OPT, PDT, ECC_BITS>(h.flags, h.wd, h.decay, gdt, one, at.grad, at.param, at.ecc, at.mu, at.nu, at.msc, at.vsc)) return;
      }
      warm_chunk<OPT, PDT, ECC_BITS, STATE, AUX>(L, h, gdt, base, one, lut_mw, peers, clip);
      return;
    }
  }
  // ---- stores ---------------------------------------------------------------------------------------------
  if constexpr (REPAIR && MASKED) {
    // the ragged end of a leaf (ragged_chunk only): the piece that straddles the end stores its
    // valid elements one by one, pieces beyond it store nothing; a group's scale is stored by the
    // lanes of a group that has an element at all
    if (n_valid < kPiece) {
      for (int j = 0; j < n_valid; ++j) {
        const float2 t = theta[j >> 1];
        if constexpr (PDT == FO_F32) {
          ((float*)at.param)[j] = (j & 1) ? t.y : t.x;
        } else {
          ((unsigned short*)at.param)[j] = (unsigned short)(nw[j >> 1] >> (16 * (j & 1)));
          const uint32_t ew[4] = {ecc_out.x, ecc_out.y, ecc_out.z, ecc_out.w};
          if constexpr (ECC_BITS == 16) ((unsigned short*)at.ecc)[j] = (unsigned short)(ew[j >> 1] >> (16 * (j & 1)));
          if constexpr (ECC_BITS == 8) ((unsigned char*)at.ecc)[j] = (unsigned char)(ew[j >> 2] >> (8 * (j & 3)));
        }
        if constexpr (STATE == FO_STATE_FULL) {
          ((float*)at.mu)[j] = (j & 1) ? m[j >> 1].y : m[j >> 1].x;
          if constexpr (OPT == FO_OPT_ADAM) ((float*)at.nu)[j] = (j & 1) ? v[j >> 1].y : v[j >> 1].x;
        } else if constexpr (STATE == FO_STATE_QUANT) {
          ((unsigned char*)at.mu)[j] = (unsigned char)(((j & 4) ? mq.y : mq.x) >> (8 * (j & 3)));
          if constexpr (OPT == FO_OPT_ADAM) ((unsigned char*)at.nu)[j] = (unsigned char)(((j & 4) ? vq.y : vq.x) >> (8 * (j & 3)));
        }
      }
      if constexpr (STATE == FO_STATE_QUANT) {
        if (group_valid) {
          *(__half*)at.msc = __float2half_rn(am);
          if constexpr (OPT == FO_OPT_ADAM) *(__half*)at.vsc = __float2half_rn(av);
        }
      }
      return;
    }
  }
  if constexpr (PDT == FO_F32) {
    const float4 lo = make_float4(theta[0].x, theta[0].y, theta[1].x, theta[1].y);
    const float4 hi = make_float4(theta[2].x, theta[2].y, theta[3].x, theta[3].y);
    if (AUX && peers.mc_pdelta != 0) {
      char* mc = at.param + peers.mc_pdelta;
      multicast_store(mc, make_uint4(__float_as_uint(lo.x), __float_as_uint(lo.y), __float_as_uint(lo.z), __float_as_uint(lo.w)));
      multicast_store(mc + 16, make_uint4(__float_as_uint(hi.x), __float_as_uint(hi.y), __float_as_uint(hi.z), __float_as_uint(hi.w)));
    } else {
      __stcs((float4*)at.param, lo);
      __stcs((float4*)at.param + 1, hi);
      if constexpr (AUX) {
        store_to_peers(peers, (float4*)at.param, lo);
        store_to_peers(peers, (float4*)at.param + 1, hi);
      }
    }
  } else {
    const uint4 w = make_uint4(nw[0], nw[1], nw[2], nw[3]);
    if (AUX && peers.mc_pdelta != 0) {
      multicast_store(at.param + peers.mc_pdelta, w);
    } else {
      __stcs((uint4*)at.param, w);
      if constexpr (AUX) store_to_peers(peers, (uint4*)at.param, w);
    }
    if constexpr (ECC_BITS == 16) __stcs((uint4*)at.ecc, ecc_out);
    if constexpr (ECC_BITS == 8) __stcs((uint2*)at.ecc, make_uint2(ecc_out.x, ecc_out.y));
  }
  if constexpr (STATE == FO_STATE_FULL) {
    __stcs((float4*)at.mu, make_float4(m[0].x, m[0].y, m[1].x, m[1].y));
    __stcs((float4*)at.mu + 1, make_float4(m[2].x, m[2].y, m[3].x, m[3].y));
    if constexpr (OPT == FO_OPT_ADAM) {
      __stcs((float4*)at.nu, make_float4(v[0].x, v[0].y, v[1].x, v[1].y));
      __stcs((float4*)at.nu + 1, make_float4(v[2].x, v[2].y, v[3].x, v[3].y));
    }
  } else if constexpr (STATE == FO_STATE_QUANT) {
    // the four lanes of a group all store its scale: same value to the same address, one
    // unpredicated instruction
    __stcs((uint2*)at.mu, mq);
    *(__half*)at.msc = __float2half_rn(am);
    if constexpr (OPT == FO_OPT_ADAM) {
      __stcs((uint2*)at.nu, vq);
      *(__half*)at.vsc = __float2half_rn(av);
    }
  }
}

// words of eight consecutive elements of which only the first n_valid exist (the rest read as zero)
template <int BYTES>
FO_DEVI void masked_words(const void* src, const int n_valid, uint32_t (&w)[2 * BYTES]) {
#pragma unroll
  for (int k = 0; k < 2 * BYTES; ++k) w[k] = 0u;
  for (int j = 0; j < n_valid; ++j) {
    if constexpr (BYTES == 4) w[j] = ((const uint32_t*)src)[j];
    if constexpr (BYTES == 2) w[j >> 1] |= (uint32_t)((const unsigned short*)src)[j] << (16 * (j & 1));
    if constexpr (BYTES == 1) w[j >> 2] |= (uint32_t)((const unsigned char*)src)[j] << (8 * (j & 3));
  }
}
template <int OPT, int PDT, int ECC_BITS, int STATE>
__device__ __noinline__ void masked_load(const Piece& at, const int gdt, const int n_valid, Raw<OPT, PDT, ECC_BITS, STATE>& r) {
  uint32_t w4[8], w2[4], w1[2];
  if constexpr (PDT == FO_F32) {
    masked_words<4>(at.param, n_valid, w4);
    r.p0 = make_uint4(w4[0], w4[1], w4[2], w4[3]); r.p1 = make_uint4(w4[4], w4[5], w4[6], w4[7]);
  } else {
    masked_words<2>(at.param, n_valid, w2);
    r.p0 = make_uint4(w2[0], w2[1], w2[2], w2[3]);
  }
  if constexpr (ECC_BITS == 16) { masked_words<2>(at.ecc, n_valid, w2); r.e = make_uint4(w2[0], w2[1], w2[2], w2[3]); }
  if constexpr (ECC_BITS == 8) { masked_words<1>(at.ecc, n_valid, w1); r.e.x = w1[0]; r.e.y = w1[1]; }
  if constexpr (STATE == FO_STATE_QUANT) {
    masked_words<1>(at.mu, n_valid, w1); r.mq = make_uint2(w1[0], w1[1]);
    if constexpr (OPT == FO_OPT_ADAM) { masked_words<1>(at.nu, n_valid, w1); r.vq = make_uint2(w1[0], w1[1]); }
  } else if constexpr (STATE == FO_STATE_FULL) {
    masked_words<4>(at.mu, n_valid, w4);
    r.m0 = make_uint4(w4[0], w4[1], w4[2], w4[3]); r.m1 = make_uint4(w4[4], w4[5], w4[6], w4[7]);
    if constexpr (OPT == FO_OPT_ADAM) {
      masked_words<4>(at.nu, n_valid, w4);
      r.v0 = make_uint4(w4[0], w4[1], w4[2], w4[3]); r.v1 = make_uint4(w4[4], w4[5], w4[6], w4[7]);
    }
  }
  if (gdt == FO_F32) {
    masked_words<4>(at.grad, n_valid, w4);
    r.g0 = make_uint4(w4[0], w4[1], w4[2], w4[3]); r.g1 = make_uint4(w4[4], w4[5], w4[6], w4[7]);
  } else {
    masked_words<2>(at.grad, n_valid, w2);
    r.g0 = make_uint4(w2[0], w2[1], w2[2], w2[3]);
  }
}

// The repairing pass with a limit, for a leaf's ragged last chunk and for leaves shorter than a chunk
// (called from the tail kernel only): elements from n_limit on do not exist; they read as
// zeros (flashoptim_jax/quantization.py:20-26) and nothing is stored for them.  Warps that lie wholly
// beyond the end return at once.  (Not with peer replicas: their stores are whole vectors.)
template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__device__ __noinline__ void ragged_chunk(const DevLeaf& L, const Hyp& h, const int gdt, const uint32_t base,
                                        const float one, const float* lut_mw, const Peers& peers, const Clip* clip,
                                        const uint32_t n_limit) {
  const uint32_t i0 = base + threadIdx.x * kPiece;
  if ((i0 & ~255u) >= n_limit) return;  // the warp's first element: the same answer in all its lanes
  const int n_valid = i0 >= n_limit ? 0 : (n_limit - i0 < (uint32_t)kPiece ? (int)(n_limit - i0) : kPiece);
  const bool group_valid = (i0 & ~31u) < n_limit;
  const Piece at = piece_at<PDT, ECC_BITS, STATE>(L, gdt, i0);
  Raw<OPT, PDT, ECC_BITS, STATE> raw;
  if (n_valid == kPiece) {
    hot_load<OPT, PDT, ECC_BITS, STATE>(L, gdt, i0, raw);
  } else {
    masked_load<OPT, PDT, ECC_BITS, STATE>(at, gdt, n_valid, raw);
    if constexpr (STATE == FO_STATE_QUANT) {
      raw.msc = group_valid ? *(const __half*)at.msc : __float2half(0.0f);
      if constexpr (OPT == FO_OPT_ADAM) raw.vsc = group_valid ? *(const __half*)at.vsc : __float2half(0.0f);
    }
  }
  Unpacked u;
  hot_unpack<true, OPT, PDT, ECC_BITS, STATE>(raw, gdt, lut_mw, one, u);
  if (AUX && peers.ng > 0) {
    merge_peer_grads<true>(u.g, gdt, peers, [&](int r, uint4& w0, uint4& w1) {
      const char* g = (const char*)L.grad + peers.gdelta[r];
      if (gdt == FO_F32) {
        w0 = __ldcs((const uint4*)((const float*)g + i0));
        w1 = __ldcs((const uint4*)((const float*)g + i0) + 1);
      } else {
        w0 = __ldcs((const uint4*)((const unsigned short*)g + i0));
      }
    });
  }
  if (AUX && clip->active) clip_grads<true>(u.g, gdt, *clip);
  hot_finish<true, OPT, PDT, ECC_BITS, STATE, AUX, true>(L, h, gdt, base, at, one, false, u, lut_mw, peers, clip, n_valid, group_valid);
}

// Second chance for a warp whose first pass met a value outside a shortcut's range: the same
// packed arithmetic from a fresh load, with per-lane IEEE repairs.  About twice the cost of a
// first pass for that warp, against about seven times for the scalar IEEE path.
template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__device__ __noinline__ void warm_chunk(const DevLeaf& L, const Hyp& h, const int gdt, const uint32_t base,
                                        const float one, const float* lut_mw, const Peers& peers, const Clip* clip) {
  Raw<OPT, PDT, ECC_BITS, STATE> raw;
  hot_load<OPT, PDT, ECC_BITS, STATE>(L, gdt, base + threadIdx.x * kPiece, raw);
  Unpacked u;
  hot_unpack<true, OPT, PDT, ECC_BITS, STATE>(raw, gdt, lut_mw, one, u);
  if (AUX && peers.ng > 0) {
    const uint32_t i0 = base + threadIdx.x * kPiece;
    merge_peer_grads<true>(u.g, gdt, peers, [&](int r, uint4& w0, uint4& w1) {
      const char* g = (const char*)L.grad + peers.gdelta[r];
      if (gdt == FO_F32) {
        w0 = __ldcs((const uint4*)((const float*)g + i0));
        w1 = __ldcs((const uint4*)((const float*)g + i0) + 1);
      } else {
        w0 = __ldcs((const uint4*)((const unsigned short*)g + i0));
      }
    });
  }
  if (AUX && clip->active) clip_grads<true>(u.g, gdt, *clip);
  const Piece at = piece_at<PDT, ECC_BITS, STATE>(L, gdt, base + threadIdx.x * kPiece);
  hot_finish<true, OPT, PDT, ECC_BITS, STATE, AUX>(L, h, gdt, base, at, one, false, u, lut_mw, peers, clip);
}

// One block's run of consecutive whole chunks [ch, hot_end) of a leaf, for the kernel without peer or
// clipping code.  Three stages of compile-time size; the loop body is unrolled three times, so
// that the stage an iteration reads and the one it fills are fixed, and the thread's addresses
// move once per three chunks: every access inside is a register plus an immediate.
template <int OPT, int PDT, int ECC_BITS, int STATE>
FO_DEVI void hot_run(const DevLeaf& L, const Hyp& h, const int gdt, const uint32_t ch, const uint32_t hot_end, const uint32_t stage0,
                     const float one, const float* lut_mw, const Peers& peers) {
  using S = Stage<OPT, PDT, ECC_BITS, STATE>;
  constexpr int kPsz = PDT == FO_F32 ? 4 : 2, kEsz = ECC_BITS == 16 ? 2 : 1;
  constexpr int kSsz = STATE == FO_STATE_FULL ? 4 : 1;   // bytes per element of a moment stream
  constexpr uint32_t kSB = (uint32_t)S::bytes(FO_F32, 0);  // room for the widest gradients, whatever they are
  const uint32_t n_it = hot_end - ch;
  uint32_t base = ch * (uint32_t)kChunk;
  uint32_t tid;
  asm volatile("mov.u32 %0, %%tid.x;" : "=r"(tid));  // read once: otherwise re-read at every use
  Piece at = piece_at<PDT, ECC_BITS, STATE>(L, gdt, base + tid * kPiece);
  const uint32_t s16 = stage0 + tid * 16u, s8 = stage0 + tid * 8u;
  const int gsz = gdt == FO_F32 ? 4 : 2;
  // copies of the chunk `ahead` chunks after the one `at` points to, into stage `slot`
  auto fill = [&](const int slot, const int ahead) {
    const uint32_t o = (uint32_t)slot * kSB;
    const char* pp = at.param + ahead * (kChunk * kPsz);
    if constexpr (PDT == FO_F32) {
      copy_async16_l1(s16 + o, pp);
      copy_async16_l1(s16 + o + 16u * kThreads, pp + 16);
    } else {
      copy_async16(s16 + o, pp);
    }
    if constexpr (ECC_BITS == 16) copy_async16(s16 + o + S::kOffEcc, at.ecc + ahead * (kChunk * kEsz));
    if constexpr (ECC_BITS == 8) copy_async8(s8 + o + S::kOffEcc, at.ecc + ahead * (kChunk * kEsz));
    if constexpr (STATE == FO_STATE_QUANT) {
      copy_async8(s8 + o + S::kOffMu, at.mu + ahead * kChunk);
      if constexpr (OPT == FO_OPT_ADAM) copy_async8(s8 + o + S::kOffNu, at.nu + ahead * kChunk);
    } else if constexpr (STATE == FO_STATE_FULL) {
      copy_async16_l1(s16 + o + S::kOffMu, at.mu + ahead * (kChunk * 4));
      copy_async16_l1(s16 + o + S::kOffMu + 16u * kThreads, at.mu + ahead * (kChunk * 4) + 16);
      if constexpr (OPT == FO_OPT_ADAM) {
        copy_async16_l1(s16 + o + S::kOffNu, at.nu + ahead * (kChunk * 4));
        copy_async16_l1(s16 + o + S::kOffNu + 16u * kThreads, at.nu + ahead * (kChunk * 4) + 16);
      }
    }
    if (gdt == FO_F32) {
      copy_async16_l1(s16 + o + S::kOffGrad, at.grad + ahead * (kChunk * 4));
      copy_async16_l1(s16 + o + S::kOffGrad + 16u * kThreads, at.grad + ahead * (kChunk * 4) + 16);
    } else {
      copy_async16(s16 + o + S::kOffGrad, at.grad + ahead * (kChunk * 2));
    }
  };
  auto read = [&](const int slot, Raw<OPT, PDT, ECC_BITS, STATE>& r) {
    const uint32_t o = (uint32_t)slot * kSB;
    r.p0 = lds128(s16 + o);
    if constexpr (PDT == FO_F32) r.p1 = lds128(s16 + o + 16u * kThreads);
    if constexpr (ECC_BITS == 16) r.e = lds128(s16 + o + S::kOffEcc);
    if constexpr (ECC_BITS == 8) {
      const uint2 t = lds64(s8 + o + S::kOffEcc);
      r.e.x = t.x; r.e.y = t.y;
    }
    if constexpr (STATE == FO_STATE_QUANT) {
      r.mq = lds64(s8 + o + S::kOffMu);
      if constexpr (OPT == FO_OPT_ADAM) r.vq = lds64(s8 + o + S::kOffNu);
    } else if constexpr (STATE == FO_STATE_FULL) {
      r.m0 = lds128(s16 + o + S::kOffMu);
      r.m1 = lds128(s16 + o + S::kOffMu + 16u * kThreads);
      if constexpr (OPT == FO_OPT_ADAM) {
        r.v0 = lds128(s16 + o + S::kOffNu);
        r.v1 = lds128(s16 + o + S::kOffNu + 16u * kThreads);
      }
    }
    r.g0 = lds128(s16 + o + S::kOffGrad);
    if (gdt == FO_F32) r.g1 = lds128(s16 + o + S::kOffGrad + 16u * kThreads);
  };
  constexpr int kS = kPlainStages;
#pragma unroll
  for (int k = 0; k < kS - 1; ++k) {
    if ((uint32_t)k < n_it) fill(k, k);
    copy_commit();
  }
  __half msc = __float2half(0.0f), vsc = msc;  // the group scales go through registers, one chunk ahead
  if constexpr (STATE == FO_STATE_QUANT) {
    msc = *(const __half*)at.msc;
    if constexpr (OPT == FO_OPT_ADAM) vsc = *(const __half*)at.vsc;
  }
  for (uint32_t it = 0; it < n_it; it += (uint32_t)kS) {
#pragma unroll
    for (int k = 0; k < kS; ++k) {
      if (it + (uint32_t)k >= n_it) break;
      if (it + (uint32_t)(k + kS - 1) < n_it) fill((k + kS - 1) % kS, k + kS - 1);
      copy_commit();
      copy_wait<kS - 1>();
      Raw<OPT, PDT, ECC_BITS, STATE> raw;
      read(k, raw);
      raw.msc = msc; raw.vsc = vsc;
      if constexpr (STATE == FO_STATE_QUANT) {
        if (it + (uint32_t)(k + 1) < n_it) {
          msc = *(const __half*)(at.msc + (k + 1) * (kChunk / 32 * 2));
          if constexpr (OPT == FO_OPT_ADAM) vsc = *(const __half*)(at.vsc + (k + 1) * (kChunk / 32 * 2));
        }
      }
      Unpacked u;
      const bool rare = hot_unpack<false, OPT, PDT, ECC_BITS, STATE>(raw, gdt, lut_mw, one, u);
      Piece cur;
      cur.grad = at.grad + k * (kChunk * gsz);
      cur.param = at.param + k * (kChunk * kPsz);
      cur.ecc = at.ecc + k * (kChunk * kEsz);
      cur.mu = at.mu + k * (kChunk * kSsz);
      cur.nu = at.nu + k * (kChunk * kSsz);
      cur.msc = at.msc + k * (kChunk / 32 * 2);
      cur.vsc = at.vsc + k * (kChunk / 32 * 2);
      hot_finish<false, OPT, PDT, ECC_BITS, STATE, false>(L, h, gdt, base + (uint32_t)k * kChunk, cur, one, rare, u, lut_mw, peers, nullptr);
    }
    base += (uint32_t)(kS * kChunk);
    at.grad += kS * kChunk * gsz;
    at.param += kS * kChunk * kPsz;
    if constexpr (ECC_BITS != 0) at.ecc += kS * kChunk * kEsz;
    if constexpr (STATE != FO_STATE_NONE) {
      at.mu += kS * kChunk * kSsz;
      if constexpr (OPT == FO_OPT_ADAM) at.nu += kS * kChunk * kSsz;
    }
    if constexpr (STATE == FO_STATE_QUANT) {
      at.msc += kS * (kChunk / 32 * 2);
      if constexpr (OPT == FO_OPT_ADAM) at.vsc += kS * (kChunk / 32 * 2);
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
// The momentum table once more in kLutCopies interleaved copies (entry of code b for lane l at
// b*kLutCopies + l % kLutCopies): the straight-line path looks eight random codes up per
// thread, and with a single copy a warp's 32 look-ups fall three deep on some bank.
FO_DEVI void build_wide_lut(const float* lut_m, float* lut_mw) {
  for (int i = threadIdx.x; i < 256 * kLutCopies; i += blockDim.x) lut_mw[i] = lut_m[i / kLutCopies];
  __syncthreads();
}

template <int OPT>
FO_DEVI bool leaf_is_hot(const StepParams& p, int l) {
#ifdef FO_NAIVE_MATH
  return false;
#else
  return p.aligned[l] != 0;
#endif
}

// The chunks [ch, end) of leaf l that the straight-line path does not take.  An aligned leaf under
// ordinary hyper-parameters goes through the repairing pass with a limit (vector accesses, masked at
// the leaf's end); the scalar path keeps unaligned leaves, the CPU-path parameter hand-back and peer
// replicas.  Out of line and fed by reference to the kernel's parameters, so that the persistent loop's
// register allocation does not see it.
template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__device__ __noinline__ void leaf_tail(const StepParams& p, const int l, uint32_t ch, const uint32_t end, const float* lut_all,
                                       const Clip* clip) {
  const DevLeaf& L = p.leaf[l];
  const Hyp h = load_hyper<OPT>(p.hyper[p.hyper_of[l]]);
  const float* lut_m = lut_all;
  const float* lut_v = lut_all + 256;
  const float* lut_mw = lut_all + 512 + (STATE == FO_STATE_QUANT ? (threadIdx.x & (kLutCopies - 1)) : 0);
  bool hyper_ok = (h.flags & FO_FLAG_LP_DELTA) == 0;  // as in the kernel: what the straight-line arithmetic may take
  if constexpr (OPT == FO_OPT_ADAM) hyper_ok = hyper_ok && (h.flags & kFlagTameAdam) != 0;
  const bool vector_ok = leaf_is_hot<OPT>(p, l) && hyper_ok &&
                         (!AUX || (p.peers.n == 0 && p.peers.ng == 0 && p.peers.mc_pdelta == 0 && p.peers.mc_gdelta == 0));
  Clip none;
  none.active = false; none.div_ok = true; none.n_g = 1.0f; none.rcp_n = 1.0f; none.m_g = 1.0f;
  for (; ch < end; ++ch) {
    if (vector_ok)
      ragged_chunk<OPT, PDT, ECC_BITS, STATE, AUX>(L, h, p.grad_dtype, ch * (uint32_t)kChunk, p.one, lut_mw, p.peers, clip, (uint32_t)L.n);
    else
      cold_chunk<OPT, PDT, ECC_BITS, STATE>(L, h, p.grad_dtype, (unsigned long long)ch * kChunk, lut_m, lut_v, p.peers, clip != nullptr ? *clip : none);
  }
}

// Second walk over the runs of this block, for what the straight-line loop of step_kernel skipped.
template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__device__ __noinline__ void block_tails(const StepParams& p, const float* lut_all) {
  const Clip clip = load_clip(AUX ? p.sq_norm : nullptr, p.max_norm, p.grad_dtype);
  const uint32_t total = p.first_block[p.n_leaves];
  for (uint32_t run0 = blockIdx.x * p.run_chunks; run0 < total; run0 += gridDim.x * p.run_chunks) {
    uint32_t c = run0;
    const uint32_t c_hi = min(total, run0 + p.run_chunks);
    int l_first = 0;
    for (int l_end = p.n_leaves; l_end - l_first > 1;) {
      const int mid = (l_first + l_end) >> 1;
      if (p.first_block[mid] <= c) l_first = mid; else l_end = mid;
    }
    for (int l = l_first; l < p.n_leaves && c < c_hi; ++l) {
      const uint32_t first = p.first_block[l];
      const uint32_t next = min(p.first_block[l + 1], c_hi);
      if (c >= next) continue;
      const uint32_t end = next - first;
      uint32_t ch = c - first;
      const uint32_t flags = p.hyper[p.hyper_of[l]].dyn != nullptr ? load_hyper<OPT>(p.hyper[p.hyper_of[l]]).flags : p.hyper[p.hyper_of[l]].flags;
      bool hyper_ok = (flags & FO_FLAG_LP_DELTA) == 0;
      if constexpr (OPT == FO_OPT_ADAM) hyper_ok = hyper_ok && (flags & kFlagTameAdam) != 0;
      const uint32_t hot_end = (leaf_is_hot<OPT>(p, l) && hyper_ok) ? min(end, (uint32_t)(p.leaf[l].n / kChunk)) : 0u;
      if (ch < hot_end) ch = hot_end;  // those were done
      if (ch < end) leaf_tail<OPT, PDT, ECC_BITS, STATE, AUX>(p, l, ch, end, lut_all, AUX ? &clip : nullptr);
      c = next;
    }
  }
}

// Persistent grid.  The chunks of all leaves form one sequence (first_block[] gives each leaf's
// first position in it) and block b takes positions b, b + grid, b + 2*grid, ...: at any moment
// the blocks work on neighbouring chunks, which keeps the DRAM pages they stream from few.
// Every block walks the leaves in order.  Inside a leaf its whole aligned chunks are taken by
// the straight-line path with nothing per chunk but a counter and the prefetch of the block's
// next chunk; what is left (a ragged last chunk, unaligned leaves, hyper-parameter sets outside
// the shortcuts' range) goes to the scalar IEEE path.
// AUX: the instantiation that also averages the peers' gradients and / or clips by the global
// norm; the plain one carries none of that code or state.
template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__global__ void __launch_bounds__(kThreads, min_blocks(OPT)) step_kernel(const __grid_constant__ StepParams p) {
  // one array for the three tables, so that the out-of-line paths need one pointer: [0, 256) momentum,
  // [256, 512) second moment, [512, 512 + 256 * kLutCopies) the interleaved momentum copies
  __shared__ float lut_all[512 + (STATE == FO_STATE_QUANT ? 256 * kLutCopies : 1)];
  float* const lut_m = lut_all;
  float* const lut_v = lut_all + 256;
  float* const lut_m_wide = lut_all + 512;
  if constexpr (STATE == FO_STATE_QUANT) {
    build_luts(lut_m, lut_v);
    build_wide_lut(lut_m, lut_m_wide);
  }
  const float* lut_mw = lut_m_wide + (STATE == FO_STATE_QUANT ? (threadIdx.x & (kLutCopies - 1)) : 0);
  extern __shared__ __align__(16) unsigned char stage_mem[];  // p.stages stages of Stage::bytes(grad dtype)
  using S = Stage<OPT, PDT, ECC_BITS, STATE>;
  // gradients summed in the NVLink switch (16-bit gradients only; fp32 leaves take the point-to-point route)
  const bool switch_sum = AUX && p.peers.mc_gdelta != 0 && p.grad_dtype != FO_F32;
  const int ng = (AUX && !switch_sum) ? p.peers.ng : 0;
  const uint32_t stage_bytes = (uint32_t)S::bytes(p.grad_dtype, ng);
  const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(stage_mem);
  const uint32_t stage_end = stage0 + (uint32_t)p.stages * stage_bytes;
  // Ring of kSwitchBatch thread-private slots behind the stages.  A multicast load-reduce takes
  // several microseconds and no asynchronous copy can issue one, so each thread keeps a batch of
  // them in registers: at every kSwitchBatch-th iteration it parks the batch that has arrived in
  // the ring (the sums for this and the next iterations) and issues the next batch.
  const uint32_t ring0 = stage_end;
  const uint32_t toff = threadIdx.x * kPiece;
  const Clip clip = load_clip(AUX ? p.sq_norm : nullptr, p.max_norm, p.grad_dtype);
  // The chunks of all leaves form one sequence, cut into runs of p.run_chunks consecutive chunks; block b
  // takes runs b, b + grid, b + 2 grid, ...  Inside a run every address advances by compile-time
  // constants; dealing the runs out in turn spreads regions that cost more (rows at rest, ragged ends,
  // values outside the shortcuts' ranges) over all blocks.
  const uint32_t total = p.first_block[p.n_leaves];
  constexpr uint32_t grid = 1u;   // chunk stride inside a run
  for (uint32_t run0 = blockIdx.x * p.run_chunks; run0 < total; run0 += gridDim.x * p.run_chunks) {
  uint32_t c = run0;  // this block's next position in the sequence
  const uint32_t c_hi = min(total, run0 + p.run_chunks);
  int l_first = 0;
  for (int l_end = p.n_leaves; l_end - l_first > 1;) {  // the leaf that holds position c
    const int mid = (l_first + l_end) >> 1;
    if (p.first_block[mid] <= c) l_first = mid; else l_end = mid;
  }
  for (int l = l_first; l < p.n_leaves; ++l) {
    const uint32_t first = p.first_block[l];
    if (c >= c_hi) break;
    const uint32_t next = min(p.first_block[l + 1], c_hi);
    if (c >= next) continue;
    const uint32_t end = next - first;  // chunks in this leaf
    uint32_t ch = c - first;            // this block's first chunk inside the leaf
    const DevLeaf& L = p.leaf[l];
    const Hyp h = load_hyper<OPT>(p.hyper[p.hyper_of[l]]);
    // the CPU-path parameter hand-back (FO_FLAG_LP_DELTA) needs the old stored value to the end: IEEE path only
    bool hyper_ok = (h.flags & FO_FLAG_LP_DELTA) == 0;
    if constexpr (OPT == FO_OPT_ADAM) hyper_ok = hyper_ok && (h.flags & kFlagTameAdam) != 0;  // the reciprocal shortcut in the denominator
    const uint32_t hot_end = (leaf_is_hot<OPT>(p, l) && hyper_ok) ? min(end, (uint32_t)(L.n / kChunk)) : 0u;  // whole chunks
    if constexpr (!AUX) {
      if (ch < hot_end) {
        hot_run<OPT, PDT, ECC_BITS, STATE>(L, h, p.grad_dtype, ch, hot_end, stage0, p.one, lut_mw, p.peers);
        ch = hot_end;
      }
    } else if (ch < hot_end) {
      const uint32_t stride = grid * (uint32_t)kChunk;
      uint32_t base = ch * (uint32_t)kChunk;
      // Copy pipeline: one group per chunk (empty past the end of the run, so that the count of
      // groups still pending always tells which chunk has landed).  The stage filled in an
      // iteration is the one read in the iteration before, whose values have been consumed.
      uint32_t fill_ch = ch, fill_base = base, wr = stage0;
      uint4 batch[kSwitchBatch] = {};
      uint32_t turn = 0;  // iteration number inside the run, modulo kSwitchBatch
      const char* mc_grad = (const char*)L.grad + p.peers.mc_gdelta;
      if (switch_sum) {
#pragma unroll
        for (int k = 0; k < kSwitchBatch; ++k)
          if (ch + (uint32_t)k * grid < hot_end)
            batch[k] = multicast_sum(mc_grad + (size_t)(base + (uint32_t)k * stride + toff) * 2u, p.grad_dtype);
      }
      for (int k = 1; k < p.stages; ++k) {
        if (fill_ch < hot_end) stage_fill<OPT, PDT, ECC_BITS, STATE>(L, p.grad_dtype, fill_base + toff, wr, p.peers, ng, !switch_sum);
        copy_commit();
        fill_ch += grid; fill_base += stride; wr += stage_bytes;
      }
      uint32_t rd = stage0;
      // the group scales go through registers, one chunk ahead
      __half msc = __float2half(0.0f), vsc = msc;
      if constexpr (STATE == FO_STATE_QUANT) {
        msc = ((const __half*)L.mu_scales)[(base + toff) >> 5];
        if constexpr (OPT == FO_OPT_ADAM) vsc = ((const __half*)L.nu_scales)[(base + toff) >> 5];
      }
      for (; ch < hot_end; ch += grid, base += stride) {
        if (switch_sum && turn == 0) {
#pragma unroll
          for (int k = 0; k < kSwitchBatch; ++k) {  // park what has arrived, ask for the batch after it
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(ring0 + (uint32_t)k * (16u * kThreads) + threadIdx.x * 16u),
                         "r"(batch[k].x), "r"(batch[k].y), "r"(batch[k].z), "r"(batch[k].w) : "memory");
            if (ch + (uint32_t)(kSwitchBatch + k) * grid < hot_end)
              batch[k] = multicast_sum(mc_grad + (size_t)(base + (uint32_t)(kSwitchBatch + k) * stride + toff) * 2u, p.grad_dtype);
          }
        }
        if (fill_ch < hot_end) stage_fill<OPT, PDT, ECC_BITS, STATE>(L, p.grad_dtype, fill_base + toff, wr, p.peers, ng, !switch_sum);
        copy_commit();
        fill_ch += grid; fill_base += stride;
        wr += stage_bytes;
        if (wr == stage_end) wr = stage0;
        if (!AUX || p.stages <= 3) {  // all but the oldest group may still be pending; local streams use 2 or 3 stages
          if (p.stages == 3) copy_wait<2>();
          else copy_wait<1>();
        } else switch (p.stages) {
          case 2: copy_wait<1>(); break;
          case 3: copy_wait<2>(); break;
          case 4: copy_wait<3>(); break;
          case 5: copy_wait<4>(); break;
          case 6: copy_wait<5>(); break;
          case 7: copy_wait<6>(); break;
          default: copy_wait<7>(); break;
        }
        Raw<OPT, PDT, ECC_BITS, STATE> raw;
        stage_read<OPT, PDT, ECC_BITS, STATE>(p.grad_dtype, rd, raw);
        const uint32_t peer_grads = rd + S::kOffGrad + (uint32_t)S::grad_bytes(p.grad_dtype);
        rd += stage_bytes;
        if (rd == stage_end) rd = stage0;
        raw.msc = msc; raw.vsc = vsc;
        if constexpr (STATE == FO_STATE_QUANT) {
          if (ch + grid < hot_end) {
            msc = ((const __half*)L.mu_scales)[(base + stride + toff) >> 5];
            if constexpr (OPT == FO_OPT_ADAM) vsc = ((const __half*)L.nu_scales)[(base + stride + toff) >> 5];
          }
        }
        Unpacked u;
        bool rare = hot_unpack<false, OPT, PDT, ECC_BITS, STATE>(raw, p.grad_dtype, lut_mw, p.one, u);
        if (switch_sum) {
          const uint4 sum = lds128(ring0 + turn * (16u * kThreads) + threadIdx.x * 16u);
          turn = turn + 1 == kSwitchBatch ? 0u : turn + 1;
          grad_pairs(sum, sum, p.grad_dtype, u.g);
          const bool odd = mean_of_sum<false>(u.g, p.grad_dtype, p.peers);
          rare = rare || odd;
        }
        if (AUX && ng > 0) {
          const bool odd = merge_peer_grads<false>(u.g, p.grad_dtype, p.peers, [&](int r, uint4& w0, uint4& w1) {
            const uint32_t at = peer_grads + (uint32_t)r * (uint32_t)S::grad_bytes(p.grad_dtype) + threadIdx.x * 16u;
            w0 = lds128(at);
            if (p.grad_dtype == FO_F32) w1 = lds128(at + 16u * kThreads);
          });
          rare = rare || odd;
        }
        if (AUX && clip.active) {
          const bool odd = clip_grads<false>(u.g, p.grad_dtype, clip);
          rare = rare || odd;
        }
        const Piece at = piece_at<PDT, ECC_BITS, STATE>(L, p.grad_dtype, base + toff);
        hot_finish<false, OPT, PDT, ECC_BITS, STATE, AUX>(L, h, p.grad_dtype, base, at, p.one, rare, u, lut_mw, p.peers, AUX ? &clip : nullptr);
      }
    }
    ch = end;  // the rest of the leaf in this run is taken after the loop (block_tails)
    c = first + ch;
  }
  }
  // What the loop left (ragged last chunks, leaves the straight-line path does not take) is the work of
  // step_tail_kernel, a launch of its own: measured on the 80-register Lion / SGD kernels, a call to
  // that code from this kernel, inside the leaf loop or after it, cost a quarter of their throughput
  // (spills in the loop, no uniform registers).
}

// The same walk over the same runs for what step_kernel skipped; launched after it with the same grid
// when the leaf table has a ragged end, an unaligned leaf or hyper-parameters outside the shortcuts'
// range (the launcher looks).
template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
__global__ void __launch_bounds__(kThreads, min_blocks(OPT)) step_tail_kernel(const __grid_constant__ StepParams p) {
  __shared__ float lut_all[512 + (STATE == FO_STATE_QUANT ? 256 * kLutCopies : 1)];
  if constexpr (STATE == FO_STATE_QUANT) {
    build_luts(lut_all, lut_all + 256);
    build_wide_lut(lut_all, lut_all + 512);
  }
  block_tails<OPT, PDT, ECC_BITS, STATE, AUX>(p, lut_all);
}

// ---- any group size (1..1024): one block per tile of whole groups, group maxima through
// shared-memory atomics on the (non-negative) float bit patterns; IEEE arithmetic only ------
template <int OPT, int PDT, int ECC_BITS>
__global__ void __launch_bounds__(256) step_kernel_generic(const __grid_constant__ StepParams p) {
  __shared__ float lut_m[256], lut_v[256];
  __shared__ unsigned int smax_m[kGenericTile], smax_v[kGenericTile];
  build_luts(lut_m, lut_v);
  const Clip clip = load_clip(p.sq_norm, p.max_norm, p.grad_dtype);
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
      const float g = clip_ieee(load_grad(L.grad, p.grad_dtype, i), clip, p.grad_dtype);
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

// elements one block of the any-group-size kernel covers
inline unsigned int generic_tile_elems(int group_size) {
  return (unsigned int)(kGenericTile / group_size > 0 ? kGenericTile / group_size : 1) * (unsigned int)group_size;
}

// grid of the persistent kernel: resident blocks per SM x SMs of the current device
struct LaunchInfo {
  unsigned int total_chunks;
  int sm_count;
};
using LaunchFn = cudaError_t (*)(const StepParams&, const LaunchInfo&, cudaStream_t);
// A kernel slice and the elements one of its chunks covers.  Block size, and with it the chunk, is a
// property of the slice (the slices are compiled with their own FO_THREADS): the host builds
// first_block[] from this number.
struct Launcher {
  LaunchFn launch;
  unsigned int chunk;
};

// Shared memory of one SM that blocks may use, and what each block loses to the system.
constexpr int kSmemPerSm = 227 * 1024, kSmemReservedPerBlock = 1024;

// whether a step needs the kernel that carries the peer and clipping code
inline bool step_needs_aux(const StepParams& p) {
  return p.peers.n > 0 || p.peers.ng > 0 || p.sq_norm != nullptr || p.peers.mc_pdelta != 0 || p.peers.mc_gdelta != 0;
}

template <int OPT, int PDT, int ECC_BITS, int STATE, bool AUX>
cudaError_t launch_step(const StepParams& p_in, const LaunchInfo& info, cudaStream_t s) {
  constexpr bool aux = AUX;
  if (step_needs_aux(p_in) != aux) return cudaErrorInvalidValue;
  const bool switch_sum = p_in.peers.mc_gdelta != 0 && p_in.grad_dtype != FO_F32;
  const int ring_bytes = switch_sum ? kSwitchBatch * 16 * kThreads : 0;
  auto kernel = step_kernel<OPT, PDT, ECC_BITS, STATE, AUX>;
  // Two caches, per instantiation of this function (one kernel each): the kernel's static shared memory
  // (the same on every device) and whether a device's copy of the function has been opted in above
  // 48 KB.  Atomics: concurrent first calls may both query and both set, which is harmless (same
  // values, idempotent calls), and no call ever reads a half-written entry.
  static std::atomic<int> static_smem_cache{-1};
  int static_smem = static_smem_cache.load(std::memory_order_acquire);
  if (static_smem < 0) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess) return e;
    static_smem = (int)attr.sharedSizeBytes;
    static_smem_cache.store(static_smem, std::memory_order_release);
  }
  // as many stages as fit beside the tables with min_blocks(OPT) blocks on an SM; when the peers'
  // gradient pieces make a stage too large for two of them, with one block on an SM
  // (the plain kernel runs three stages, each with room for fp32 gradients: see hot_run)
  const int per_stage = Stage<OPT, PDT, ECC_BITS, STATE>::bytes(aux ? p_in.grad_dtype : FO_F32, switch_sum ? 0 : p_in.peers.ng);
  int blocks_per_sm = min_blocks(OPT);
  int stages = (kSmemPerSm / blocks_per_sm - kSmemReservedPerBlock - static_smem - ring_bytes) / per_stage;
  while (stages < (aux ? 2 : kPlainStages) && blocks_per_sm > 1) {
    --blocks_per_sm;
    stages = (kSmemPerSm / blocks_per_sm - kSmemReservedPerBlock - static_smem - ring_bytes) / per_stage;
  }
  const int max_stages = !aux ? kPlainStages : ((p_in.peers.ng > 0 && !switch_sum) ? kMaxStagesPeers : kMaxStages);
  if (stages > max_stages) stages = max_stages;
  if (stages < (aux ? 2 : kPlainStages)) return cudaErrorInvalidConfiguration;
  const int dynamic_smem = stages * per_stage + ring_bytes;
  static std::atomic<bool> opted_in[64];  // per device ordinal (zero-initialised)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !opted_in[dev].load(std::memory_order_acquire)) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerSm - kSmemReservedPerBlock - static_smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) opted_in[dev].store(true, std::memory_order_release);
  }
  StepParams p = p_in;
  p.stages = stages;
  unsigned int grid = (unsigned int)info.sm_count * blocks_per_sm;
  if (grid > info.total_chunks) grid = info.total_chunks;
  // Run length: at most FO_RUN_MAX chunks (filling and draining the copy pipeline at a run's ends costs
  // about one chunk's time, 0.5 % of such a run), and for small launches a quarter of a block's share,
  // rounded up, so that no block gets more than four runs.
#ifndef FO_RUN_DIV
#define FO_RUN_DIV 4u
#endif
#ifndef FO_RUN_MAX
#define FO_RUN_MAX 192u
#endif
  unsigned int run = (info.total_chunks + grid * FO_RUN_DIV - 1u) / (grid * FO_RUN_DIV);
  // is there anything the straight-line loop leaves (a ragged end, a misaligned leaf, hyper-parameters
  // outside the shortcuts' range)?  Device-resident scalars can move Adam's hyper-parameters out of that
  // range at run time: then the tail kernel is launched to look for itself.
  bool dynamic = false;
  int tails = 0;  // leaves with work for the tail kernel
  for (int l = 0; l < p.n_leaves; ++l) {
    const DevHyper& h = p.hyper[p.hyper_of[l]];
    bool ok = (h.flags & FO_FLAG_LP_DELTA) == 0 && p.aligned[l] != 0;
    if (OPT == FO_OPT_ADAM) {
      ok = ok && (h.flags & kFlagTameAdam) != 0;
      dynamic = dynamic || h.dyn != nullptr;
    }
    if (!ok || p.leaf[l].n % (unsigned long long)kChunk != 0) ++tails;
  }
#ifdef FO_NAIVE_MATH
  tails = p.n_leaves;
#endif
  const bool ragged = tails > 0;
  // A launch of at most FO_RUN_WHOLE chunks per block with next to no tail work is dealt out as one run
  // per block: it lasts tens of microseconds, a second fill and drain of the pipeline per block shows
  // (4 M parameters: 31 -> 24 us), and an uneven count of short runs per block costs more than it
  // spreads.  (With many ragged leaves in the table the short runs stay: they spread the tail kernel's
  // work, which follows the same runs, over four times as many blocks.)
#ifndef FO_RUN_WHOLE
#define FO_RUN_WHOLE 32u
#endif
  const unsigned int share = (info.total_chunks + grid - 1u) / grid;
  if (share <= FO_RUN_WHOLE && tails <= 4) run = share;
  p.run_chunks = run < 1u ? 1u : (run > FO_RUN_MAX ? FO_RUN_MAX : run);
  kernel<<<grid, kThreads, dynamic_smem, s>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const bool need_tails = ragged || dynamic;
  if (need_tails) {
    step_tail_kernel<OPT, PDT, ECC_BITS, STATE, AUX><<<grid, kThreads, 0, s>>>(p);
    e = cudaGetLastError();
  }
  return e;
}
template <int OPT, int PDT, int ECC_BITS>
cudaError_t launch_step_generic(const StepParams& p, const LaunchInfo& info, cudaStream_t s) {
  step_kernel_generic<OPT, PDT, ECC_BITS><<<info.total_chunks, 256, 0, s>>>(p);
  return cudaGetLastError();
}

// lookups implemented by the instantiation units (fo_step_inst.cu, one per slice: optimizer x state
// kind x with / without the peer and clipping code); each returns {nullptr, 0} for a (param dtype,
// ecc width) pair that does not exist
#define FO_DECLARE_LOOKUP(name) Launcher name(int pdt, int ecc_bits);
#define FO_DECLARE_PAIR(stem) FO_DECLARE_LOOKUP(stem##_plain) FO_DECLARE_LOOKUP(stem##_aux)
FO_DECLARE_PAIR(lookup_adam_quant) FO_DECLARE_PAIR(lookup_adam_full) FO_DECLARE_LOOKUP(lookup_adam_generic)
FO_DECLARE_PAIR(lookup_lion_quant) FO_DECLARE_PAIR(lookup_lion_full) FO_DECLARE_LOOKUP(lookup_lion_generic)
FO_DECLARE_PAIR(lookup_sgd_quant) FO_DECLARE_PAIR(lookup_sgd_full) FO_DECLARE_LOOKUP(lookup_sgd_generic)
FO_DECLARE_PAIR(lookup_sgd_none)
#undef FO_DECLARE_PAIR
#undef FO_DECLARE_LOOKUP

}  // namespace fo
