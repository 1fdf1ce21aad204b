// Device self-checks: every arithmetic shortcut in fo_math.cuh (namespace fast) against the
// plain IEEE formulation (namespace ieee), exhaustively where the input space allows.
#include <mutex>

#include "fo_step.cuh"

namespace fo {
int fail(int code, const char* fmt, ...);

FO_DEVI bool same_float(float a, float b) {
  return __float_as_uint(a) == __float_as_uint(b) || (a != a && b != b);
}

FO_DEVI void tally(unsigned long long bad, unsigned long long* out) {
  for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xFFFFFFFFu, bad, o);
  if ((threadIdx.x & 31) == 0 && bad) atomicAdd(out, bad);
}

// every non-negative finite fp32, zero and subnormals included
__global__ void selftest_sqrt(const float one, unsigned long long* out) {
  unsigned long long bad = 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long b = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b < 0x7F800000ull; b += stride) {
    float v = __uint_as_float((uint32_t)b);
    bad += !same_float(fast::sqrt_rn(v), fsqrt(v));
    if (v >= 1.0e-30f) {
      bad += !same_float(fast::sqrt_core(v), fsqrt(v));
      const float w = __uint_as_float(0x7F7FFFFFu - (uint32_t)b + __float_as_uint(1.0e-30f));  // a second, unrelated lane
      const float2 r2 = fast2::neg_sqrt_core2(make_float2(-v, -w));
      bad += !same_float(r2.x, -fsqrt(v)) || !same_float(r2.y, -fsqrt(w));
    }
  }
  tally(bad, out);
}

// every fp32 with |n| <= 1: the int8 code through the shortcut division vs the IEEE one
__global__ void selftest_softsign(const float one, unsigned long long* out) {
  unsigned long long bad = 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long b = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b <= 0x3F800000ull; b += stride) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      float n = __uint_as_float((uint32_t)b | (s ? 0x80000000u : 0u));
      bad += fast::softsign_code(n) != ieee::quant_m(n, 1.0f);
      uint32_t c0, c1;
      fast2::softsign_code_bits2(make_float2(n, -n), fast2::sp(one), c0, c1);
      bad += (int)(signed char)(c0 & 0xFFu) != ieee::quant_m(n, 1.0f);
      bad += (int)(signed char)(c1 & 0xFFu) != ieee::quant_m(-n, 1.0f);
    }
  }
  tally(bad, out);
}

template <int PDT, int ECC_BITS>
__global__ void selftest_reconstruct(const float one, unsigned long long* out) {
  unsigned long long bad = 0;
  constexpr unsigned long long kEcc = 1ull << ECC_BITS;
  const unsigned long long total = 65536ull * kEcc;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    uint32_t bits = (uint32_t)(i / kEcc);
    int e = (int)(i % kEcc) - (int)(kEcc / 2);
    const float want = ieee::reconstruct<PDT, ECC_BITS>(bits, e);
    bad += !same_float(fast::reconstruct<PDT, ECC_BITS>(bits, e), want);
    const float lpf = Lp<PDT>::to_f32(bits);
    if (fabsf(lpf) >= fast::Ordinary<PDT>::kMin && fabsf(lpf) <= 3.0e38f)
    {
      bad += !same_float(fast::reconstruct_ordinary<PDT, ECC_BITS>(lpf, (float)e), want);
      const int en = (e == -(1 << (ECC_BITS - 1))) ? e : -e;  // the most negative pattern has no negation
      const float2 t2 = fast2::reconstruct_ordinary2<PDT, ECC_BITS>(make_float2(lpf, -lpf), make_float2((float)e, (float)en), fast2::sp(one));
      const float want_neg = ieee::reconstruct<PDT, ECC_BITS>(bits ^ 0x8000u, en);
      bad += !same_float(t2.x, want) || !same_float(t2.y, want_neg);
    }
  }
  tally(bad, out);
}

template <int PDT, int ECC_BITS>
__global__ void selftest_split(const float one, unsigned long long* out) {
  unsigned long long bad = 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long b = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b < (1ull << 32); b += stride) {
    float theta = __uint_as_float((uint32_t)b);
    if (theta != theta) continue;
    uint32_t b0, b1;
    int e0, e1;
    fast::split<PDT, ECC_BITS>(theta, b0, e0);
    ieee::split<PDT, ECC_BITS>(theta, b1, e1);
    bad += (b0 != b1) || (e0 != e1);
    const float lpf = Lp<PDT>::to_f32(b1);
    if (fabsf(lpf) >= fast::Ordinary<PDT>::kMin && fabsf(lpf) <= 3.0e38f)
    {
      bad += fast::ecc_ordinary<PDT, ECC_BITS>(theta, lpf) != e1;
      int p0, p1;
      fast2::ecc_ordinary2<PDT, ECC_BITS>(make_float2(theta, -theta), make_float2(lpf, -lpf), p0, p1);
      bad += (p0 != e1) || (p1 != -e1);
    }
    // the packed conversion the hot path uses must agree with the scalar one
    float lo, hi;
    unpack2<PDT>(pack2<PDT>(theta, -theta), lo, hi);
    bad += !same_float(lo, lpf) || !same_float(hi, -lpf);
  }
  tally(bad, out);
}

FO_DEVI uint32_t mix(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return (uint32_t)x;
}

// random (value, group scale) pairs with |value| <= scale: codes through the reciprocal
// shortcut vs the IEEE divisions; and the Adam denominator sqrt(nu)/sqrt(bc2) + eps.
__global__ void selftest_group_div(const float one, unsigned long long pairs, unsigned long long* out) {
  unsigned long long bad = 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += stride) {
    uint32_t r0 = mix(i * 4 + 0), r1 = mix(i * 4 + 1), r2 = mix(i * 4 + 2), r3 = mix(i * 4 + 3);
    // scale: random mantissa, exponent field in [28, 226] (about 1e-30 .. 1e30)
    float safe = __uint_as_float(((28u + r0 % 199u) << 23) | (r1 & 0x7FFFFFu));
    // value: scale shrunk by a random factor in (0, 1], heavy weight near 1 and across 40 binades
    float frac = __uint_as_float(((127u - (r2 >> 8) % ((r2 & 1u) ? 2u : 40u)) << 23) | (r3 & 0x7FFFFFu));
    float x = fminf(fmul(safe, fmul(frac, 0.5f)), safe);
    if (r2 & 2u) x = safe;  // the group maximum itself
    fast::GroupScale gs = fast::group_scale(safe, false);
    bad += fast::quant_m(x, gs) != ieee::quant_m(x, safe);
    bad += fast::quant_m(-x, gs) != ieee::quant_m(-x, safe);
    bad += fast::quant_v(x, gs) != ieee::quant_v(x, safe);
    if (gs.tame) {
      uint32_t c0, c1;
      fast2::softsign_code_bits2(fast2::div_by_rcp2(make_float2(x, -x), fast2::sp(-safe), fast2::sp(gs.rcp)), fast2::sp(one), c0, c1);
      bad += (int)(signed char)(c0 & 0xFFu) != ieee::quant_m(x, safe);
      bad += (int)(signed char)(c1 & 0xFFu) != ieee::quant_m(-x, safe);
      fast2::quant_v_bits2(make_float2(-x, -safe), fast2::sp(safe), fast2::sp(-gs.rcp), fast2::sp(one), c0, c1);
      bad += (int)(c0 & 0xFFu) != ieee::quant_v(x, safe);
      bad += (int)(c1 & 0xFFu) != 255;
      bad += (int)(signed char)(fast::softsign_code_bits(fast::div_by_rcp(x, safe, gs.rcp)) & 0xFFu) != ieee::quant_m(x, safe);
      bad += !same_float(gs.rcp, __frcp_rn(safe));
    }
    // Adam denominator: sqrt_bc2 in [2^-16, 2), eps in [1e-12, 1], root anywhere in [0, 1e30]
    float sq = __uint_as_float(((111u + r1 % 17u) << 23) | (r0 & 0x7FFFFFu));
    float eps = __uint_as_float(((87u + r3 % 40u) << 23) | (r2 & 0x7FFFFFu));
    float root = (r0 & 4u) ? x : __uint_as_float(((r2 >> 3) % 227u << 23) | (r1 & 0x7FFFFFu));
    {
      // the update division: numerator magnitude in [2^-70, 2^60], denominator in [2^-39, 2^47]
      const float num = __uint_as_float((r3 & 0x80000000u) | ((57u + r1 % 131u) << 23) | (r2 & 0x7FFFFFu));
      const float den = __uint_as_float(((88u + r0 % 86u) << 23) | (r3 & 0x7FFFFFu));
      const float den2 = __uint_as_float(((88u + r2 % 86u) << 23) | (r1 & 0x7FFFFFu));
      const float2 q = fast2::neg_div2(make_float2(num, -num), make_float2(den, den2));
      bad += !same_float(q.x, fdiv(-num, den)) || !same_float(q.y, fdiv(num, den2));
    }
    if (adam_is_tame(eps, sq)) {
      float a = fadd(fast::div_by_rcp(root, sq, __frcp_rn(sq)), eps);
      float b = fadd(fdiv(root, sq), eps);
      bad += !same_float(a, b);
    }
  }
  tally(bad, out);
}

// every float in [1e-30, 1e30]: reciprocal by MUFU.RCP + k correction steps vs the IEEE one.
// out[0] counts mismatches of the variant the kernels use, out[1] of one step, out[2] of two.
__global__ void selftest_rcp(unsigned long long* out) {
  unsigned long long bad0 = 0, bad1 = 0, bad2 = 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long lo = __float_as_uint(1.0e-30f), hi = __float_as_uint(1.0e30f);
  for (unsigned long long b = lo + (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b <= hi; b += stride) {
    const float s = __uint_as_float((uint32_t)b);
    const float want = __frcp_rn(s);
    bad0 += !same_float(fast::rcp_rn(s), want);
    {  // the packed form, which starts from the reciprocal of -s
      const float2 ny = fast2::neg_rcp2(make_float2(s, s));
      bad0 += !same_float(ny.x, -want) || !same_float(ny.y, -want);
    }
    bad1 += !same_float(fast::rcp_steps<1>(s), want);
    bad2 += !same_float(fast::rcp_steps<2>(s), want);
  }
  tally(bad0, out);
  tally(bad1, out + 1);
  tally(bad2, out + 2);
}

// Are "product then sum" sequences of packed operations kept as two roundings?
// out[0]: x*1 + y form (the one the kernels use), out[1]: plain add of a product.
__global__ void selftest_packed(const float one, unsigned long long pairs, unsigned long long* out) {
  unsigned long long bad0 = 0, bad1 = 0;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += stride) {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t r = mix(i * 8 + k);
      x[k] = __uint_as_float((r & 0x80000000u) | ((100u + (r >> 8) % 40u) << 23) | (mix(i * 8 + k + 77) & 0x7FFFFFu));
    }
    using namespace fast2;
    const f2 a = mk(x[0], x[1]), b = mk(x[2], x[3]), c = mk(x[4], x[5]), d = mk(x[6], x[7]);
    const float w0 = fadd(fmul(a.x, b.x), fmul(c.x, d.x)), w1 = fadd(fmul(a.y, b.y), fmul(c.y, d.y));
    const f2 s0 = sum2(mul2(a, b), mul2(c, d), sp(one));
    const f2 s1 = add2(mul2(a, b), mul2(c, d));
    bad0 += !same_float(s0.x, w0) || !same_float(s0.y, w1);
    bad1 += !same_float(s1.x, w0) || !same_float(s1.y, w1);
  }
  tally(bad0, out);
  tally(bad1, out + 1);
}

__global__ void selftest_code_tables(unsigned long long* out) {
  unsigned long long bad = 0;
  const int stride = gridDim.x * blockDim.x;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 65536; i += stride) {
    int e16 = i - 32768;
    bad += !same_float(fast::ecc_fraction<16>(e16), fdiv((float)e16, 32767.0f));
    if (i < 256) {
      int e8 = i - 128;
      bad += !same_float(fast::ecc_fraction<8>(e8), fdiv((float)e8, 127.0f));
      // second-moment codes in every byte position of a word, next to an unrelated neighbour
      const uint32_t j = (uint32_t)(255 - i);
      const float2 lo = fast2::codes_over_255((uint32_t)i | (j << 8) | 0xA5000000u, 0);
      const float2 hi = fast2::codes_over_255(0x5Au | (j << 16) | ((uint32_t)i << 24), 2);
      bad += !same_float(lo.x, ieee::deq_v_norm(i)) || !same_float(lo.y, ieee::deq_v_norm((int)j));
      bad += !same_float(hi.x, ieee::deq_v_norm((int)j)) || !same_float(hi.y, ieee::deq_v_norm(i));
    }
  }
  tally(bad, out);
}

// Is (which, arg) a sweep this library has?  Checked before anything is queued on the stream.
static int validate_sweep(const char* who, int32_t which, int64_t arg) {
  switch (which) {
    case FO_SELFTEST_SQRT: case FO_SELFTEST_SOFTSIGN: case FO_SELFTEST_GROUP_DIV: case FO_SELFTEST_CODE_TABLES:
    case FO_SELFTEST_RCP: case FO_SELFTEST_PACKED:
      return FO_OK;
    case FO_SELFTEST_RECONSTRUCT:
    case FO_SELFTEST_SPLIT: {
      const int pdt = (int)(arg / 100), eb = (int)(arg % 100);
      if ((pdt == FO_BF16 || pdt == FO_F16) && (eb == 8 || eb == 16)) return FO_OK;
      return fail(FO_ERR_INVALID_ARG, "%s: arg %lld names no (dtype, ecc) pair", who, (long long)arg);
    }
    default: return fail(FO_ERR_INVALID_ARG, "%s: unknown test %d", who, which);
  }
}

// The one dispatch table of the sweeps, shared by both entry points: launches sweep `which` with its
// mismatch counters at `d` (zeroed by the caller).  (which, arg) has passed validate_sweep.
static void launch_sweep(int32_t which, int64_t arg, unsigned long long* d, cudaStream_t s) {
  const int grid = 148 * 8, block = 256;
  volatile float one_src = 1.0f;  // a run-time 1.0f, as the step kernels receive it
  const float one = one_src;
  switch (which) {
    case FO_SELFTEST_SQRT: selftest_sqrt<<<grid, block, 0, s>>>(one, d); return;
    case FO_SELFTEST_SOFTSIGN: selftest_softsign<<<grid, block, 0, s>>>(one, d); return;
    case FO_SELFTEST_GROUP_DIV:
      selftest_group_div<<<grid, block, 0, s>>>(one, (unsigned long long)(arg > 0 ? arg : 1) * 1000000ull, d);
      return;
    case FO_SELFTEST_CODE_TABLES: selftest_code_tables<<<64, block, 0, s>>>(d); return;
    case FO_SELFTEST_RCP: selftest_rcp<<<grid, block, 0, s>>>(d); return;
    case FO_SELFTEST_PACKED: selftest_packed<<<grid, block, 0, s>>>(one, 1000000000ull, d); return;
    case FO_SELFTEST_RECONSTRUCT:
    case FO_SELFTEST_SPLIT: {
      const int pdt = (int)(arg / 100), eb = (int)(arg % 100);
#define X(P, E)                                                                                  \
  if (pdt == P && eb == E) {                                                                     \
    if (which == FO_SELFTEST_RECONSTRUCT) selftest_reconstruct<P, E><<<grid, block, 0, s>>>(one, d); \
    else selftest_split<P, E><<<grid, block, 0, s>>>(one, d);                                    \
    return;                                                                                      \
  }
      X(FO_BF16, 8) X(FO_BF16, 16) X(FO_F16, 8) X(FO_F16, 16)
#undef X
      return;
    }
    default: return;
  }
}

}  // namespace fo

using namespace fo;

extern "C" int fo_selftest(int32_t which, int64_t arg, uint64_t* mismatches, void* cuda_stream) {
  if (mismatches == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_selftest: null result pointer");
  int rc = validate_sweep("fo_selftest", which, arg);
  if (rc != FO_OK) return rc;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  unsigned long long* d = nullptr;
  // the only allocation in the library: a test-only counter, freed before returning
  cudaError_t e = cudaMalloc(&d, 4 * sizeof(unsigned long long));
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_selftest: %s", cudaGetErrorString(e));
  cudaMemsetAsync(d, 0, 4 * sizeof(unsigned long long), s);
  launch_sweep(which, arg, d, s);
  e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  unsigned long long h[4] = {0, 0, 0, 0};
  if (e == cudaSuccess) e = cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) rc = fail(FO_ERR_CUDA, "fo_selftest: %s", cudaGetErrorString(e));
  // arg selects which counter of a multi-counter test is reported (FO_SELFTEST_RCP: 0 in use, 1 one step, 2 two steps)
  *mismatches = ((which == FO_SELFTEST_RCP || which == FO_SELFTEST_PACKED) && arg >= 0 && arg < 3) ? h[arg] : h[0];
  cudaFree(d);
  return rc;
}


// ---------------------------------------------------------------------------------------------
// fo_selftest_static: the same sweeps with the mismatch counters in a statically allocated
// device array instead of a cudaMalloc'd one.
//
// Some hosts of this library must not allocate device memory at call time: a framework that
// hands the whole GPU to its own allocator up front, a serving process that forbids
// cudaMalloc after start-up because its implicit device-wide synchronisation stalls other
// streams, or a plug-in sandbox in which the allocation calls are simply not permitted.  For
// them the only scratch the self-checks need, a few 64-bit counters, lives in the array below.
// Every GPU that loads the library carries these 32 bytes until the process exits.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned long long g_static_counters[FO_SELFTEST_STATIC_MAX_COUNTERS];

namespace fo {

// In host code `g_static_counters` is only a handle for the runtime, not an address a kernel
// may dereference; the device address is asked for once per device, with that device current.
static int static_counters_address(unsigned long long** out) {
  static unsigned long long* cache[64] = {nullptr};
  static std::mutex lock;
  std::lock_guard<std::mutex> guard(lock);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_selftest_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(FO_ERR_UNSUPPORTED, "fo_selftest_static: device ordinal %d beyond 63", dev);
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_counters);
    if (e != cudaSuccess || p == nullptr)
      return fail(FO_ERR_CUDA, "fo_selftest_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    cache[dev] = static_cast<unsigned long long*>(p);
  }
  *out = cache[dev];
  return FO_OK;
}

}  // namespace fo

extern "C" int fo_selftest_static(int32_t which, int64_t arg, uint64_t* counters, uint32_t n_counters, void* cuda_stream) {
  if (counters == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_selftest_static: null result pointer");
  if (n_counters == 0) return fail(FO_ERR_INVALID_ARG, "fo_selftest_static: n_counters is 0");
  if (n_counters > FO_SELFTEST_STATIC_MAX_COUNTERS)
    return fail(FO_ERR_TOO_LARGE, "fo_selftest_static: %u counters asked for, the static scratch holds %d", n_counters,
                FO_SELFTEST_STATIC_MAX_COUNTERS);
  int rc = validate_sweep("fo_selftest_static", which, arg);  // before the shared array is touched
  if (rc != FO_OK) return rc;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  unsigned long long* d = nullptr;
  rc = static_counters_address(&d);
  if (rc != FO_OK) return rc;
  // the array keeps what the previous call left: counters must start from zero
  cudaError_t e = cudaMemsetAsync(d, 0, FO_SELFTEST_STATIC_MAX_COUNTERS * sizeof(unsigned long long), s);
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_selftest_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
  launch_sweep(which, arg, d, s);
  e = cudaGetLastError();
  unsigned long long h[FO_SELFTEST_STATIC_MAX_COUNTERS] = {0};
  if (e == cudaSuccess) e = cudaMemcpyAsync(h, d, sizeof(h), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_selftest_static: %s", cudaGetErrorString(e));
  for (uint32_t i = 0; i < n_counters; ++i) counters[i] = h[i];
  return FO_OK;
}
