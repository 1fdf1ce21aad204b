// Stand-alone codecs over fp32 arrays: the pieces of the step that the reference also
// exposes on their own (quantize_* / dequantize_* of flashoptim_jax/quantization.py,
// split_leaf / reconstruct_leaf of flashoptim_jax/compression.py).  Used for state
// initialisation from existing moments, checkpoint export/import and tests; same device
// arithmetic as the step kernels.
#include "fo_step.cuh"

namespace fo {
int fail(int code, const char* fmt, ...);
constexpr int kCodecThreads = 256;

// One block per tile of whole groups (any group size 1..1024), group maxima through
// shared-memory atomics on non-negative float bit patterns.
template <bool VARIANCE>
__global__ void __launch_bounds__(256) quantize_kernel(const float* __restrict__ x, void* __restrict__ values,
                                                            __half* __restrict__ scales, unsigned long long n, int G,
                                                            int floor_mode) {
  __shared__ unsigned int smax[kGenericTile];
  const int groups_per_tile = max(1, kGenericTile / G);
  const int tile = groups_per_tile * G;
  const unsigned long long base = (unsigned long long)blockIdx.x * tile;
  for (int i = threadIdx.x; i < groups_per_tile; i += kCodecThreads) smax[i] = 0u;
  __syncthreads();
  constexpr int kPer = kGenericTile / kCodecThreads;
  float val[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int li = threadIdx.x + k * kCodecThreads;
    const unsigned long long i = base + li;
    val[k] = 0.0f;
    if (li < tile && i < n) {
      float v = x[i];
      val[k] = VARIANCE ? fast::sqrt_rn(v) : v;
      atomicMax(&smax[li / G], __float_as_uint(fabsf(val[k])));
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int li = threadIdx.x + k * kCodecThreads;
    const unsigned long long i = base + li;
    if (li < tile && i < n) {
      const float a = __uint_as_float(smax[li / G]);
      const fast::GroupScale gs = fast::group_scale(a, floor_mode != 0);
      if (VARIANCE) ((unsigned char*)values)[i] = (unsigned char)fast::quant_v(val[k], gs);
      else ((signed char*)values)[i] = (signed char)fast::quant_m(val[k], gs);
      if (li % G == 0) scales[i / G] = __float2half_rn(a);
    }
  }
}

template <bool VARIANCE>
__global__ void __launch_bounds__(kCodecThreads) dequantize_kernel(const void* __restrict__ values,
                                                              const __half* __restrict__ scales, float* __restrict__ out,
                                                              unsigned long long n, int G) {
  __shared__ float lut_m[256], lut_v[256];
  build_luts(lut_m, lut_v);
  const unsigned long long stride = (unsigned long long)gridDim.x * kCodecThreads;
  for (unsigned long long i = (unsigned long long)blockIdx.x * kCodecThreads + threadIdx.x; i < n; i += stride) {
    const float sc = __half2float(scales[i / G]);
    const unsigned int b = ((const unsigned char*)values)[i];
    if (VARIANCE) {
      float s = fmul(lut_v[b], sc);
      out[i] = fmul(s, s);
    } else {
      out[i] = fmul(lut_m[b], sc);
    }
  }
}

template <int PDT, int ECC_BITS>
__global__ void __launch_bounds__(kCodecThreads) split_kernel(const float* __restrict__ theta, unsigned short* __restrict__ lp,
                                                         void* __restrict__ ecc, unsigned long long n) {
  const unsigned long long stride = (unsigned long long)gridDim.x * kCodecThreads;
  for (unsigned long long i = (unsigned long long)blockIdx.x * kCodecThreads + threadIdx.x; i < n; i += stride) {
    uint32_t nb;
    int e = 0;
    if constexpr (ECC_BITS != 0) fast::split<PDT, ECC_BITS>(theta[i], nb, e);
    else nb = Lp<PDT>::from_f32(theta[i]);
    lp[i] = (unsigned short)nb;
    if constexpr (ECC_BITS == 16) ((short*)ecc)[i] = (short)e;
    if constexpr (ECC_BITS == 8) ((signed char*)ecc)[i] = (signed char)e;
  }
}

template <int PDT, int ECC_BITS>
__global__ void __launch_bounds__(kCodecThreads) reconstruct_kernel(const unsigned short* __restrict__ lp,
                                                               const void* __restrict__ ecc, float* __restrict__ theta,
                                                               unsigned long long n) {
  const unsigned long long stride = (unsigned long long)gridDim.x * kCodecThreads;
  for (unsigned long long i = (unsigned long long)blockIdx.x * kCodecThreads + threadIdx.x; i < n; i += stride) {
    int e = 0;
    if constexpr (ECC_BITS == 16) e = ((const short*)ecc)[i];
    if constexpr (ECC_BITS == 8) e = ((const signed char*)ecc)[i];
    if constexpr (ECC_BITS != 0) theta[i] = fast::reconstruct<PDT, ECC_BITS>(lp[i], e);
    else theta[i] = Lp<PDT>::to_f32(lp[i]);
  }
}

static unsigned int stride_grid(unsigned long long n) {
  unsigned long long b = (n + kCodecThreads - 1) / kCodecThreads;
  const unsigned long long cap = 148ull * 8ull * 4ull;
  return (unsigned int)(b < cap ? (b ? b : 1) : cap);
}

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return FO_OK;
}

template <bool VARIANCE>
static int quantize_entry(const float* x, void* values, void* scales, uint64_t n, int32_t G, int32_t floor_mode, void* stream,
                          const char* what) {
  if (n == 0) return FO_OK;
  if (x == nullptr || values == nullptr || scales == nullptr) return fail(FO_ERR_INVALID_ARG, "%s: null pointer", what);
  if (G < 1) return fail(FO_ERR_INVALID_ARG, "%s: group_size %d", what, G);
  if (G > kGenericTile) return fail(FO_ERR_UNSUPPORTED, "%s: group_size %d > %d", what, G, kGenericTile);
  const unsigned long long tile = (unsigned long long)(kGenericTile / G) * G;
  const unsigned long long blocks = (n + tile - 1) / tile;
  if (blocks > 0x7FFFFFFFull) return fail(FO_ERR_TOO_LARGE, "%s: %llu elements exceed one launch", what, (unsigned long long)n);
  quantize_kernel<VARIANCE><<<(unsigned int)blocks, kCodecThreads, 0, (cudaStream_t)stream>>>(x, values, (__half*)scales, n, G, floor_mode);
  return check_launch(what);
}

template <bool VARIANCE>
static int dequantize_entry(const void* values, const void* scales, float* out, uint64_t n, int32_t G, void* stream,
                            const char* what) {
  if (n == 0) return FO_OK;
  if (values == nullptr || scales == nullptr || out == nullptr) return fail(FO_ERR_INVALID_ARG, "%s: null pointer", what);
  if (G < 1) return fail(FO_ERR_INVALID_ARG, "%s: group_size %d", what, G);
  dequantize_kernel<VARIANCE><<<stride_grid(n), kCodecThreads, 0, (cudaStream_t)stream>>>(values, (const __half*)scales, out, n, G);
  return check_launch(what);
}

}  // namespace fo

using namespace fo;

extern "C" int fo_quantize_momentum(const float* x, int8_t* values, void* scales, uint64_t n, int32_t G, int32_t floor_mode,
                                    void* stream) {
  return quantize_entry<false>(x, values, scales, n, G, floor_mode, stream, "fo_quantize_momentum");
}
extern "C" int fo_quantize_variance(const float* x, uint8_t* values, void* scales, uint64_t n, int32_t G, int32_t floor_mode,
                                    void* stream) {
  return quantize_entry<true>(x, values, scales, n, G, floor_mode, stream, "fo_quantize_variance");
}
extern "C" int fo_dequantize_momentum(const int8_t* values, const void* scales, float* out, uint64_t n, int32_t G, void* stream) {
  return dequantize_entry<false>(values, scales, out, n, G, stream, "fo_dequantize_momentum");
}
extern "C" int fo_dequantize_variance(const uint8_t* values, const void* scales, float* out, uint64_t n, int32_t G, void* stream) {
  return dequantize_entry<true>(values, scales, out, n, G, stream, "fo_dequantize_variance");
}

#define FO_LP_COMBOS(X) X(FO_BF16, 0) X(FO_BF16, 8) X(FO_BF16, 16) X(FO_F16, 0) X(FO_F16, 8) X(FO_F16, 16)

extern "C" int fo_split(const float* theta, void* lp, void* ecc, int32_t pdt, int32_t ecc_bits, uint64_t n, void* stream) {
  if (n == 0) return FO_OK;
  if (theta == nullptr || lp == nullptr || (ecc_bits != 0 && ecc == nullptr)) return fail(FO_ERR_INVALID_ARG, "fo_split: null pointer");
#define X(P, E)                                                                                                         \
  if (pdt == P && ecc_bits == E) {                                                                                      \
    split_kernel<P, E><<<stride_grid(n), kCodecThreads, 0, (cudaStream_t)stream>>>(theta, (unsigned short*)lp, ecc, n);       \
    return check_launch("fo_split");                                                                                    \
  }
  FO_LP_COMBOS(X)
#undef X
  return fail(FO_ERR_INVALID_ARG, "fo_split: param_dtype %d with ecc_bits %d", pdt, ecc_bits);
}

extern "C" int fo_reconstruct(const void* lp, const void* ecc, float* theta, int32_t pdt, int32_t ecc_bits, uint64_t n,
                              void* stream) {
  if (n == 0) return FO_OK;
  if (theta == nullptr || lp == nullptr || (ecc_bits != 0 && ecc == nullptr)) return fail(FO_ERR_INVALID_ARG, "fo_reconstruct: null pointer");
#define X(P, E)                                                                                                         \
  if (pdt == P && ecc_bits == E) {                                                                                      \
    reconstruct_kernel<P, E><<<stride_grid(n), kCodecThreads, 0, (cudaStream_t)stream>>>((const unsigned short*)lp, ecc, theta, n); \
    return check_launch("fo_reconstruct");                                                                              \
  }
  FO_LP_COMBOS(X)
#undef X
  return fail(FO_ERR_INVALID_ARG, "fo_reconstruct: param_dtype %d with ecc_bits %d", pdt, ecc_bits);
}
