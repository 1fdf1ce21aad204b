// Sum of squares of a gradient pytree (the global norm of optax.clip_by_global_norm, which the
// reference's GPT-2 recipe chains in front of the optimizer, examples/train_gpt2_pretrain.py:56-70).
// A pure read sweep: 128-bit loads, squares exact in fp32, eight-element runs summed in fp32 and
// added to a per-thread double; block and grid reductions in double in a fixed order.
#include "fo_step.cuh"

namespace fo {
int fail(int code, const char* fmt, ...);

constexpr int kNormMaxArrays = 160;   // per launch (kernel-parameter table)
constexpr int kNormBlocksPerSm = 8;
constexpr int kNormMaxBlocks = 2048;  // doubles in the workspace

struct NormParams {
  const void* data[kNormMaxArrays];
  unsigned long long n[kNormMaxArrays];
  uint32_t first_chunk[kNormMaxArrays + 1];
  uint8_t aligned[kNormMaxArrays];
  int32_t n_arrays;
  int32_t dtype;
};

FO_DEVI float sq_run(const uint4& w0, const uint4& w1, int dt) {
  float2 v[4];
  grad_pairs(w0, w1, dt, v);
  float s = 0.0f;
#pragma unroll
  for (int k = 0; k < 4; ++k) s = __fmaf_rn(v[k].y, v[k].y, __fmaf_rn(v[k].x, v[k].x, s));
  return s;
}

// one chunk of this kernel: kNormPieces pieces of kPiece elements per thread, kChunk apart, so that
// every thread has that many independent 128-bit loads in flight
constexpr int kNormPieces = 4;
constexpr unsigned long long kNormChunk = (unsigned long long)kChunk * kNormPieces;

__global__ void __launch_bounds__(kThreads) sq_norm_partial(const __grid_constant__ NormParams p, double* partials) {
  __shared__ double warp_sums[kThreads / 32];
  double acc = 0.0;
  const uint32_t total = p.first_chunk[p.n_arrays];
  int a = 0;
  for (uint32_t c = blockIdx.x; c < total; c += gridDim.x) {
    while (c >= p.first_chunk[a + 1]) ++a;
    const unsigned long long base = (unsigned long long)(c - p.first_chunk[a]) * kNormChunk + (unsigned long long)threadIdx.x * kPiece;
    const unsigned long long n = p.n[a];
    if (p.aligned[a] && base + (kNormPieces - 1) * (unsigned long long)kChunk + kPiece <= n) {
      uint4 w0[kNormPieces], w1[kNormPieces];
#pragma unroll
      for (int k = 0; k < kNormPieces; ++k) {
        const unsigned long long i0 = base + (unsigned long long)k * kChunk;
        w1[k] = make_uint4(0u, 0u, 0u, 0u);
        if (p.dtype == FO_F32) {
          w0[k] = __ldcs((const uint4*)((const float*)p.data[a] + i0));
          w1[k] = __ldcs((const uint4*)((const float*)p.data[a] + i0) + 1);
        } else {
          w0[k] = __ldcs((const uint4*)((const unsigned short*)p.data[a] + i0));
        }
      }
#pragma unroll
      for (int k = 0; k < kNormPieces; ++k) acc += (double)sq_run(w0[k], w1[k], p.dtype);
    } else {
      for (int k = 0; k < kNormPieces; ++k) {
        const unsigned long long i0 = base + (unsigned long long)k * kChunk;
        float s = 0.0f;
        for (int j = 0; j < kPiece && i0 + j < n; ++j) {
          const float g = load_grad(p.data[a], p.dtype, i0 + j);
          s = __fmaf_rn(g, g, s);
        }
        acc += (double)s;
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) s += warp_sums[w];
    partials[blockIdx.x] = s;
  }
}

// reduce-scatter by peer loads, the mean written out, its squares summed (see fo_mean_sq_norm)
struct MeanParams {
  const void* grad;
  void* mean_out;
  unsigned long long n;
  long long gdelta[kMaxPeers];
  int32_t n_peers;
  int32_t dtype;
};

__global__ void __launch_bounds__(kThreads) mean_sq_norm_partial(const __grid_constant__ MeanParams p, double* partials) {
  __shared__ double warp_sums[kThreads / 32];
  double acc = 0.0;
  const float ranks = (float)(p.n_peers + 1);
  const unsigned long long pieces = p.n / kPiece;
  for (unsigned long long q = (unsigned long long)blockIdx.x * kThreads + threadIdx.x; q < pieces; q += (unsigned long long)gridDim.x * kThreads) {
    const unsigned long long i0 = q * kPiece;
    const size_t off = (size_t)i0 * (p.dtype == FO_F32 ? 4u : 2u);
    uint4 w0, w1 = make_uint4(0u, 0u, 0u, 0u);
    w0 = __ldcs((const uint4*)((const char*)p.grad + off));
    if (p.dtype == FO_F32) w1 = __ldcs((const uint4*)((const char*)p.grad + off) + 1);
    float2 g[4];
    grad_pairs(w0, w1, p.dtype, g);
    for (int r = 0; r < p.n_peers; ++r) {
      const char* src = (const char*)p.grad + p.gdelta[r] + off;
      uint4 v0 = __ldcs((const uint4*)src), v1 = make_uint4(0u, 0u, 0u, 0u);
      if (p.dtype == FO_F32) v1 = __ldcs((const uint4*)src + 1);
      float2 pg[4];
      grad_pairs(v0, v1, p.dtype, pg);
#pragma unroll
      for (int k = 0; k < 4; ++k) { g[k].x = fadd(g[k].x, pg[k].x); g[k].y = fadd(g[k].y, pg[k].y); }
    }
    float s = 0.0f;
    uint32_t packed[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float a = fdiv(g[k].x, ranks), b = fdiv(g[k].y, ranks);
      if (p.dtype == FO_BF16) { packed[k] = pack2<FO_BF16>(a, b); unpack2<FO_BF16>(packed[k], a, b); }
      if (p.dtype == FO_F16) { packed[k] = pack2<FO_F16>(a, b); unpack2<FO_F16>(packed[k], a, b); }
      g[k].x = a; g[k].y = b;
      s = __fmaf_rn(b, b, __fmaf_rn(a, a, s));
    }
    if (p.dtype == FO_F32) {
      __stcs((float4*)((char*)p.mean_out + off), make_float4(g[0].x, g[0].y, g[1].x, g[1].y));
      __stcs((float4*)((char*)p.mean_out + off) + 1, make_float4(g[2].x, g[2].y, g[3].x, g[3].y));
    } else {
      __stcs((uint4*)((char*)p.mean_out + off), make_uint4(packed[0], packed[1], packed[2], packed[3]));
    }
    acc += (double)s;
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) t += warp_sums[w];
    partials[blockIdx.x] = t;
  }
}

__global__ void sq_norm_final(const double* partials, int n, double* out, int accumulate) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  double s = accumulate ? *out : 0.0;
  for (int i = 0; i < n; ++i) s += partials[i];
  *out = s;
}

__global__ void step_scalars_kernel(const int32_t* count, const float* lr_dev, float lr_const, float b1, float b2, float* out3,
                                    int32_t* count_out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int32_t c = *count + 1;
  out3[0] = lr_dev != nullptr ? *lr_dev : lr_const;
  out3[1] = fsub(1.0f, (float)pow((double)b1, (double)c));
  out3[2] = fsub(1.0f, (float)pow((double)b2, (double)c));
  if (count_out != nullptr) *count_out = c;
}

// examples/example_utils.py:94-103, one fp32 rounding per written operation
FO_DEVI float warmup_cosine(float step, float total, float warmup, float peak) {
  if (warmup > 0.0f && step < warmup) return fdiv(fmul(peak, fadd(step, 1.0f)), warmup);
  const float span = fmaxf(1.0f, fsub(total, warmup));
  const float progress = fminf(fmaxf(fdiv(fsub(step, warmup), span), 0.0f), 1.0f);
  const float c = (float)cos((double)fmul(3.14159274101257324f, progress));  // f32(pi) * progress, as jnp.pi * progress
  return fmul((float)((double)peak * 0.5), fadd(1.0f, c));
}

__global__ void step_scalars_schedule_kernel(const int32_t* count, int32_t schedule, float p0, float p1, float p2, float b1, float b2,
                                             float* out3, int32_t* count_out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int32_t before = *count, c = before + 1;
  float lr = 0.0f;
  if (schedule == FO_SCHEDULE_WARMUP_COSINE) lr = warmup_cosine((float)before, p0, p1, p2);
  out3[0] = lr;
  out3[1] = fsub(1.0f, (float)pow((double)b1, (double)c));
  out3[2] = fsub(1.0f, (float)pow((double)b2, (double)c));
  if (count_out != nullptr) *count_out = c;
}

}  // namespace fo

using namespace fo;

extern "C" int fo_sq_norm(const FoArray* arrays, uint32_t n_arrays, int32_t dtype, int32_t accumulate, double* out,
                          void* workspace, void* cuda_stream) {
  static_assert(kNormMaxBlocks * sizeof(double) <= FO_SQ_NORM_WORKSPACE_BYTES, "workspace too small");
  if (out == nullptr || workspace == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_sq_norm: null out / workspace");
  if (dtype < FO_F32 || dtype > FO_F16) return fail(FO_ERR_INVALID_ARG, "fo_sq_norm: bad dtype %d", dtype);
  if (n_arrays > 0 && arrays == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_sq_norm: null table");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return fail(FO_ERR_CUDA, "fo_sq_norm: cannot query the current device");
  double* partials = static_cast<double*>(workspace);
  NormParams p;
  memset(&p, 0, sizeof(p));
  p.dtype = dtype;
  int count = 0;
  unsigned long long chunks = 0;
  bool launched = false;
  auto flush = [&]() -> int {
    // an empty list still has to define *out
    if (count == 0 && launched) return FO_OK;
    p.n_arrays = count;
    p.first_chunk[count] = (uint32_t)chunks;
    unsigned int grid = (unsigned int)(sms * kNormBlocksPerSm);
    if (grid > kNormMaxBlocks) grid = kNormMaxBlocks;
    if (grid > chunks) grid = (unsigned int)chunks;
    if (grid > 0) sq_norm_partial<<<grid, kThreads, 0, stream>>>(p, partials);
    sq_norm_final<<<1, 32, 0, stream>>>(partials, (int)grid, out, launched ? 1 : accumulate);
    launched = true;
    count = 0;
    chunks = 0;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_sq_norm: launch failed: %s", cudaGetErrorString(e));
    return FO_OK;
  };
  for (uint32_t i = 0; i < n_arrays; ++i) {
    if (arrays[i].n == 0) continue;
    if (arrays[i].data == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_sq_norm: array %u: null data", i);
    const unsigned long long nc = (arrays[i].n + kNormChunk - 1) / kNormChunk;
    if (nc > 0x7FFFFFFFull) return fail(FO_ERR_TOO_LARGE, "fo_sq_norm: array %u with %llu elements exceeds one launch", i, (unsigned long long)arrays[i].n);
    if (count == kNormMaxArrays || chunks + nc > 0x7FFFFFFFull) {
      int rc = flush();
      if (rc != FO_OK) return rc;
    }
    p.data[count] = arrays[i].data;
    p.n[count] = arrays[i].n;
    p.first_chunk[count] = (uint32_t)chunks;
    p.aligned[count] = ((uintptr_t)arrays[i].data & 15u) == 0;
    chunks += nc;
    ++count;
  }
  return flush();
}

extern "C" int fo_mean_sq_norm(const void* grad, void* mean_out, uint64_t n, int32_t dtype, const int64_t* peer_grad_offsets,
                               uint32_t n_peers, int32_t accumulate, double* out, void* workspace, void* cuda_stream) {
  if (out == nullptr || workspace == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_mean_sq_norm: null out / workspace");
  if (dtype < FO_F32 || dtype > FO_F16) return fail(FO_ERR_INVALID_ARG, "fo_mean_sq_norm: bad dtype %d", dtype);
  if (n_peers > (uint32_t)kMaxPeers) return fail(FO_ERR_TOO_LARGE, "fo_mean_sq_norm: %u peers, at most %d", n_peers, kMaxPeers);
  if (n_peers > 0 && peer_grad_offsets == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_mean_sq_norm: n_peers without peer_grad_offsets");
  if (n > 0 && (grad == nullptr || mean_out == nullptr)) return fail(FO_ERR_INVALID_ARG, "fo_mean_sq_norm: null grad / mean_out");
  if (n % kPiece != 0 || ((uintptr_t)grad & 15u) != 0 || ((uintptr_t)mean_out & 15u) != 0)
    return fail(FO_ERR_INVALID_ARG, "fo_mean_sq_norm: n must be a multiple of %d and the pointers 16-byte aligned", kPiece);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return fail(FO_ERR_CUDA, "fo_mean_sq_norm: cannot query the current device");
  MeanParams p;
  memset(&p, 0, sizeof(p));
  p.grad = grad; p.mean_out = mean_out; p.n = n; p.n_peers = (int32_t)n_peers; p.dtype = dtype;
  for (uint32_t r = 0; r < n_peers; ++r) p.gdelta[r] = (long long)peer_grad_offsets[r];
  double* partials = static_cast<double*>(workspace);
  unsigned long long want = (n / kPiece + kThreads - 1) / kThreads;
  unsigned int grid = (unsigned int)(sms * kNormBlocksPerSm);
  if (grid > kNormMaxBlocks) grid = kNormMaxBlocks;
  if ((unsigned long long)grid > want) grid = (unsigned int)want;
  if (grid > 0) mean_sq_norm_partial<<<grid, kThreads, 0, stream>>>(p, partials);
  sq_norm_final<<<1, 32, 0, stream>>>(partials, (int)grid, out, accumulate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_mean_sq_norm: launch failed: %s", cudaGetErrorString(e));
  return FO_OK;
}

extern "C" int fo_step_scalars(const int32_t* count, const float* lr_dev, float lr_const, float b1, float b2, float* out3,
                               int32_t* count_out, void* cuda_stream) {
  if (count == nullptr || out3 == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step_scalars: null count / out3");
  step_scalars_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(count, lr_dev, lr_const, b1, b2, out3, count_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_step_scalars: launch failed: %s", cudaGetErrorString(e));
  return FO_OK;
}

extern "C" int fo_step_scalars_schedule(const int32_t* count, int32_t schedule, const float* p, float b1, float b2, float* out3,
                                        int32_t* count_out, void* cuda_stream) {
  if (count == nullptr || out3 == nullptr || p == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step_scalars_schedule: null argument");
  if (schedule != FO_SCHEDULE_WARMUP_COSINE) return fail(FO_ERR_INVALID_ARG, "fo_step_scalars_schedule: unknown schedule %d", schedule);
  step_scalars_schedule_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(count, schedule, p[0], p[1], p[2], b1, b2, out3, count_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_step_scalars_schedule: launch failed: %s", cudaGetErrorString(e));
  return FO_OK;
}
