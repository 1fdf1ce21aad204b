// extern "C" surface of libflashoptim_b200.so: argument checking, building the kernel
// parameter tables, launching.  No allocation, no synchronisation, caller's stream only.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "fo_step.cuh"

namespace fo {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static Launcher find_launcher(int opt, int pdt, int ecc_bits, int state, bool generic, bool aux) {
#define FO_PICK(stem) return aux ? stem##_aux(pdt, ecc_bits) : stem##_plain(pdt, ecc_bits)
  if (opt == FO_OPT_ADAM) {
    if (generic) return lookup_adam_generic(pdt, ecc_bits);
    if (state == FO_STATE_QUANT) FO_PICK(lookup_adam_quant);
    if (state == FO_STATE_FULL) FO_PICK(lookup_adam_full);
  } else if (opt == FO_OPT_LION) {
    if (generic) return lookup_lion_generic(pdt, ecc_bits);
    if (state == FO_STATE_QUANT) FO_PICK(lookup_lion_quant);
    if (state == FO_STATE_FULL) FO_PICK(lookup_lion_full);
  } else if (opt == FO_OPT_SGD) {
    if (generic) return lookup_sgd_generic(pdt, ecc_bits);
    if (state == FO_STATE_QUANT) FO_PICK(lookup_sgd_quant);
    if (state == FO_STATE_FULL) FO_PICK(lookup_sgd_full);
    if (state == FO_STATE_NONE) FO_PICK(lookup_sgd_none);
  }
#undef FO_PICK
  return Launcher{nullptr, 0u};
}

static DevHyper make_dev_hyper(const FoHyper& h, int opt) {
  DevHyper d;
  memset(&d, 0, sizeof(d));
  d.lr = h.lr; d.wd = h.wd; d.b1 = h.b1; d.b2 = h.b2;
  d.omb1 = h.one_minus_b1; d.omb2 = h.one_minus_b2;
  d.eps = h.eps; d.bc1 = h.bc1; d.bc2 = h.bc2;
  // single IEEE fp32 operations, as the reference forms them (adamw.py:103-105)
  volatile float prod = h.lr * h.wd;
  d.decay = 1.0f - prod;
  d.flags = h.flags & (FO_FLAG_DECOUPLED_WD | FO_FLAG_NESTEROV | FO_FLAG_LION_LERP | FO_FLAG_LP_DELTA | FO_FLAG_SCALE_FLOOR);
  if (opt == FO_OPT_ADAM) {
    d.lr_bc1 = h.lr / h.bc1;
    d.sqrt_bc2 = sqrtf(h.bc2);
    d.rcp_sqrt_bc2 = 1.0f / d.sqrt_bc2;
    if (adam_is_tame(h.eps, d.sqrt_bc2)) d.flags |= kFlagTameAdam;
  }
  d.dyn = h.dev_scalars;
  return d;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// SM count of the device that is current on the calling thread (cached per device ordinal; atomics,
// so that concurrent first calls from several threads are well defined: they store the same number)
static int sm_count_of_current_device() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (dev >= 0 && dev < 64) {
    const int known = cache[dev].load(std::memory_order_acquire);
    if (known > 0) return known;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (dev >= 0 && dev < 64) cache[dev].store(sms, std::memory_order_release);
  return sms;
}

}  // namespace fo

using namespace fo;

extern "C" int fo_step(const FoStepDesc* d, void* cuda_stream) {
  if (d == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: null descriptor");
  if (d->struct_size != sizeof(FoStepDesc))
    return fail(FO_ERR_INVALID_ARG, "fo_step: struct_size %u != %zu (ABI mismatch)", d->struct_size, sizeof(FoStepDesc));
  if (d->opt < FO_OPT_ADAM || d->opt > FO_OPT_SGD) return fail(FO_ERR_INVALID_ARG, "fo_step: bad opt %d", d->opt);
  if (d->param_dtype < FO_F32 || d->param_dtype > FO_F16) return fail(FO_ERR_INVALID_ARG, "fo_step: bad param_dtype %d", d->param_dtype);
  if (d->grad_dtype < FO_F32 || d->grad_dtype > FO_F16) return fail(FO_ERR_INVALID_ARG, "fo_step: bad grad_dtype %d", d->grad_dtype);
  if (d->ecc_bits != 0 && d->ecc_bits != 8 && d->ecc_bits != 16) return fail(FO_ERR_INVALID_ARG, "fo_step: ecc_bits must be 0, 8 or 16, got %d", d->ecc_bits);
  if (d->param_dtype == FO_F32 && d->ecc_bits != 0) return fail(FO_ERR_INVALID_ARG, "fo_step: fp32 params carry no ECC");
  if (d->state < FO_STATE_QUANT || d->state > FO_STATE_NONE) return fail(FO_ERR_INVALID_ARG, "fo_step: bad state %d", d->state);
  if (d->state == FO_STATE_NONE && d->opt != FO_OPT_SGD) return fail(FO_ERR_INVALID_ARG, "fo_step: only SGD can run without a momentum buffer");
  if (d->n_leaves == 0) return FO_OK;
  if (d->leaves == nullptr || d->hypers == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: null table");
  if (d->n_hypers == 0) return fail(FO_ERR_INVALID_ARG, "fo_step: no hyper-parameter set");
  if (d->n_hypers > FO_MAX_HYPERS) return fail(FO_ERR_TOO_LARGE, "fo_step: %u hyper sets, at most %d per call", d->n_hypers, FO_MAX_HYPERS);
  bool generic = false;
  if (d->state == FO_STATE_QUANT) {
    if (d->group_size < 1) return fail(FO_ERR_INVALID_ARG, "fo_step: group_size %d", d->group_size);
    if (d->group_size > kGenericTile) return fail(FO_ERR_UNSUPPORTED, "fo_step: group_size %d > %d", d->group_size, kGenericTile);
    generic = d->group_size != 32;
  }
  if (d->n_peers > (uint32_t)kMaxPeers) return fail(FO_ERR_TOO_LARGE, "fo_step: %u peers, at most %d", d->n_peers, kMaxPeers);
  if (d->n_peers > 0 && d->peer_param_offsets == nullptr && d->peer_grad_offsets == nullptr)
    return fail(FO_ERR_INVALID_ARG, "fo_step: n_peers without peer_param_offsets or peer_grad_offsets");
  if (d->n_peers > 0 && generic) return fail(FO_ERR_UNSUPPORTED, "fo_step: peer replicas need group_size 32");
  if (find_launcher(d->opt, d->param_dtype, d->ecc_bits, d->state, generic, false).launch == nullptr)
    return fail(FO_ERR_UNSUPPORTED, "fo_step: no kernel for this combination");

  const bool need_mu = d->state != FO_STATE_NONE;
  const bool need_nu = need_mu && d->opt == FO_OPT_ADAM;
  const bool need_scales = d->state == FO_STATE_QUANT;
  for (uint32_t i = 0; i < d->n_leaves; ++i) {
    const FoLeaf& L = d->leaves[i];
    if (L.n == 0) continue;
    if (L.grad == nullptr || L.param == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: null grad/param", i);
    if (d->ecc_bits != 0 && L.ecc == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: null ecc", i);
    if (need_mu && L.mu == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: null mu", i);
    if (need_nu && L.nu == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: null nu", i);
    if (need_scales && L.mu_scales == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: null mu_scales", i);
    if (need_scales && need_nu && L.nu_scales == nullptr) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: null nu_scales", i);
    if (L.hyper >= d->n_hypers) return fail(FO_ERR_INVALID_ARG, "fo_step: leaf %u: hyper index %u out of range", i, L.hyper);
  }

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  LaunchInfo info;
  info.sm_count = sm_count_of_current_device();
  if (info.sm_count <= 0) return fail(FO_ERR_CUDA, "fo_step: cannot query the current device");
  const unsigned long long kMaxBlocks = 0x7FFFFFFFull;

  StepParams p;
  memset(&p, 0, sizeof(p));
  for (uint32_t h = 0; h < d->n_hypers; ++h) p.hyper[h] = make_dev_hyper(d->hypers[h], d->opt);
  p.grad_dtype = d->grad_dtype;
  p.group_size = d->state == FO_STATE_QUANT ? d->group_size : 32;
  p.one = 1.0f;
  if (d->peer_param_offsets != nullptr) {
    p.peers.n = (int)d->n_peers;
    for (uint32_t r = 0; r < d->n_peers; ++r) p.peers.delta[r] = (long long)d->peer_param_offsets[r];
  }
  if (d->peer_grad_offsets != nullptr && d->n_peers > 0) {
    const uint32_t ranks = d->n_peers + 1;
    p.peers.ng = (int)d->n_peers;
    for (uint32_t r = 0; r < d->n_peers; ++r) p.peers.gdelta[r] = (long long)d->peer_grad_offsets[r];
    p.peers.neg_ranks = -(float)ranks;
    p.peers.rcp_ranks = 1.0f / (float)ranks;  // correctly rounded (IEEE division on the host)
    p.peers.ranks_pow2 = (ranks & (ranks - 1)) == 0;
  }

  if (d->mc_param_offset != 0) {
    if (d->peer_param_offsets == nullptr || d->n_peers == 0) return fail(FO_ERR_INVALID_ARG, "fo_step: mc_param_offset without peer_param_offsets");
    p.peers.mc_pdelta = (long long)d->mc_param_offset;
  }
  if (d->mc_grad_offset != 0) {
    if (d->peer_grad_offsets == nullptr || d->n_peers == 0) return fail(FO_ERR_INVALID_ARG, "fo_step: mc_grad_offset without peer_grad_offsets");
    p.peers.mc_gdelta = (long long)d->mc_grad_offset;
  }
  p.sq_norm = d->grad_sq_norm;
  p.max_norm = d->max_grad_norm;
  // the slice that runs this step, and the elements one of its chunks covers
  const Launcher launcher = find_launcher(d->opt, d->param_dtype, d->ecc_bits, d->state, generic, step_needs_aux(p));
  if (launcher.launch == nullptr) return fail(FO_ERR_UNSUPPORTED, "fo_step: no kernel for this combination");
  const LaunchFn launch = launcher.launch;
  const unsigned long long chunk = generic ? generic_tile_elems(d->group_size) : launcher.chunk;

  int count = 0;
  unsigned long long blocks = 0;
  auto flush = [&]() -> int {
    if (count == 0) return FO_OK;
    p.n_leaves = count;
    p.first_block[count] = (uint32_t)blocks;
    info.total_chunks = (unsigned int)blocks;
    cudaError_t e = launch(p, info, stream);
    count = 0;
    blocks = 0;
    if (e != cudaSuccess) return fail(FO_ERR_CUDA, "fo_step: launch failed: %s", cudaGetErrorString(e));
    return FO_OK;
  };
  // The 32-group kernels address elements with 32-bit offsets: a longer leaf goes in as several
  // leaves of 2^31 elements (a multiple of the chunk and of the group, so every piece keeps
  // its alignment and its own whole groups).
  const unsigned long long kMaxLeafElems = generic ? ~0ull : (1ull << 31);
  const size_t grad_size = d->grad_dtype == FO_F32 ? 4 : 2, param_size = d->param_dtype == FO_F32 ? 4 : 2;
  const size_t ecc_size = (size_t)d->ecc_bits / 8, moment_size = d->state == FO_STATE_FULL ? 4 : 1;
  auto advance = [](const void* base, unsigned long long elems, size_t size) -> void* {
    return base == nullptr ? nullptr : (void*)((const char*)base + elems * size);
  };
  for (uint32_t i = 0; i < d->n_leaves; ++i) {
    const FoLeaf& L = d->leaves[i];
    for (unsigned long long done = 0; done < L.n; done += kMaxLeafElems) {
      const unsigned long long n = L.n - done < kMaxLeafElems ? L.n - done : kMaxLeafElems;
      const unsigned long long nb = (n + chunk - 1) / chunk;
      if (nb > kMaxBlocks) return fail(FO_ERR_TOO_LARGE, "fo_step: leaf %u with %llu elements exceeds one launch", i, (unsigned long long)L.n);
      if (count == kMaxLeaves || blocks + nb > kMaxBlocks) {
        int rc = flush();
        if (rc != FO_OK) return rc;
      }
      DevLeaf& D = p.leaf[count];
      D.grad = advance(L.grad, done, grad_size);
      D.param = advance(L.param, done, param_size);
      D.ecc = advance(L.ecc, done, ecc_size);
      D.mu = advance(L.mu, done, moment_size);
      D.nu = advance(L.nu, done, moment_size);
      D.mu_scales = advance(L.mu_scales, done / 32, 2);
      D.nu_scales = advance(L.nu_scales, done / 32, 2);
      D.n = n;
      p.first_block[count] = (uint32_t)blocks;
      p.hyper_of[count] = (uint8_t)L.hyper;
      p.aligned[count] = aligned16(D.grad) && aligned16(D.param) && aligned16(D.ecc) && aligned16(D.mu) && aligned16(D.nu);
      blocks += nb;
      ++count;
    }
  }
  return flush();
}

extern "C" int fo_version(void) { return FO_ABI_VERSION; }

extern "C" const char* fo_status_string(int status) {
  switch (status) {
    case FO_OK: return "ok";
    case FO_ERR_INVALID_ARG: return "invalid argument";
    case FO_ERR_UNSUPPORTED: return "unsupported configuration";
    case FO_ERR_CUDA: return "CUDA error";
    case FO_ERR_TOO_LARGE: return "size beyond a stated maximum";
    default: return "unknown status";
  }
}

extern "C" const char* fo_last_error(void) { return fo::g_err; }
