/*
 * flashoptim_b200 — C ABI of the B200-native optimizer-step library.
 *
 * One shared object (libflashoptim_b200.so), plain C types only.  Every array argument
 * is a DEVICE pointer unless it is called a table; tables (leaf / hyper-parameter
 * descriptors) are HOST memory and are copied into kernel parameters at launch.  The
 * library never allocates, frees or keeps caller memory, never synchronises the device
 * and launches only on the stream it is given, so a call can sit inside any framework's
 * stream order (XLA custom call, PyTorch, CUDA graph).  All updates are in place: the
 * reference's fused kernels alias every output onto its input
 * (flashoptim_jax/adamw.py:268,293; flashoptim_jax/momentum_kernel.py:222,246).
 *
 * All functions return FO_OK or an FO_ERR_* code; fo_status_string() names a code and
 * fo_last_error() returns a thread-local detail message.
 *
 * Citations "file:line" refer to the reference project (samacqua/flashoptim-jax).
 */
#ifndef FLASHOPTIM_B200_H_
#define FLASHOPTIM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FO_ABI_VERSION 3

/* status codes */
#define FO_OK 0
#define FO_ERR_INVALID_ARG 1  /* null pointer, bad enum, inconsistent descriptor */
#define FO_ERR_UNSUPPORTED 2  /* legal in the reference but not built here (e.g. group_size > 1024) */
#define FO_ERR_CUDA 3         /* a CUDA runtime call failed; see fo_last_error() */
#define FO_ERR_TOO_LARGE 4    /* more hyper-parameter sets than one call can carry, or a size beyond a stated maximum */

/* element types of params / grads (the dtypes the fused path accepts, flashoptim_jax/utils.py:26-31) */
#define FO_F32 0
#define FO_BF16 1
#define FO_F16 2

/* optimizer family: Adam/AdamW share a kernel (flashoptim_jax/adamw.py:28-222), Lion and
 * SGD/SGDW share the other (flashoptim_jax/momentum_kernel.py:21-180, switch do_lion) */
#define FO_OPT_ADAM 0
#define FO_OPT_LION 1
#define FO_OPT_SGD 2

/* how the moments are stored */
#define FO_STATE_QUANT 0 /* int8 mu / uint8 nu codes + fp16 group scales (quantize=True) */
#define FO_STATE_FULL 1  /* fp32 mu / nu (quantize=False; adamw.py:148-222, momentum_kernel.py:115-180) */
#define FO_STATE_NONE 2  /* SGD with momentum == 0: no buffer (flashoptim_jax/sgd.py:50-57, utils.py:351-352) */

/* FoHyper.flags */
#define FO_FLAG_DECOUPLED_WD 1u /* AdamW / SGDW: theta *= 1 - lr*wd (adamw.py:102-103); clear = wd added to the grad (adamw.py:95-96) */
#define FO_FLAG_NESTEROV 2u     /* SGD: step = grad + momentum*mu (momentum_kernel.py:82) */
#define FO_FLAG_LION_LERP 4u    /* Lion written as mu + (1-b)(g-mu) (lion.py:50-52) instead of b*mu + (1-b)*g (momentum_kernel.py:78-79) */
#define FO_FLAG_LP_DELTA 8u     /* Adam hands back param + lp(new - param) like the CPU path (adamw.py:411,415,463) instead of new (adamw.py:134) */
#define FO_FLAG_SCALE_FLOOR 16u /* group scale guard max(absmax,1e-12) (adamw.py:121,128) instead of where(absmax>0,absmax,1) (quantization.py:41,64) */

/*
 * One set of hyper-parameters (one param group, flashoptim_jax/utils.py:138-154).
 * These are the 0-d fp32 operands of the reference kernels (adamw.py:272-278,
 * momentum_kernel.py:230-233) plus the two derived constants the two reference texts form
 * differently (see FO_FLAG_*).  Field use by family:
 *   ADAM: lr wd b1 b2 one_minus_b1 one_minus_b2 eps bc1 bc2
 *   LION: lr wd b1 b2 one_minus_b1 one_minus_b2          (b1 = update coef, b2 = momentum coef)
 *   SGD : lr wd b1(=momentum) one_minus_b1(= 1 - dampening)
 * dev_scalars, when not NULL, is a device float[3] = {lr, bc1, bc2} read by the kernel in
 * place of the host values, so a traced schedule / step count needs no host round trip.
 */
typedef struct FoHyper {
  float lr, wd;
  float b1, b2;
  float one_minus_b1, one_minus_b2;
  float eps;
  float bc1, bc2; /* 1 - b^count, count = step number after increment (adamw.py:510,527-528) */
  uint32_t flags;
  const float* dev_scalars;
} FoHyper;

/*
 * One pytree leaf, flattened row-major (flashoptim_jax/utils.py:450-496).
 *   grad       n elements of grad dtype
 *   param      n elements of param dtype, updated in place
 *   ecc        n int8 (ecc_bits 8) / int16 (ecc_bits 16), or NULL when ecc_bits == 0
 *   mu         n int8 codes (QUANT) or n fp32 (FULL), NULL for NONE
 *   mu_scales  ceil(n / group_size) fp16 (QUANT), else NULL
 *   nu, nu_scales  same for the second moment (uint8 codes), ADAM only, else NULL
 *   hyper      index into the hyper table
 */
typedef struct FoLeaf {
  const void* grad;
  void* param;
  void* ecc;
  void* mu;
  void* mu_scales;
  void* nu;
  void* nu_scales;
  uint64_t n;
  uint32_t hyper;
  uint32_t reserved;
} FoLeaf;

/*
 * One multi-tensor step: every leaf of the table shares the compile-time switches of the
 * reference's pallas_call (adamw.py:309-320, momentum_kernel.py:262-275); leaves that
 * differ in them go into separate calls.  Any number of leaves; at most FO_MAX_HYPERS
 * hyper sets.
 */
#define FO_MAX_HYPERS 16
typedef struct FoStepDesc {
  uint32_t struct_size; /* sizeof(FoStepDesc), guards against ABI skew */
  int32_t opt;          /* FO_OPT_* */
  int32_t param_dtype;  /* FO_F32 / FO_BF16 / FO_F16 */
  int32_t grad_dtype;   /* FO_F32 / FO_BF16 / FO_F16 (the reference upcasts grads to fp32 first, adamw.py:531) */
  int32_t ecc_bits;     /* 0, 8 (master_weight_bits 24 on a 16-bit param) or 16 (32) */
  int32_t state;        /* FO_STATE_* */
  int32_t group_size;   /* elements per quantization group, 1..1024 (QUANT only; default 32) */
  uint32_t n_leaves;
  uint32_t n_hypers;
  const FoLeaf* leaves;   /* host table */
  const FoHyper* hypers;  /* host table */
  /* ZeRO-1 all-gather folded into the step (no counterpart in the reference, which replicates
   * state and all-reduces gradients, examples/train_gpt2_pretrain.py:412-441): every updated
   * parameter vector is also stored at (param address + peer_param_offsets[r]) for r < n_peers,
   * i.e. into the same element of peer r's replica of the parameter array.  The offsets are byte
   * distances between peer-mapped allocations (host table, at most FO_MAX_PEERS); plain stores,
   * the kernel never waits on a peer.  The caller orders the launch after the peers' last reads
   * of their replicas and makes the peers wait for this stream before they read again. */
  uint32_t n_peers;
  uint32_t reserved;
  const int64_t* peer_param_offsets; /* NULL: parameters are stored locally only */
  /* ZeRO-1 reduce-scatter folded into the step (same remark): the gradient of element i of a
   * leaf is the mean over the ranks of the values at (grad address + peer_grad_offsets[r]),
   * r < n_peers, and the local one: summed in fp32 in the order local, peer 0, peer 1, ...,
   * divided by (n_peers + 1), rounded once to grad_dtype.  Each leaf's `grad` then points into this
   * rank's copy of the full gradient array.  Plain loads; the caller makes sure every peer has
   * finished writing its gradients before the launch and does not overwrite them before all
   * ranks' kernels have completed.  NULL: the local gradient is used as it is.
   * With n_peers > 0 at least one of the two offset tables must be given; group size 32 only. */
  const int64_t* peer_grad_offsets;
  /* Global-norm gradient clipping folded into the step (optax.clip_by_global_norm chained in front
   * of the optimizer by the reference's GPT-2 recipe, examples/train_gpt2_pretrain.py:56-70):
   * grad_sq_norm points to a device double holding the sum of squares of ALL gradients of the
   * step (fo_sq_norm writes it; with sharded gradients the caller adds the ranks' sums first).
   * With norm = (float)sqrt(*grad_sq_norm): gradients are used as they are if norm < max_grad_norm,
   * else each is replaced by RN_g(RN_g(g / RN_g(norm)) * RN_g(max_grad_norm)), RN_g = rounding to
   * grad_dtype.  Applied after the averaging over peers.  NULL: no clipping.
   * The sum of squares is the caller's: fo_sq_norm forms it exactly (fp32 squares, fp64 sums), where
   * optax sums every leaf in the leaf's own dtype; for 16-bit gradients the two norms, and with them
   * the clip / no-clip decision right at the threshold and the divisor, can differ by places of that
   * dtype.  The element-wise rescaling is optax's bit for bit given the same sum. */
  const double* grad_sq_norm;
  float max_grad_norm;
  uint32_t reserved2;
  /* The same two exchanges through the NVLink switch (0 = off).  Byte distances from a local
   * address to the multicast address that maps the same element on every rank (a multicast
   * object bound to all ranks' buffers, e.g. the multicast pointer of a symmetric allocation).
   * mc_param_offset: whole aligned chunks store their parameters once through the multicast address
   * (the switch replicates them to every rank, this one included) instead of once per peer.
   * mc_grad_offset: for 16-bit gradients, whole aligned chunks read one multicast load-reduce (the
   * switch adds all ranks' values in fp32 and rounds the sum to grad_dtype) instead of one load per
   * peer; the mean is that sum divided by (n_peers + 1), rounded to grad_dtype.  For a power-of-two
   * rank count this equals the single rounding described above whenever the order of the additions
   * does not matter (two ranks; equal gradients); otherwise the switch's order applies.
   * Both need the matching point-to-point table as well, which serves ragged ends and rare values. */
  int64_t mc_param_offset;
  int64_t mc_grad_offset;
} FoStepDesc;
#define FO_MAX_PEERS 7

/* Replaces pl.pallas_call(...) of _fused_flash_adamw_leaf_impl (adamw.py:225-353) and of
 * fused_momentum_leaf_impl (momentum_kernel.py:183-302), for a whole pytree at once. */
int fo_step(const FoStepDesc* desc, void* cuda_stream);

/* Per-step scalars formed on the device, so that a whole step can be captured in a CUDA graph
 * with no host scalar in it (the reference forms them as traced values inside its jitted step:
 * count + 1 at adamw.py:510, learning rate at adamw.py:526, bias corrections at adamw.py:527-528).
 *   c = *count + 1;  out3 = { lr, 1 - b1^c, 1 - b2^c }   (the power in float64, rounded once to fp32)
 * lr = *lr_dev when lr_dev is not NULL, else lr_const.  count_out (may equal count, may be NULL)
 * receives c.  out3 is what FoHyper.dev_scalars points to. */
int fo_step_scalars(const int32_t* count, const float* lr_dev, float lr_const, float b1, float b2, float* out3,
                    int32_t* count_out, void* cuda_stream);

/* The same with the learning rate taken from a schedule evaluated on the device at the zero-based
 * step *count (adamw.py:526 passes the count before its increment to the schedule).
 * FO_SCHEDULE_WARMUP_COSINE restates make_warmup_cosine_schedule of the reference's examples
 * (examples/example_utils.py:94-103) in fp32, p = host array {total_steps, warmup_steps, peak_lr}:
 *   step < warmup:  peak * (step + 1) / warmup
 *   else:           f32(peak * 0.5) * (1 + cos(pi * clip((step - warmup) / max(1, total - warmup), 0, 1)))
 * with the cosine taken in float64 and rounded once (XLA's fp32 cos may differ in the last place). */
#define FO_SCHEDULE_WARMUP_COSINE 1
int fo_step_scalars_schedule(const int32_t* count, int32_t schedule, const float* p, float b1, float b2, float* out3,
                             int32_t* count_out, void* cuda_stream);

/* Sum of squares of a list of device arrays of one dtype (the gradient pytree, or one dtype
 * bucket of it), for global-norm clipping (optax.global_norm as used through
 * examples/train_gpt2_pretrain.py:58): squares exact in fp32, summed in fp32 over short runs and
 * in fp64 beyond, in an order that depends only on the array sizes (same inputs, same bits).
 * *out (device) receives the sum, or has it added when accumulate != 0 (further buckets).
 * workspace: FO_SQ_NORM_WORKSPACE_BYTES bytes of device memory the calls of one stream may share. */
typedef struct FoArray {
  const void* data;
  uint64_t n;
} FoArray;
#define FO_SQ_NORM_WORKSPACE_BYTES 16384
int fo_sq_norm(const FoArray* arrays, uint32_t n_arrays, int32_t dtype, int32_t accumulate, double* out,
               void* workspace, void* cuda_stream);

/* Reduce-scatter and norm in one sweep, for ZeRO-1 steps that clip by the global norm: this rank's
 * slice of the averaged gradient is needed twice (for the norm of the whole averaged gradient, then
 * for the step), but should cross NVLink once.  grad points at the slice inside this rank's copy of
 * the gradient buffer; the same elements of peer r lie peer_grad_offsets[r] bytes away (peer-mapped
 * memory, as for FoStepDesc.peer_grad_offsets).  mean_out[i] = RN_g((g_own[i] + g_peer0[i] + ...) /
 * (n_peers + 1)): fp32 sum in that order, one rounding to the gradient dtype, the value the step
 * kernel's own averaging produces (the reference's pmean, examples/train_gpt2_pretrain.py:429); the sum of
 * mean_out[i]^2 is added to / stored in *out as fo_sq_norm does.  n must be a multiple of 8 and both
 * pointers 16-byte aligned (a ZeRO-1 slice is).  The caller orders the ranks around the call like around a
 * fused reduce-scatter. */
int fo_mean_sq_norm(const void* grad, void* mean_out, uint64_t n, int32_t dtype, const int64_t* peer_grad_offsets,
                    uint32_t n_peers, int32_t accumulate, double* out, void* workspace, void* cuda_stream);

/* Codecs on fp32 arrays; n elements, scales has ceil(n/group_size) fp16 entries.
 * scale_floor selects the guard of FO_FLAG_SCALE_FLOOR.
 *   fo_quantize_momentum   flashoptim_jax/quantization.py:37-46
 *   fo_dequantize_momentum flashoptim_jax/quantization.py:49-56
 *   fo_quantize_variance   flashoptim_jax/quantization.py:59-68
 *   fo_dequantize_variance flashoptim_jax/quantization.py:71-77 */
int fo_quantize_momentum(const float* x, int8_t* values, void* scales_f16, uint64_t n, int32_t group_size,
                         int32_t scale_floor, void* cuda_stream);
int fo_dequantize_momentum(const int8_t* values, const void* scales_f16, float* out, uint64_t n, int32_t group_size,
                           void* cuda_stream);
int fo_quantize_variance(const float* x, uint8_t* values, void* scales_f16, uint64_t n, int32_t group_size,
                         int32_t scale_floor, void* cuda_stream);
int fo_dequantize_variance(const uint8_t* values, const void* scales_f16, float* out, uint64_t n, int32_t group_size,
                           void* cuda_stream);

/* fp32 master weight <-> (16-bit param, ECC).  ecc_bits 0 means a plain cast (ecc unused).
 *   fo_split        flashoptim_jax/compression.py:84-104, utils.py:539-557
 *   fo_reconstruct  flashoptim_jax/compression.py:107-121, utils.py:521-536 */
int fo_split(const float* theta, void* param_lp, void* ecc, int32_t param_dtype, int32_t ecc_bits, uint64_t n,
             void* cuda_stream);
int fo_reconstruct(const void* param_lp, const void* ecc, float* theta, int32_t param_dtype, int32_t ecc_bits,
                   uint64_t n, void* cuda_stream);

/*
 * Device self-checks of the exact-arithmetic shortcuts the kernels use (no counterpart in
 * the reference).  Each runs a sweep on the current device and writes the number of inputs
 * on which the shortcut and the plain IEEE formulation disagree into *mismatches (host).
 * These calls synchronise the stream.  `which` is one of FO_SELFTEST_*; `arg` selects a
 * sub-case (see the test-suite).
 */
#define FO_SELFTEST_SQRT 0        /* every non-negative finite fp32 */
#define FO_SELFTEST_SOFTSIGN 1    /* every fp32 in [-1, 1] */
#define FO_SELFTEST_RECONSTRUCT 2 /* every (param bits, ecc) pair; arg = param_dtype*100 + ecc_bits */
#define FO_SELFTEST_SPLIT 3       /* every fp32 bit pattern; arg = param_dtype*100 + ecc_bits */
#define FO_SELFTEST_GROUP_DIV 4   /* arg = number of random (a, b) pairs in millions */
#define FO_SELFTEST_CODE_TABLES 5 /* every int8 / uint8 code and every int16 ECC value */
#define FO_SELFTEST_PACKED 7      /* 1e9 random (a*b + c*d) pairs through the packed fp32x2 forms vs scalar; arg 0 = form in use, 1 = plain packed add */
#define FO_SELFTEST_RCP 6         /* reciprocal of every fp32 in [1e-30, 1e30]; arg 0 = variant in use, 1 / 2 = one / two correction steps */
int fo_selftest(int32_t which, int64_t arg, uint64_t* mismatches, void* cuda_stream);

/*
 * fo_selftest without any allocation (no counterpart in the reference).
 *
 * Meant for hosts that may not allocate device memory when they call into the library: the
 * GPU's memory belongs to the embedding framework's own allocator, or cudaMalloc is banned
 * after start-up because it synchronises the whole device, or the allocation entry points
 * are not reachable from the sandbox the plug-in runs in.  The counters the sweeps need live
 * in a static device array of FO_SELFTEST_STATIC_MAX_COUNTERS 64-bit words (32 bytes, held
 * by every GPU that loads the library until the process exits); the call uses no cudaMalloc,
 * cudaFree or other allocating routine.
 *
 * Writes the first n_counters counters of the sweep to `counters` (host): counter 0 is what
 * fo_selftest reports by default; FO_SELFTEST_RCP fills three, FO_SELFTEST_PACKED two.
 * n_counters above FO_SELFTEST_STATIC_MAX_COUNTERS is refused with FO_ERR_TOO_LARGE.
 *
 * The first call on a device looks up the array's device address (with that device current)
 * and caches it; make that first call before starting any stream capture.  All calls share
 * the one array, which is zeroed at the start of each call: calls that overlap on the same
 * GPU (different streams or threads) race on it and must be serialised by the caller.  Like
 * fo_selftest, the call synchronises the stream before it returns.
 */
#define FO_SELFTEST_STATIC_MAX_COUNTERS 4
int fo_selftest_static(int32_t which, int64_t arg, uint64_t* counters, uint32_t n_counters, void* cuda_stream);

int fo_version(void);
const char* fo_status_string(int status);
const char* fo_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHOPTIM_B200_H_ */
