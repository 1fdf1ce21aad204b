// XLA typed-FFI shim over the C ABI: what replaces the reference's pl.pallas_call
// (flashoptim_jax/adamw.py:308-330, flashoptim_jax/momentum_kernel.py:261-286) when the library is
// called from JAX.  Two handlers, one per kernel family, both variadic: one call carries every leaf
// of a pytree that shares the compile-time switches of the reference's call (param dtype, ECC width,
// quantized or full moments, group size) and makes ONE fo_step call (the multi-tensor launch).
//
// Compiled only where jaxlib's headers exist (python -m flashoptim_jax_b200.build looks for
// jax.ffi.include_dir()); it needs nothing but xla/ffi/api/ffi.h, the CUDA runtime and
// include/flashoptim_b200.h.
//
// Operand layout.  Per leaf, in the reference's own operand order, then one device float[3]
// {lr, bias_correction1, bias_correction2} per hyper-parameter set (the reference's traced 0-d
// operands adamw.py:272-278, momentum_kernel.py:230-233 stay device values: no host round trip
// under jit; the momentum family reads lr only):
//   fo_adam_step,     quantize=1: grad, param, ecc, mu_values, nu_values, mu_scales, nu_scales   (adamw.py:269-279)
//                     quantize=0: grad, param, ecc, mu, nu                                       (adamw.py:294-297)
//   fo_momentum_step, quantize=1: grad, param, ecc, mu_values, mu_scales                         (momentum_kernel.py:224-229)
//                     quantize=0: grad, param, ecc, mu                                           (momentum_kernel.py:247-251)
// Results per leaf, in the reference's output order, each meant to alias its operand (the Python
// side passes input_output_aliases built by the tables below times the leaf index, exactly the
// reference's maps adamw.py:268,293 and momentum_kernel.py:222,246); when XLA did not alias a pair
// (no donation) the operand is copied into the result first and the kernel updates the result:
//   adam quantize=1: param, ecc, mu_values, mu_scales, nu_values, nu_scales     aliases {1:0, 2:1, 3:2, 5:3, 4:4, 6:5}
//   adam quantize=0: param, ecc, mu, nu                                         aliases {1:0, 2:1, 3:2, 4:3}
//   momentum quantize=1: param, ecc, mu_values, mu_scales                       aliases {1:0, 2:1, 3:2, 4:3}
//   momentum quantize=0: param, ecc, mu                                         aliases {1:0, 2:1, 3:2}
// As in the reference, a leaf without ECC still passes a dummy ecc array (utils.py:459-461); with
// use_ecc = 0 it is handed through untouched.
//
// Attributes: n_leaves, n_hypers, quantize, use_ecc, group_size (i32); hyper_of (i32 per leaf);
// per hyper set the compile-time floats of the reference's call as arrays of length n_hypers:
//   adam:     wd, b1, b2, one_minus_b1, one_minus_b2, eps, flags (u32 bits as i32: FO_FLAG_*)
//   momentum: wd, mom_coef, update_coef, one_minus_update_coef, one_minus_mom_coef, flags, and do_lion (i32)
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "../../include/flashoptim_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

struct Family {
  int inputs_per_leaf;
  int outputs_per_leaf;
  int alias_of_output[6];  // operand slot (inside the leaf's group) each result aliases
};
// the reference's alias maps, inverted (result -> operand)
constexpr Family kAdamQuant = {7, 6, {1, 2, 3, 5, 4, 6}};
constexpr Family kAdamFull = {5, 4, {1, 2, 3, 4, 0, 0}};
constexpr Family kMomentumQuant = {5, 4, {1, 2, 3, 4, 0, 0}};
constexpr Family kMomentumFull = {4, 3, {1, 2, 3, 0, 0, 0}};

ffi::Error Invalid(const std::string& what) { return ffi::Error(ffi::ErrorCode::kInvalidArgument, what); }

int DtypeCode(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F32: return FO_F32;
    case ffi::DataType::BF16: return FO_BF16;
    case ffi::DataType::F16: return FO_F16;
    default: return -1;
  }
}

size_t ByteWidth(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F32: case ffi::DataType::S32: case ffi::DataType::U32: return 4;
    case ffi::DataType::BF16: case ffi::DataType::F16: case ffi::DataType::S16: case ffi::DataType::U16: return 2;
    case ffi::DataType::S8: case ffi::DataType::U8: return 1;
    default: return 0;
  }
}

// One step of either family.  `hypers` arrives filled except for dev_scalars.
ffi::Error Step(cudaStream_t stream, ffi::RemainingArgs args, ffi::RemainingRets rets, const Family& fam, int opt, int state,
                int32_t n_leaves, int32_t n_hypers, bool has_nu, bool quantize, bool use_ecc, int32_t group_size,
                ffi::Span<const int32_t> hyper_of, std::vector<FoHyper>& hypers) {
  if (n_leaves < 0 || n_hypers < 1 || n_hypers > FO_MAX_HYPERS) return Invalid("n_leaves / n_hypers out of range");
  if ((int64_t)args.size() != (int64_t)n_leaves * fam.inputs_per_leaf + n_hypers) return Invalid("operand count does not match n_leaves, n_hypers");
  if ((int64_t)rets.size() != (int64_t)n_leaves * fam.outputs_per_leaf) return Invalid("result count does not match n_leaves");
  if ((int64_t)hyper_of.size() != n_leaves) return Invalid("hyper_of needs one entry per leaf");
  for (int32_t h = 0; h < n_hypers; ++h) {
    auto s = args.get<ffi::AnyBuffer>((size_t)n_leaves * fam.inputs_per_leaf + h);
    if (!s.has_value()) return s.error();
    if (s->element_type() != ffi::DataType::F32 || s->element_count() < 3) return Invalid("scalars operand must be f32[3]: lr, bias_correction1, bias_correction2");
    hypers[h].dev_scalars = reinterpret_cast<const float*>(s->untyped_data());
  }
  if (n_leaves == 0) return ffi::Error::Success();

  std::vector<FoLeaf> leaves((size_t)n_leaves);
  int param_dtype = -1, grad_dtype = -1, ecc_bits = 0;
  for (int32_t i = 0; i < n_leaves; ++i) {
    const size_t in0 = (size_t)i * fam.inputs_per_leaf, out0 = (size_t)i * fam.outputs_per_leaf;
    // results first: copy an operand into a result XLA did not alias, then work on the results
    void* out_ptr[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    for (int o = 0; o < fam.outputs_per_leaf; ++o) {
      auto src = args.get<ffi::AnyBuffer>(in0 + fam.alias_of_output[o]);
      auto dst = rets.get<ffi::AnyBuffer>(out0 + o);
      if (!src.has_value()) return src.error();
      if (!dst.has_value()) return dst.error();
      const size_t bytes = src->element_count() * ByteWidth(src->element_type());
      if ((*dst)->element_count() != src->element_count() || (*dst)->element_type() != src->element_type())
        return Invalid("a result does not have the shape / dtype of the operand it aliases");
      out_ptr[o] = (*dst)->untyped_data();
      if (out_ptr[o] != src->untyped_data() && bytes != 0) {
        cudaError_t e = cudaMemcpyAsync(out_ptr[o], src->untyped_data(), bytes, cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) return ffi::Error(ffi::ErrorCode::kInternal, std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e));
      }
    }
    auto grad = args.get<ffi::AnyBuffer>(in0 + 0);
    auto param = args.get<ffi::AnyBuffer>(in0 + 1);
    auto ecc = args.get<ffi::AnyBuffer>(in0 + 2);
    if (!grad.has_value()) return grad.error();
    if (!param.has_value()) return param.error();
    if (!ecc.has_value()) return ecc.error();
    const int pdt = DtypeCode(param->element_type()), gdt = DtypeCode(grad->element_type());
    if (pdt < 0 || gdt < 0) return Invalid("param / grad dtype must be f32, bf16 or f16");
    int eb = 0;
    if (use_ecc) {
      if (ecc->element_type() == ffi::DataType::S8) eb = 8;
      else if (ecc->element_type() == ffi::DataType::S16) eb = 16;
      else return Invalid("ecc dtype must be int8 or int16");
    }
    if (i == 0) {
      param_dtype = pdt; grad_dtype = gdt; ecc_bits = eb;
    } else if (pdt != param_dtype || gdt != grad_dtype || eb != ecc_bits) {
      return Invalid("all leaves of one call share param dtype, grad dtype and ECC width");
    }
    if (grad->element_count() != param->element_count()) return Invalid("grad and param differ in size");
    if (hyper_of[i] < 0 || hyper_of[i] >= n_hypers) return Invalid("hyper_of entry out of range");
    FoLeaf& L = leaves[(size_t)i];
    L.grad = grad->untyped_data();
    L.param = out_ptr[0];
    L.ecc = use_ecc ? out_ptr[1] : nullptr;
    L.mu = out_ptr[2];
    // result order (quantized): adam  param, ecc, mu_values, mu_scales, nu_values, nu_scales;  momentum  param, ecc, mu_values, mu_scales
    L.mu_scales = quantize ? out_ptr[3] : nullptr;
    L.nu = has_nu ? (quantize ? out_ptr[4] : out_ptr[3]) : nullptr;
    L.nu_scales = (has_nu && quantize) ? out_ptr[5] : nullptr;
    L.n = (uint64_t)param->element_count();
    L.hyper = (uint32_t)hyper_of[i];
    L.reserved = 0;
  }

  FoStepDesc d = {};
  d.struct_size = sizeof(FoStepDesc);
  d.opt = opt;
  d.param_dtype = param_dtype;
  d.grad_dtype = grad_dtype;
  d.ecc_bits = ecc_bits;
  d.state = state;
  d.group_size = group_size;
  d.n_leaves = (uint32_t)n_leaves;
  d.n_hypers = (uint32_t)n_hypers;
  d.leaves = leaves.data();
  d.hypers = hypers.data();
  const int rc = fo_step(&d, stream);  // copies the tables into kernel parameters before it returns
  if (rc != FO_OK) return ffi::Error(rc == FO_ERR_INVALID_ARG ? ffi::ErrorCode::kInvalidArgument : ffi::ErrorCode::kInternal,
                                     std::string(fo_status_string(rc)) + ": " + fo_last_error());
  return ffi::Error::Success();
}

ffi::Error AdamStep(cudaStream_t stream, ffi::RemainingArgs args, ffi::RemainingRets rets, int32_t n_leaves, int32_t n_hypers,
                    int32_t quantize, int32_t use_ecc, int32_t group_size, ffi::Span<const int32_t> hyper_of,
                    ffi::Span<const float> wd, ffi::Span<const float> b1, ffi::Span<const float> b2,
                    ffi::Span<const float> one_minus_b1, ffi::Span<const float> one_minus_b2, ffi::Span<const float> eps,
                    ffi::Span<const int32_t> flags) {
  const size_t nh = n_hypers < 0 ? 0 : (size_t)n_hypers;
  if (wd.size() != nh || b1.size() != nh || b2.size() != nh || one_minus_b1.size() != nh || one_minus_b2.size() != nh ||
      eps.size() != nh || flags.size() != nh)
    return Invalid("every hyper-parameter array needs n_hypers entries");
  std::vector<FoHyper> hypers(nh);
  for (size_t h = 0; h < nh; ++h) {
    FoHyper& H = hypers[h];
    H.lr = 0.0f; H.bc1 = 1.0f; H.bc2 = 1.0f;  // read from dev_scalars
    H.wd = wd[h]; H.b1 = b1[h]; H.b2 = b2[h]; H.one_minus_b1 = one_minus_b1[h]; H.one_minus_b2 = one_minus_b2[h]; H.eps = eps[h];
    H.flags = (uint32_t)flags[h];
    H.dev_scalars = nullptr;
  }
  return Step(stream, args, rets, quantize ? kAdamQuant : kAdamFull, FO_OPT_ADAM, quantize ? FO_STATE_QUANT : FO_STATE_FULL, n_leaves,
              n_hypers, /*has_nu=*/true, quantize != 0, use_ecc != 0, group_size, hyper_of, hypers);
}

ffi::Error MomentumStep(cudaStream_t stream, ffi::RemainingArgs args, ffi::RemainingRets rets, int32_t n_leaves, int32_t n_hypers,
                        int32_t quantize, int32_t use_ecc, int32_t group_size, int32_t do_lion, ffi::Span<const int32_t> hyper_of,
                        ffi::Span<const float> wd, ffi::Span<const float> mom_coef, ffi::Span<const float> update_coef,
                        ffi::Span<const float> one_minus_update_coef, ffi::Span<const float> one_minus_mom_coef,
                        ffi::Span<const int32_t> flags) {
  const size_t nh = n_hypers < 0 ? 0 : (size_t)n_hypers;
  if (wd.size() != nh || mom_coef.size() != nh || update_coef.size() != nh || one_minus_update_coef.size() != nh ||
      one_minus_mom_coef.size() != nh || flags.size() != nh)
    return Invalid("every hyper-parameter array needs n_hypers entries");
  std::vector<FoHyper> hypers(nh);
  for (size_t h = 0; h < nh; ++h) {
    FoHyper& H = hypers[h];
    H.lr = 0.0f; H.bc1 = 1.0f; H.bc2 = 1.0f; H.eps = 0.0f;
    H.wd = wd[h];
    if (do_lion) {
      // lion.py:95-96: mom_coef = b2, update_coef = b1; FoHyper: b1 = update coefficient, b2 = momentum coefficient
      H.b1 = update_coef[h]; H.b2 = mom_coef[h];
      H.one_minus_b1 = one_minus_update_coef[h]; H.one_minus_b2 = one_minus_mom_coef[h];
    } else {
      // sgd.py:104-105: mom_coef = momentum, update_coef = 1 - dampening; FoHyper: b1 = momentum, one_minus_b1 = 1 - dampening
      H.b1 = mom_coef[h]; H.b2 = 0.0f;
      H.one_minus_b1 = update_coef[h]; H.one_minus_b2 = 0.0f;
    }
    H.flags = (uint32_t)flags[h];
    H.dev_scalars = nullptr;
  }
  return Step(stream, args, rets, quantize ? kMomentumQuant : kMomentumFull, do_lion ? FO_OPT_LION : FO_OPT_SGD,
              quantize ? FO_STATE_QUANT : FO_STATE_FULL, n_leaves, n_hypers, /*has_nu=*/false, quantize != 0, use_ecc != 0, group_size,
              hyper_of, hypers);
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(FoAdamStep, AdamStep,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .RemainingArgs()
                                  .RemainingRets()
                                  .Attr<int32_t>("n_leaves")
                                  .Attr<int32_t>("n_hypers")
                                  .Attr<int32_t>("quantize")
                                  .Attr<int32_t>("use_ecc")
                                  .Attr<int32_t>("group_size")
                                  .Attr<ffi::Span<const int32_t>>("hyper_of")
                                  .Attr<ffi::Span<const float>>("wd")
                                  .Attr<ffi::Span<const float>>("b1")
                                  .Attr<ffi::Span<const float>>("b2")
                                  .Attr<ffi::Span<const float>>("one_minus_b1")
                                  .Attr<ffi::Span<const float>>("one_minus_b2")
                                  .Attr<ffi::Span<const float>>("eps")
                                  .Attr<ffi::Span<const int32_t>>("flags"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(FoMomentumStep, MomentumStep,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .RemainingArgs()
                                  .RemainingRets()
                                  .Attr<int32_t>("n_leaves")
                                  .Attr<int32_t>("n_hypers")
                                  .Attr<int32_t>("quantize")
                                  .Attr<int32_t>("use_ecc")
                                  .Attr<int32_t>("group_size")
                                  .Attr<int32_t>("do_lion")
                                  .Attr<ffi::Span<const int32_t>>("hyper_of")
                                  .Attr<ffi::Span<const float>>("wd")
                                  .Attr<ffi::Span<const float>>("mom_coef")
                                  .Attr<ffi::Span<const float>>("update_coef")
                                  .Attr<ffi::Span<const float>>("one_minus_update_coef")
                                  .Attr<ffi::Span<const float>>("one_minus_mom_coef")
                                  .Attr<ffi::Span<const int32_t>>("flags"));
