// Instantiates one slice of the step-kernel family.  Compiled once per (optimizer, state
// kind) with -DFO_INST_OPT=<FO_OPT_*> -DFO_INST_KIND=<0 quant32 | 1 full | 2 none | 3 generic>
// -DFO_INST_NAME=<lookup function name>, so the slices build in parallel.
#include "fo_step.cuh"

#if !defined(FO_INST_OPT) || !defined(FO_INST_KIND) || !defined(FO_INST_NAME)
#error "FO_INST_OPT, FO_INST_KIND and FO_INST_NAME must be defined"
#endif

namespace fo {

#define FO_COMBOS(X) \
  X(FO_BF16, 0) X(FO_BF16, 8) X(FO_BF16, 16) X(FO_F16, 0) X(FO_F16, 8) X(FO_F16, 16) X(FO_F32, 0)

LaunchFn FO_INST_NAME(int pdt, int ecc_bits) {
#if FO_INST_KIND == 3
#define X(P, E) \
  if (pdt == P && ecc_bits == E) return &launch_step_generic<FO_INST_OPT, P, E>;
#else
#define X(P, E) \
  if (pdt == P && ecc_bits == E) return &launch_step<FO_INST_OPT, P, E, FO_INST_KIND>;
#endif
  FO_COMBOS(X)
#undef X
  return nullptr;
}

}  // namespace fo
