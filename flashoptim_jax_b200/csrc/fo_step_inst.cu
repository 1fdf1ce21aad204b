// Instantiates one slice of the step-kernel family.  Compiled once per (optimizer, state kind,
// with / without the peer and clipping code) with -DFO_INST_OPT=<FO_OPT_*>
// -DFO_INST_KIND=<0 quant32 | 1 full | 2 none | 3 generic> -DFO_INST_AUX=<0 | 1>
// -DFO_INST_NAME=<lookup function name>, so the slices build in parallel and each can have its own
// block size (-DFO_THREADS, -DFO_MIN_BLOCKS_*).
#include "fo_step.cuh"

#if !defined(FO_INST_OPT) || !defined(FO_INST_KIND) || !defined(FO_INST_NAME) || !defined(FO_INST_AUX)
#error "FO_INST_OPT, FO_INST_KIND, FO_INST_AUX and FO_INST_NAME must be defined"
#endif

namespace fo {

#define FO_COMBOS(X) \
  X(FO_BF16, 0) X(FO_BF16, 8) X(FO_BF16, 16) X(FO_F16, 0) X(FO_F16, 8) X(FO_F16, 16) X(FO_F32, 0)

Launcher FO_INST_NAME(int pdt, int ecc_bits) {
#if FO_INST_KIND == 3
#define X(P, E) \
  if (pdt == P && ecc_bits == E) return Launcher{&launch_step_generic<FO_INST_OPT, P, E>, 0u};
#else
#define X(P, E) \
  if (pdt == P && ecc_bits == E) return Launcher{&launch_step<FO_INST_OPT, P, E, FO_INST_KIND, FO_INST_AUX != 0>, (unsigned int)kChunk};
#endif
  FO_COMBOS(X)
#undef X
  return Launcher{nullptr, 0u};
}

}  // namespace fo
