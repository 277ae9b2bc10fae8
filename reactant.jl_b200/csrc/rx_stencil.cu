// Stencil step.  First path: the generic strided map kernel (neighbouring reads
// are served by L1/L2).  The TMA-staged shared-memory kernel replaces it for
// f32 windows when the tensor-map entry point is available.
#include "rx_stencil.h"

namespace rx {

cudaError_t run_stencil_tma(RxDevice* d, const Step& st, const VmProgram& P, bool* handled);

cudaError_t run_stencil(RxDevice* d, const Step& st, const VmProgram& P) {
  bool handled = false;
  cudaError_t e = run_stencil_tma(d, st, P, &handled);
  d->last_stencil_tma = handled;
  if (handled) return e;
  return launch_map(d->ctx(), P);
}

__attribute__((weak)) cudaError_t run_stencil_loop(RxDevice*, const std::vector<const Step*>&, const std::vector<VmProgram>&, int64_t, bool* handled) {
  *handled = false;
  return cudaSuccess;
}

__attribute__((weak)) cudaError_t run_stencil_tma(RxDevice*, const Step&, const VmProgram&, bool* handled) {
  *handled = false;
  return cudaSuccess;
}

}  // namespace rx
