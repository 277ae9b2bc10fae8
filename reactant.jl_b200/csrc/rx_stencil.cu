// Stencil step: the TMA-staged shared-memory kernel (rx_stencil_tma.cu) takes f32 windows whose row pitch is a
// multiple of 16 bytes; any other window runs the generic strided map kernel (neighbouring reads are served by
// L1/L2).  Both are part of the library: a build without rx_stencil_tma.cu does not link.
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

}  // namespace rx
