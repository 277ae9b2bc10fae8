// Stencil step launcher: shifted-window sums written into an interior window
// (slice/add chains + dynamic_update_slice, src/Indexing.jl:350-446, 552-627).
#pragma once
#include "rx_runtime.h"

namespace rx {
cudaError_t run_stencil(RxDevice* d, const Step& st, const VmProgram& bound);
}
