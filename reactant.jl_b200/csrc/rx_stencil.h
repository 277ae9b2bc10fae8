// Stencil step launcher: shifted-window sums written into an interior window
// (slice/add chains + dynamic_update_slice, src/Indexing.jl:350-446, 552-627).
#pragma once
#include <vector>

#include "rx_runtime.h"

namespace rx {
cudaError_t run_stencil(RxDevice* d, const Step& st, const VmProgram& bound);
// `total` sweeps cycling through `steps` (bound to their buffers) in one launch; *handled = false: not taken.
cudaError_t run_stencil_loop(RxDevice* d, const std::vector<const Step*>& steps, const std::vector<VmProgram>& bound, int64_t total, bool* handled);
}
