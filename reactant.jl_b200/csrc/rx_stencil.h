// Stencil step launcher: shifted-window sums written into an interior window
// (slice/add chains + dynamic_update_slice, src/Indexing.jl:350-446, 552-627).
#pragma once
#include <vector>

#include "rx_halo.cuh"
#include "rx_runtime.h"

namespace rx {
cudaError_t run_stencil(RxDevice* d, const Step& st, const VmProgram& bound);
// For a loop over row-sharded arrays: the kernel exchanges boundary rows with the neighbouring devices between sweeps
// (rx_halo.cuh).  args.block / args.epoch are per sweep: block[i] is the array step i writes, the exchange after
// sweep s carries sequence number epoch0 + s.
struct StencilLoopHalo {
  HaloArgs args;
  std::vector<float*> block;
  unsigned epoch0 = 0;
  // whether update-window rows lie directly above / below the rows this device owns (they are a neighbour's): with
  // two sweeps per pass the intermediate state of those rows is computed here too
  bool window_above = false, window_below = false;
};
// `total` sweeps cycling through `steps` (bound to their buffers) in one launch; *handled = false: not taken.
// dry_run: decide only (every device of a sharded loop must take the launch, or none).  *passes (optional): how many
// passes over memory the launch makes (double sweeps count once); a sharded loop exchanges rows after all but the last.
cudaError_t run_stencil_loop(RxDevice* d, const std::vector<const Step*>& steps, const std::vector<VmProgram>& bound, int64_t total, bool* handled,
                             const StencilLoopHalo* halo = nullptr, bool dry_run = false, int* passes = nullptr);
}
