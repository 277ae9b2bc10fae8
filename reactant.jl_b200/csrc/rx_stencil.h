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
};
// `total` sweeps cycling through `steps` (bound to their buffers) in one launch; *handled = false: not taken.
// dry_run: decide only (every device of a sharded loop must take the launch, or none).
cudaError_t run_stencil_loop(RxDevice* d, const std::vector<const Step*>& steps, const std::vector<VmProgram>& bound, int64_t total, bool* handled,
                             const StencilLoopHalo* halo = nullptr, bool dry_run = false);
}
