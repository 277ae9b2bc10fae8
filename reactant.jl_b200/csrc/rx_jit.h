// Run-time specialisation of fused chains.
//
// The ahead-of-time kernels evaluate a fusion group's elementwise chain with a bytecode
// interpreter, which costs tens of machine instructions per chain op.  For launches large
// enough to be bandwidth-bound, the same kernel skeleton (rx_chain_kernels.cuh) is compiled
// once per distinct chain with NVRTC for sm_100a, with the chain as straight-line code and
// the leaf kinds, register numbers and reduction kind as constants; the cubin is loaded
// through the driver API and cached per device.  XLA plays this role for Reactant
// (src/Compiler.jl:1402-1480 hands the module to XLA.compile, which emits PTX per fusion).
//
// Specialisation never changes results: generated code pastes the op expressions of
// RX_VM_UNARY_OPS / RX_VM_BINARY_OPS (rx_vm.h) that the interpreter itself is built from,
// and a constant that starts a value is read from the program at run time rather than
// written as a literal, so the compiler cannot evaluate tanhf(c) and the like on its own
// (its value may differ in the last bit from the device's).  A side effect: chains that
// differ only in such constants share one compiled kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "rx_vm.h"

namespace rx {

struct JitKernel {
  void* fn = nullptr;  // CUfunction
  int occupancy = 1;   // resident CTAs per SM at 256 threads
  mutable int smem_limit = 0;  // dynamic shared memory the function has been allowed so far
};

// A kernel of `family` (e.g. "k_map_rows<rx::SpecChain, 2>") specialised for P's chain.
// nullptr when specialisation is switched off, the work is below the threshold, or NVRTC /
// the driver entry points are not available (the caller then runs the interpreter kernel).
// A chain that fails to compile is an error: *failed is set and the message goes to the
// library's last-error slot.
// `extra_members` (optional) is pasted into the generated chain policy: the GEMM epilogue uses it to say which leaf is
// the accumulator and which registers are summed.
// `force`: compile even when specialisation is switched off (a kernel that exists in compiled form only).
const JitKernel* jit_chain_kernel(int device, const VmProgram& P, const char* family, int red_code, int64_t work_elems, bool* failed,
                                  const char* extra_members = nullptr, bool force = false);
// true when the run-time compiler (NVRTC) can be loaded; the driver entry points needed to load and launch what it
// produces exist wherever a CUDA device does
bool jit_available();
// Launch as thread-block clusters of `cluster_x` CTAs with `smem_bytes` of dynamic shared memory.
cudaError_t jit_launch_cluster(const JitKernel* k, unsigned grid_x, unsigned block_x, unsigned cluster_x, size_t smem_bytes, void** args, cudaStream_t stream,
                               bool pdl = false);

// pdl: launch with the programmatic-stream-serialization attribute (the kernel may start before the one in front of
// it on the stream has completed; it synchronises with griddepcontrol.wait itself).
cudaError_t jit_launch(const JitKernel* k, dim3 grid, dim3 block, void** args, cudaStream_t stream, bool pdl = false);

// Threshold in elements per launch (default 2^20); negative switches specialisation off.
void jit_set_min_elems(int64_t n);
// {kernels compiled, in-memory cache hits, compile failures, 1 if NVRTC or the driver API is unavailable,
//  kernels taken from the on-disk cache (RX_JIT_CACHE_DIR)}
void jit_stats(int64_t out[5]);
// Compile only (needs NVRTC but no device): size of the cubin, or -1 with the compiler log in *log.
int64_t jit_compile_only(const VmProgram& P, int red_code, const char* family, std::string* log, const char* extra_members = nullptr);
// Generated source for P (exposed for tests and for reading).
std::string jit_chain_source(const VmProgram& P, int red_code, const char* family, const char* extra_members = nullptr);

}  // namespace rx
