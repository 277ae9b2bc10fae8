// Host-side launch interface of the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "rx_ir.h"
#include "rx_vm.h"

namespace rx {

struct LaunchCtx {
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  int device = 0;                // CUDA ordinal: specialised kernels are loaded per device
  uint32_t* scratch = nullptr;   // per-device partials buffer for two-pass reductions
  size_t scratch_words = 0;
  uint64_t* launches = nullptr;  // counts kernels launched through this context
  // None of the step's operands is written by the kernel launched just before it on this stream: a kernel launched
  // with programmatic stream serialization may then read them before that kernel has completed.
  bool operands_settled = false;
};

int red_code(RedK k, DT dt);

cudaError_t launch_map(const LaunchCtx& c, const VmProgram& P);
// `fused` (optional): all-reduce the scalar over the mesh in the tail of the same kernel.
cudaError_t launch_reduce_full(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, const FusedAllReduce* fused = nullptr);
cudaError_t launch_reduce_row(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, int64_t outer, int64_t red_n);
int reduce_col_splits(int64_t outer, int64_t red_n, int64_t inner, int sm_count);
cudaError_t launch_reduce_col(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, int64_t outer, int64_t red_n,
                              int64_t inner, uint32_t* partials, int nsplit);
// f64 programs (VmProgram::wide, rx_wide.cu): 64-bit-register interpreter kernels.  shape: 0 = everything to one
// value, 1 = [outer][red], 2 = [outer][red][inner]; code: the reduction kind as for f32 (R_FADD ...) with f64 = true
// when the reduced values are doubles, else the 32-bit integer / predicate code; init: raw bits of the init value.
cudaError_t launch_wide_map(const LaunchCtx& c, const VmProgram& P);
cudaError_t launch_wide_reduce(const LaunchCtx& c, const VmProgram& P, int shape, int code, bool f64, uint64_t init, int64_t outer, int64_t red_n, int64_t inner);
cudaError_t launch_wide_scan(const LaunchCtx& c, const void* src, void* dst, int code, int64_t outer, int64_t n, int64_t inner);
cudaError_t launch_wide_gemm(const LaunchCtx& c, const void* a, const void* b, void* d, int64_t M, int64_t N, int64_t K, int64_t batch, int64_t a_sm, int64_t a_sk, int64_t b_sk,
                             int64_t b_sn, int64_t a_sb, int64_t b_sb, int64_t d_sb);
// inclusive scan along the middle dim of a dense [outer][n][inner] array of 32-bit elements
cudaError_t launch_scan(const LaunchCtx& c, const void* src, void* dst, int code, int64_t outer, int64_t n, int64_t inner);
// dst[c] = init + src[0][c] + src[1][c] + ... (rows added in index order) for up to four jobs in one launch: the
// second pass of the sums a GEMM epilogue leaves as per-row-block / per-tile partials.
struct SumPartialsJob {
  const float* src;
  float* dst;
  int64_t rows, n;
  float init;
};
cudaError_t launch_sum_partials(const LaunchCtx& c, const SumPartialsJob* jobs, int n_jobs);
cudaError_t launch_logsumexp(const LaunchCtx& c, const float* x, int64_t row_stride, int64_t rows, int64_t cols, float* m, float* s, float* lse);

// 2-D stencil step: out window = chain(shifted windows of src), tiles staged through
// shared memory by TMA.  `tmap` is a CUtensorMap for the source array.
struct StencilArgs {
  const void* tmap;          // host pointer to a 128-byte CUtensorMap
  const float* src;
  float* dst;
  int64_t rows, cols;        // output window
  int64_t src_ld, dst_ld, src_off, dst_off;
  int n_taps;
  int dy[8], dx[8];
};
cudaError_t launch_stencil(const LaunchCtx& c, const VmProgram& P, const StencilArgs& a);

}  // namespace rx
