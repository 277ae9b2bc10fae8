/* CPU oracle kernels -- TEST INFRASTRUCTURE, not part of the product.
 *
 * Plain C/OpenMP restatements of the three HBM-bound benchmark programs, used
 * (a) by the parity tests at sizes where the numpy interpreter is too slow and
 * (b) as the timed CPU baseline of the benchmark.  Only tests/, the smoke check
 * and bench.py's CPU legs may load this file's library.
 *
 * What is restated (paths in the Reactant.jl tree):
 *   sinsum_add      f(x,y) = sum(sin.(x) .+ y): broadcast -> elementwise ops
 *                   (src/TracedUtils.jl:1202-1352, src/Ops.jl:398-460,536-589),
 *                   sum -> stablehlo.reduce with add/0 (src/TracedRArray.jl:187-230,
 *                   src/Ops.jl:3491-3622).
 *   logsumexp_dims1 m = maximum(x; dims=1); m .+ log.(sum(exp.(x .- m); dims=1))
 *                   (ext/ReactantLogExpFunctionsExt.jl:152-155; identities
 *                   src/TracedRArray.jl:128-140).
 *   jacobi2d        slice/add chain + interior update + swap, repeated
 *                   (benchmark/polybench/stencil.jl:263-289; src/Indexing.jl:552-627,
 *                   350-446).
 * The arithmetic of the reference itself is XLA's CPU backend (third party, not
 * in the tree, pinned through Enzyme-JAX 51a4cd6c58b1950f28b650167d1e946eec8ec0d5);
 * these loops follow the StableHLO op semantics.  fp32 sums are accumulated in
 * blocks (fp32 lanes inside a block, double across blocks) so that the result is
 * within the 1e-5*sqrt(log2 n) bar of the exact sum.
 * Arrays are in the boundary layout: row-major over reversed Julia dims.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int rx_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* The OpenMP runtime takes its default team size from OMP_NUM_THREADS, which launchers such as
 * torch.distributed.run set to 1 for every child; callers that want all host cores say so here. */
void rx_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* Ground truth for the tolerance checks at full size: sum(sin(x) + y) with sin evaluated and everything
 * accumulated in double (blocks of 4096 summed serially, block sums added in index order by the reduction),
 * together with the sum of squares of the terms (the scale an ill-conditioned sum is judged against). */
void rx_oracle_sinsum_add_f64(const float* x, const float* y, int64_t n, double* sum, double* sumsq) {
  const int64_t BLK = 4096;
  int64_t nblk = (n + BLK - 1) / BLK;
  double total = 0.0, sq = 0.0;
#pragma omp parallel for reduction(+ : total, sq) schedule(static)
  for (int64_t b = 0; b < nblk; ++b) {
    int64_t lo = b * BLK, hi = lo + BLK < n ? lo + BLK : n;
    double s = 0.0, q = 0.0;
    for (int64_t i = lo; i < hi; ++i) {
      double t = sin((double)x[i]) + (double)y[i];
      s += t;
      q += t * t;
    }
    total += s;
    sq += q;
  }
  *sum = total;
  *sumsq = sq;
}

float rx_oracle_sinsum_add(const float* x, const float* y, int64_t n) {
  const int64_t BLK = 4096;
  int64_t nblk = (n + BLK - 1) / BLK;
  double total = 0.0;
#pragma omp parallel for reduction(+ : total) schedule(static)
  for (int64_t b = 0; b < nblk; ++b) {
    int64_t lo = b * BLK, hi = lo + BLK < n ? lo + BLK : n;
    float lane[16] = {0};
    int64_t i = lo;
    for (; i + 16 <= hi; i += 16)
      for (int l = 0; l < 16; ++l) lane[l] += sinf(x[i + l]) + y[i + l];
    float s = 0.f;
    for (; i < hi; ++i) s += sinf(x[i]) + y[i];
    for (int w = 8; w > 0; w >>= 1)
      for (int l = 0; l < w; ++l) lane[l] += lane[l + w];
    total += (double)(lane[0] + s);
  }
  return (float)total;
}

/* x: [cols][rows] (Julia rows x cols, dims=1 reduces the contiguous axis); out: [cols] */
void rx_oracle_logsumexp_dims1(const float* x, int64_t rows, int64_t cols, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < cols; ++c) {
    const float* r = x + c * rows;
    float m = -INFINITY;
    for (int64_t i = 0; i < rows; ++i) m = r[i] > m ? r[i] : m;
    float lane[16] = {0};
    int64_t i = 0;
    for (; i + 16 <= rows; i += 16)
      for (int l = 0; l < 16; ++l) lane[l] += expf(r[i + l] - m);
    double s = 0.0;
    for (; i < rows; ++i) s += expf(r[i] - m);
    for (int l = 0; l < 16; ++l) s += lane[l];
    out[c] = m + logf((float)s);
  }
}

/* A, B: [n][n]; `steps` sweeps; after each sweep the roles swap.  On return A
 * holds what the program's first result holds and B the second.
 * order 0: the terms are added as centre, minor-1, minor+1, major-1, major+1 (A[c] .+ A[i-1] .+ A[i+1] .+ A[j-1]
 *          .+ A[j+1] on a column-major Julia array: i is the contiguous index);
 * order 1: centre, major-1, major+1, minor+1, minor-1 (the order of benchmark/polybench/stencil.jl:267-287, whose
 *          iteration updates B from A and then A from B: two sweeps of this function). */
void rx_oracle_jacobi2d_order(float* A, float* B, int64_t n, int64_t steps, int order) {
  float *a = A, *b = B;
  for (int64_t t = 0; t < steps; ++t) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 1; i < n - 1; ++i) {
      const float* c = a + i * n;
      float* o = b + i * n;
      if (order == 0) {
        for (int64_t j = 1; j < n - 1; ++j) {
          float s = c[j] + c[j - 1];
          s = s + c[j + 1];
          s = s + c[j - n];
          s = s + c[j + n];
          o[j] = 0.2f * s;
        }
      } else {
        for (int64_t j = 1; j < n - 1; ++j) {
          float s = c[j] + c[j - n];
          s = s + c[j + n];
          s = s + c[j + 1];
          s = s + c[j - 1];
          o[j] = 0.2f * s;
        }
      }
    }
    float* tmp = a; a = b; b = tmp;
  }
  if (a != A) { /* odd number of sweeps: results sit in swapped buffers */
    size_t bytes = (size_t)n * n * sizeof(float);
    float* t = (float*)malloc(bytes);
    memcpy(t, A, bytes); memcpy(A, B, bytes); memcpy(B, t, bytes);
    free(t);
  }
}

void rx_oracle_jacobi2d(float* A, float* B, int64_t n, int64_t steps) { rx_oracle_jacobi2d_order(A, B, n, steps, 0); }
