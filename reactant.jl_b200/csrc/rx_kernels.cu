// sm_100a kernels for the fused map / map-reduce templates.
//
//  * k_map_*           elementwise chains (StableHLO elementwise ops after
//                       Reactant's enzyme-batch pass, src/TracedUtils.jl:1202-1352)
//  * k_reduce_full_*   chain -> stablehlo.reduce to a scalar (src/Ops.jl:3491-3622),
//                       deterministic two-pass combine across CTAs
//  * k_reduce_row/col  chain -> reduce along one axis
//  * k_logsumexp       max / sum(exp(x - max)) / max + log(sum) of every row in one
//                       HBM read (ext/ReactantLogExpFunctionsExt.jl:152-155 spelling)
//
// All of them are HBM-bound streaming kernels: 128-bit coalesced loads, several
// independent loads in flight per thread, grids sized in multiples of the SM count.
#include <cstdlib>
#include "rx_kernels.h"

#include <stdio.h>
#include <stdlib.h>
#include <algorithm>
#include <utility>

#include "rx_chain_kernels.cuh"
#include "rx_jit.h"

namespace rx {

namespace {

// Chain policy of the ahead-of-time kernels: the bytecode interpreter, everything read from P.
struct InterpChain {
  static constexpr int kRegs = kVmMaxRegs;
  static __device__ __forceinline__ int n_leaves(const VmProgram& P) { return P.n_leaves; }
  static __device__ __forceinline__ int n_outs(const VmProgram& P) { return P.n_outs; }
  static __device__ __forceinline__ int result_reg(const VmProgram& P) { return P.result_reg; }
  static __device__ __forceinline__ int red_code(int c) { return c; }
  static __device__ __forceinline__ int rank(const VmProgram& P) { return P.rank; }
  static __device__ __forceinline__ int64_t dim(const VmProgram& P, int d) { return P.dim[d]; }
  static __device__ __forceinline__ int leaf_reg(const VmProgram& P, int k) { return P.leaf[k].reg; }
  static __device__ __forceinline__ int out_reg(const VmProgram& P, int k) { return P.out[k].reg; }
  static __device__ __forceinline__ const VmLeaf& leaf(const VmProgram& P, int k) { return P.leaf[k]; }
  static __device__ __forceinline__ const VmOut& out(const VmProgram& P, int k) { return P.out[k]; }
  template <int V>
  static __device__ __forceinline__ void exec(const VmProgram& P, uint32_t (*R)[V], const int64_t* idx) {
    vm_exec<V>(P, R, idx);
  }
};

// ---- full reduce: pass 1 ---------------------------------------------------------
// FAST_SIN_ADD: sum(sin(x) + y) with x = leaf 0, y = leaf 1, both contiguous f32.
__global__ void __launch_bounds__(kThreads) k_reduce_full_sinadd(const float* __restrict__ x, const float* __restrict__ y, int64_t n, uint32_t* __restrict__ partials,
                                                                 unsigned* ticket, uint32_t init_bits, VmOut out, const __grid_constant__ FusedAllReduce ar, int early) {
  __shared__ uint32_t sm[kThreads / 32];
  if (!early) {
    pdl_wait();
    pdl_release();
  }
  const float4* x4 = (const float4*)x;
  const float4* y4 = (const float4*)y;
  int64_t n4 = n >> 2;
  int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 p0 = __ldcs(x4 + i), p1 = __ldcs(x4 + i + stride), p2 = __ldcs(x4 + i + 2 * stride), p3 = __ldcs(x4 + i + 3 * stride);
    float4 q0 = __ldcs(y4 + i), q1 = __ldcs(y4 + i + stride), q2 = __ldcs(y4 + i + 2 * stride), q3 = __ldcs(y4 + i + 3 * stride);
    a0 += sinf(p0.x) + q0.x; a1 += sinf(p0.y) + q0.y; a2 += sinf(p0.z) + q0.z; a3 += sinf(p0.w) + q0.w;
    a0 += sinf(p1.x) + q1.x; a1 += sinf(p1.y) + q1.y; a2 += sinf(p1.z) + q1.z; a3 += sinf(p1.w) + q1.w;
    a0 += sinf(p2.x) + q2.x; a1 += sinf(p2.y) + q2.y; a2 += sinf(p2.z) + q2.z; a3 += sinf(p2.w) + q2.w;
    a0 += sinf(p3.x) + q3.x; a1 += sinf(p3.y) + q3.y; a2 += sinf(p3.z) + q3.z; a3 += sinf(p3.w) + q3.w;
  }
  for (; i < n4; i += stride) {
    float4 p = __ldcs(x4 + i), q = __ldcs(y4 + i);
    a0 += sinf(p.x) + q.x; a1 += sinf(p.y) + q.y; a2 += sinf(p.z) + q.z; a3 += sinf(p.w) + q.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t t = n4 * 4 + threadIdx.x;
    a0 += sinf(x[t]) + y[t];
  }
  float v = (a0 + a1) + (a2 + a3);
  uint32_t r = block_red<kThreads>(R_FADD, f2u(v), sm);
  if (early) {
    pdl_wait();
    pdl_release();
  }
  finish_in_last_block(r, partials, ticket, R_FADD, init_bits, out, sm, ar);
}

// Second pass of the strided-axis reduce: one CTA per 32 adjacent columns of one outer index.  Warp w
// adds the partials of splits w, w+8, ... (lane = column, so every read is a coalesced 128-byte row);
// the eight warp results are then combined in warp order.  The order is fixed, so the result is
// deterministic.
__global__ void __launch_bounds__(kThreads) k_reduce_col_finish(const uint32_t* __restrict__ partials, int code, uint32_t init_bits, int64_t outer, int nsplit, int64_t inner, VmOut out) {
  __shared__ uint32_t sm[kThreads / 32][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t col_blocks = (inner + 31) / 32;
  const int64_t o = blockIdx.x / col_blocks;
  const int64_t b = (blockIdx.x - o * col_blocks) * 32 + lane;
  uint32_t acc = red_identity(code);
  if (b < inner)
    for (int s = w; s < nsplit; s += kThreads / 32) acc = red_combine(code, acc, partials[(o * nsplit + s) * inner + b]);
  sm[w][lane] = acc;
  __syncthreads();
  if (w == 0 && b < inner) {
    uint32_t t = sm[0][lane];
#pragma unroll
    for (int q = 1; q < kThreads / 32; ++q) t = red_combine(code, t, sm[q][lane]);
    out_store(out, out.offset + o * out.stride[0] + b * out.stride[2], red_combine(code, init_bits, t));
  }
}

// ---- logsumexp over rows ----------------------------------------------------------------
__device__ __forceinline__ void lse_push4(float4 v, float& m, float& s) {
  float cm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
  if (cm > m) {
    s *= expf(m - cm);
    m = cm;
  }
  // while only -inf has been seen there is nothing to add (exp(-inf - finite max) = 0 once the max is known)
  if (m > -INFINITY) s += (expf(v.x - m) + expf(v.y - m)) + (expf(v.z - m) + expf(v.w - m));
}
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  float M = fmaxf(m, m2);
  float a = (m == M) ? s : s * expf(m - M);
  float b = (m2 == M) ? s2 : s2 * expf(m2 - M);
  m = M;
  s = a + b;
}

template <int TPR, bool VEC>
__global__ void __launch_bounds__(kThreads) k_logsumexp(const float* __restrict__ x, int64_t row_stride, int64_t rows, int64_t cols,
                                                        float* __restrict__ m_out, float* __restrict__ s_out, float* __restrict__ lse_out) {
  __shared__ float sm_m[kThreads / 32], sm_s[kThreads / 32];
  constexpr int RPB = kThreads / TPR;
  int64_t row = (int64_t)blockIdx.x * RPB + threadIdx.x / TPR;
  int lane = threadIdx.x % TPR;
  float m = -INFINITY, s = 0.f;
  if (row < rows) {
    const float* xr = x + row * row_stride;
    if (VEC) {
      const float4* x4 = (const float4*)xr;
      int64_t c4 = cols >> 2;
      int64_t i = lane;
      for (; i + 3 * TPR < c4; i += 4 * TPR) {
        float4 v0 = __ldcs(x4 + i), v1 = __ldcs(x4 + i + TPR), v2 = __ldcs(x4 + i + 2 * TPR), v3 = __ldcs(x4 + i + 3 * TPR);
        lse_push4(v0, m, s);
        lse_push4(v1, m, s);
        lse_push4(v2, m, s);
        lse_push4(v3, m, s);
      }
      for (; i < c4; i += TPR) lse_push4(__ldcs(x4 + i), m, s);
      for (int64_t c = c4 * 4 + lane; c < cols; c += TPR) {
        float v = xr[c];
        lse_push4(make_float4(v, -INFINITY, -INFINITY, -INFINITY), m, s);
      }
    } else {
      for (int64_t c = lane; c < cols; c += TPR) {
        float v = __ldg(xr + c);
        if (v > m) { s *= expf(m - v); m = v; }
        if (m > -INFINITY) s += expf(v - m);
      }
    }
  }
  // combine across the TPR threads of the row in a fixed order
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    if (o < TPR) {
      float m2 = __shfl_xor_sync(0xFFFFFFFFu, m, o), s2 = __shfl_xor_sync(0xFFFFFFFFu, s, o);
      lse_merge(m, s, m2, s2);
    }
  }
  if (TPR == kThreads) {
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sm_m[w] = m; sm_s[w] = s; }
    __syncthreads();
    if (w == 0) {
      m = l < kThreads / 32 ? sm_m[l] : -INFINITY;
      s = l < kThreads / 32 ? sm_s[l] : 0.f;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xFFFFFFFFu, m, o), s2 = __shfl_xor_sync(0xFFFFFFFFu, s, o);
        lse_merge(m, s, m2, s2);
      }
    }
  }
  if (threadIdx.x % TPR == 0 && row < rows && (TPR != kThreads || threadIdx.x == 0)) {
    if (m == -INFINITY) s = NAN;  // every element was -inf: x - max is inf - inf in the op sequence
    m_out[row] = m;
    s_out[row] = s;
    lse_out[row] = m + logf(s);
  }
}


// ---- inclusive scan along the middle dim of [outer][n][inner] (stablehlo.reduce_window in its cumulative form) ------
// Lines that are strided in memory (inner > 1): one thread per line, sequential along n, coalesced across lines.
// (The combiner is a template parameter of the scan kernels: red_combine() is a switch over ten cases, and a scan
// calls it several times per element.)
template <int CODE>
__global__ void __launch_bounds__(kThreads) k_scan_lines(const uint32_t* __restrict__ x, uint32_t* __restrict__ y, int64_t outer, int64_t n, int64_t inner) {
  constexpr int code = CODE;
  const int64_t line = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (line >= outer * inner) return;
  const int64_t o = line / inner, i = line - o * inner;
  const int64_t base = o * n * inner + i;
  uint32_t acc = red_identity(code);
  int64_t r = 0;
  // eight steps at a time: their loads do not depend on the running value and are issued together
  for (; r + 8 <= n; r += 8) {
    uint32_t v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = __ldg(x + base + (r + q) * inner);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      acc = red_combine(code, acc, v[q]);
      y[base + (r + q) * inner] = acc;
    }
  }
  for (; r < n; ++r) {
    acc = red_combine(code, acc, __ldg(x + base + r * inner));
    y[base + r * inner] = acc;
  }
}

// Few long strided lines do not fill the GPU with a thread per line: the lines are cut into `nseg` segments of `seg`
// steps (blockIdx.y).  Pass 1 leaves every (segment, line) total in partial[segment][line]; pass 2 folds the totals
// of the segments before its own, in order, and scans its segment from there.
template <int CODE, bool APPLY>
__global__ void __launch_bounds__(kThreads) k_scan_lines_seg(const uint32_t* __restrict__ x, uint32_t* __restrict__ y, uint32_t* __restrict__ partial, int64_t outer, int64_t n,
                                                            int64_t inner, int64_t seg) {
  constexpr int code = CODE;
  const int64_t lines = outer * inner, line = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (line >= lines) return;
  const int64_t o = line / inner, i = line - o * inner;
  const int64_t base = o * n * inner + i;
  const int64_t r0 = (int64_t)blockIdx.y * seg, r1 = min(n, r0 + seg);
  uint32_t acc = red_identity(code);
  if (APPLY)
    for (int q = 0; q < (int)blockIdx.y; ++q) acc = red_combine(code, acc, partial[q * lines + line]);
  int64_t r = r0;
  for (; r + 8 <= r1; r += 8) {
    uint32_t v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = __ldg(x + base + (r + q) * inner);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      acc = red_combine(code, acc, v[q]);
      if (APPLY) y[base + (r + q) * inner] = acc;
    }
  }
  for (; r < r1; ++r) {
    acc = red_combine(code, acc, __ldg(x + base + r * inner));
    if (APPLY) y[base + r * inner] = acc;
  }
  if (!APPLY) partial[(int64_t)blockIdx.y * lines + line] = acc;
}

// Contiguous rows (inner == 1), each row cut into `nseg` segments of `seg` elements (a multiple of 1024).
// Pass 1: the combined value of every segment.  Pass 2: every CTA folds the values of the segments before its own
// (in order), then scans its segment 1024 elements at a time: four per thread, warp shuffles, one shared-memory hop
// across the eight warps, and a running carry.  The order of combination is fixed, so results are deterministic.
template <int CODE>
__global__ void __launch_bounds__(kThreads) k_scan_row_partials(const uint32_t* __restrict__ x, uint32_t* __restrict__ partial, int64_t n, int64_t seg, int nseg) {
  constexpr int code = CODE;
  __shared__ uint32_t sm[kThreads / 32];
  const int64_t row = blockIdx.y, s0 = (int64_t)blockIdx.x * seg, s1 = min(n, s0 + seg);
  const uint32_t* xr = x + row * n;
  uint32_t acc = red_identity(code);
  for (int64_t c = s0 + threadIdx.x; c < s1; c += kThreads) acc = red_combine(code, acc, __ldg(xr + c));
  acc = block_red<kThreads>(code, acc, sm);
  if (threadIdx.x == 0) partial[row * nseg + blockIdx.x] = acc;
}

template <int CODE>
__global__ void __launch_bounds__(kThreads) k_scan_row_apply(const uint32_t* __restrict__ x, uint32_t* __restrict__ y, const uint32_t* __restrict__ partial, int64_t n, int64_t seg,
                                                            int nseg) {
  constexpr int code = CODE;
  __shared__ uint32_t warp_tot[kThreads / 32];
  __shared__ uint32_t carry_s;
  const int64_t row = blockIdx.y, s0 = (int64_t)blockIdx.x * seg, s1 = min(n, s0 + seg);
  const uint32_t* xr = x + row * n;
  uint32_t* yr = y + row * n;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  {
    // the segments before this one, folded in a fixed order: a strided share per thread, then the block tree
    uint32_t c = red_identity(code);
    for (int q = threadIdx.x; q < (int)blockIdx.x; q += kThreads) c = red_combine(code, c, partial[row * nseg + q]);
    c = block_red<kThreads>(code, c, warp_tot);
    if (threadIdx.x == 0) carry_s = c;
  }
  __syncthreads();
  uint32_t carry = carry_s;
  const uint32_t ident = red_identity(code);
  auto fetch = [&](int64_t c0, uint32_t* v) {
    const int64_t c = c0 + 4 * threadIdx.x;
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = (c + q < s1) ? __ldg(xr + c + q) : ident;
  };
  uint32_t nv[4];
  fetch(s0, nv);
  for (int64_t c0 = s0; c0 < s1; c0 += 4 * kThreads) {
    const int64_t c = c0 + 4 * threadIdx.x;
    uint32_t v[4] = {nv[0], nv[1], nv[2], nv[3]};
    if (c0 + 4 * kThreads < s1) fetch(c0 + 4 * kThreads, nv);  // the next chunk is on its way during the work on this one
    v[1] = red_combine(code, v[0], v[1]);
    v[2] = red_combine(code, v[1], v[2]);
    v[3] = red_combine(code, v[2], v[3]);
    // inclusive scan of the thread totals across the warp, then across the warps
    uint32_t t = v[3];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t u = __shfl_up_sync(0xFFFFFFFFu, t, o);
      if (lane >= o) t = red_combine(code, u, t);
    }
    if (lane == 31) warp_tot[w] = t;
    __syncthreads();
    uint32_t before = carry;  // everything left of this thread: carry, earlier warps, earlier lanes
    for (int q = 0; q < w; ++q) before = red_combine(code, before, warp_tot[q]);
    uint32_t lane_excl = __shfl_up_sync(0xFFFFFFFFu, t, 1);
    if (lane > 0) before = red_combine(code, before, lane_excl);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (c + q < s1) yr[c + q] = red_combine(code, before, v[q]);
    uint32_t total = carry;
    for (int q = 0; q < kThreads / 32; ++q) total = red_combine(code, total, warp_tot[q]);
    carry = total;
    __syncthreads();  // warp_tot is rewritten by the next chunk
  }
}

// ---- ordered sum of partial rows (second pass of the sums formed in a GEMM epilogue) -----------------------------------
struct SumJobs {
  SumPartialsJob j[4];
};
__global__ void __launch_bounds__(kThreads) k_sum_partials(const __grid_constant__ SumJobs jobs) {
  __shared__ uint32_t sm[kThreads / 32];
  const SumPartialsJob& j = jobs.j[blockIdx.y];
  if (j.n == 1) {
    // one value: every thread adds a strided subset of the rows, then the fixed block tree
    if (blockIdx.x != 0) return;
    float acc = 0.f;
    for (int64_t r = threadIdx.x; r < j.rows; r += kThreads) acc += j.src[r];
    const uint32_t t = block_red<kThreads>(R_FADD, f2u(acc), sm);
    if (threadIdx.x == 0) j.dst[0] = j.init + u2f(t);
    return;
  }
  // 32 columns per block: warp w adds rows w, w + 8, ... (lane = column, so every load is one 128-byte row piece),
  // then the eight warp results are added in warp order
  __shared__ float part[kThreads / 32][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t col = (int64_t)blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (col < j.n)
    for (int64_t r = w; r < j.rows; r += kThreads / 32) acc += __ldg(j.src + r * j.n + col);
  part[w][lane] = acc;
  __syncthreads();
  if (w == 0 && col < j.n) {
    float t = part[0][lane];
#pragma unroll
    for (int q = 1; q < kThreads / 32; ++q) t += part[q][lane];
    j.dst[col] = j.init + t;
  }
}

int grid_for(int64_t work_items, int sm_count, int per_sm) {
  int64_t blocks = (work_items + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)sm_count * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

bool vec_aligned(const VmProgram& P) {
  auto esz = [](int e) { return e == EL_F32 || e == EL_I32 ? 4 : (e == EL_BF16 ? 2 : 1); };
  for (int k = 0; k < P.n_leaves; ++k) {
    if (P.leaf[k].linear != 1) continue;
    int es = esz(P.leaf[k].elem);
    if (((uintptr_t)P.leaf[k].ptr + (uintptr_t)P.leaf[k].offset * es) % (4 * es)) return false;
  }
  for (int k = 0; k < P.n_outs; ++k) {
    int es = esz(P.out[k].elem);
    if (((uintptr_t)P.out[k].ptr + (uintptr_t)P.out[k].offset * es) % (4 * es)) return false;
  }
  return true;
}

// Can [P.dim[drow]][P.dim[dcol]] be walked 4 columns at a time with aligned vector accesses?
bool rowvec_ok(const VmProgram& P, int drow, int dcol, bool check_outs) {
  auto esz = [](int e) { return e == EL_F32 || e == EL_I32 ? 4 : (e == EL_BF16 ? 2 : 1); };
  if (P.dim[dcol] % 4) return false;
  for (int k = 0; k < P.n_instr; ++k)
    if (P.ins[k].op == VM_IOTA) return false;
  for (int k = 0; k < P.n_leaves; ++k) {
    const VmLeaf& l = P.leaf[k];
    if (l.stride[dcol] == 0) continue;
    int es = esz(l.elem);
    if (l.stride[dcol] != 1 || (l.offset % 4) || (l.stride[drow] % 4) || ((uintptr_t)l.ptr % (4 * es))) return false;
  }
  if (check_outs)
    for (int k = 0; k < P.n_outs; ++k) {
      const VmOut& o = P.out[k];
      int es = esz(o.elem);
      if (o.stride[dcol] != 1 || (o.offset % 4) || (o.stride[drow] % 4) || ((uintptr_t)o.ptr % (4 * es))) return false;
    }
  return true;
}

int64_t total_of(const VmProgram& P) {
  int64_t n = 1;
  for (int d = 0; d < P.rank; ++d) n *= P.dim[d];
  return n;
}

}  // namespace

int red_code(RedK k, DT dt) {
  bool f = dt == DT::F32 || dt == DT::BF16 || dt == DT::F64;
  switch (k) {
    case RedK::Add: return f ? R_FADD : R_IADD;
    case RedK::Max: return f ? R_FMAX : R_IMAX;
    case RedK::Min: return f ? R_FMIN : R_IMIN;
    case RedK::Mul: return f ? R_FMUL : R_IMUL;
    case RedK::Or: return R_OR;
    default: return R_AND;
  }
}

// Launch `family` specialised for P's chain when that is worthwhile and possible; otherwise (*ran == false)
// the caller launches the interpreter kernel.
cudaError_t try_specialised(const LaunchCtx& c, const VmProgram& P, const char* family, int code, int64_t work, dim3 grid, void** args, bool* ran,
                            int* occupancy = nullptr, bool pdl = false) {
  *ran = false;
  bool failed = false;
  const JitKernel* k = jit_chain_kernel(c.device, P, family, code, work, &failed);
  if (failed) return cudaErrorUnknown;
  if (!k) return cudaSuccess;
  if (occupancy) {  // the caller only wanted to size its grid
    *occupancy = k->occupancy;
    return cudaSuccess;
  }
  *ran = true;
  return jit_launch(k, grid, dim3(kThreads), args, c.stream, pdl);
}

// registers of the chain's virtual machine that the program uses
static int chain_regs(const VmProgram& P) {
  int r = P.result_reg;
  for (int k = 0; k < P.n_leaves; ++k) r = std::max<int>(r, P.leaf[k].reg);
  for (int k = 0; k < P.n_outs; ++k) r = std::max<int>(r, P.out[k].reg);
  for (int k = 0; k < P.n_instr; ++k)
    if (P.ins[k].flags & VMF_STORE) r = std::max<int>(r, P.ins[k].dst);
  return r + 1;
}

// k_map_runs steps along the last dim in 32-bit arithmetic: 8 steps of 256 elements must fit for every operand (with room to spare)
static bool runs_steps_fit(const VmProgram& P) {
  const int last = P.rank - 1;
  const int64_t lim = ((int64_t)1 << 31) / (16 * 256);
  for (int k = 0; k < P.n_leaves; ++k)
    if (std::llabs(P.leaf[k].stride[last]) >= lim) return false;
  for (int k = 0; k < P.n_outs; ++k)
    if (std::llabs(P.out[k].stride[last]) >= lim) return false;
  return true;
}

// does the chain read the element's index (stablehlo.iota)?
static bool reads_index(const VmProgram& P) {
  for (int k = 0; k < P.n_instr; ++k)
    if (P.ins[k].op == VM_IOTA) return true;
  return false;
}

cudaError_t launch_map(const LaunchCtx& c, const VmProgram& P) {
  int64_t n = total_of(P);
  if (n == 0) return cudaSuccess;
  bool ran = false;
  cudaError_t e = cudaSuccess;
  if (P.all_linear && vec_aligned(P)) {
    dim3 grid(grid_for((n + 3) / 4, c.sm_count, 8));
    void* args[] = {(void*)&P, (void*)&n};
    e = try_specialised(c, P, "k_map_linear<rx::SpecChain>", -1, n, grid, args, &ran);
    if (!ran && e == cudaSuccess) k_map_linear<InterpChain><<<grid, kThreads, 0, c.stream>>>(P, n);
  } else if (P.rank == 2 && rowvec_ok(P, 0, 1, true)) {
    int64_t rows = P.dim[0], cols = P.dim[1];
    void* args[] = {(void*)&P, (void*)&rows, (void*)&cols};
    if (cols % 8 == 0) {
      dim3 grid(grid_for(n / 8, c.sm_count, 8));
      e = try_specialised(c, P, "k_map_rows<rx::SpecChain, 2>", -1, n, grid, args, &ran);
      if (!ran && e == cudaSuccess) k_map_rows<InterpChain, 2><<<grid, kThreads, 0, c.stream>>>(P, rows, cols);
    } else {
      dim3 grid(grid_for(n / 4, c.sm_count, 8));
      e = try_specialised(c, P, "k_map_rows<rx::SpecChain, 1>", -1, n, grid, args, &ran);
      if (!ran && e == cudaSuccess) k_map_rows<InterpChain, 1><<<grid, kThreads, 0, c.stream>>>(P, rows, cols);
    }
  } else if (P.rank >= 1 && P.dim[P.rank - 1] >= 64 && !reads_index(P) && runs_steps_fit(P) && !(getenv("RX_MAP_RUNS") && atoi(getenv("RX_MAP_RUNS")) == 0)) {
    // V elements per thread along the last dim, W lanes apart (k_map_runs); rows shorter than two warps' worth
    // would leave most lanes idle and stay with one element per thread.  V = 4 in the interpreter; a specialised
    // chain with few registers takes 8 when the rows are long enough.
    int64_t inner = P.dim[P.rank - 1], rows = n / inner;
    auto geometry = [&](int v, int* log2w, int64_t* chunks_per_row) {
      *log2w = 5;
      while (*log2w < 8 && ((int64_t)v << *log2w) < inner) ++*log2w;
      *chunks_per_row = (inner + ((int64_t)v << *log2w) - 1) / ((int64_t)v << *log2w);
      return dim3(grid_for(rows * *chunks_per_row << *log2w, c.sm_count, 8));
    };
    const int regs = chain_regs(P);
    int v = (regs <= 8 && inner >= 8 * 256) ? 8 : 4;  // measured: 16 per thread is slower for every chain tried (registers)
    if (const char* ev = getenv("RX_MAP_RUNS_V")) {  // A/B measurements
      const int w = atoi(ev);
      if (w == 4 || w == 8) v = w;
    }
    int log2w;
    int64_t chunks_per_row;
    void* args[] = {(void*)&P, (void*)&rows, (void*)&inner, (void*)&log2w, (void*)&chunks_per_row};
    dim3 grid = geometry(v, &log2w, &chunks_per_row);
    e = try_specialised(c, P, v == 8 ? "k_map_runs<rx::SpecChain, 8>" : "k_map_runs<rx::SpecChain, 4>", -1, n, grid, args, &ran);
    if (!ran && e == cudaSuccess) {
      grid = geometry(4, &log2w, &chunks_per_row);
      k_map_runs<InterpChain, 4><<<grid, kThreads, 0, c.stream>>>(P, rows, inner, log2w, chunks_per_row);
    }
  } else {
    dim3 grid(grid_for(n, c.sm_count, 8));
    void* args[] = {(void*)&P, (void*)&n};
    const bool small = n < ((int64_t)1 << 31);
    e = try_specialised(c, P, small ? "k_map_generic<rx::SpecChain, true>" : "k_map_generic<rx::SpecChain, false>", -1, n, grid, args, &ran);
    if (!ran && e == cudaSuccess) {
      if (small) k_map_generic<InterpChain, true><<<grid, kThreads, 0, c.stream>>>(P, n);
      else k_map_generic<InterpChain, false><<<grid, kThreads, 0, c.stream>>>(P, n);
    }
  }
  if (e != cudaSuccess) return e;
  ++*c.launches;
  return cudaGetLastError();
}

// Resident CTAs per SM of a kernel (registers decide): grids are sized to exactly one
// resident wave so that no CTA starts late and the partial count stays fixed per device.
template <typename K>
int resident_per_sm(K kernel) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, 0) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = 4;
  }
  return n;
}

// Launch with the programmatic-stream-serialization attribute (see pdl_wait in rx_chain_kernels.cuh).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), int blocks, cudaStream_t stream, bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

cudaError_t launch_reduce_full(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, const FusedAllReduce* fused) {
  FusedAllReduce ar{};
  if (fused) ar = *fused;
  static const bool pdl = !(getenv("RX_PDL") && atoi(getenv("RX_PDL")) == 0);
  int early = pdl && c.operands_settled ? 1 : 0;
  int64_t n = total_of(P);
  static const int occ_sinadd = resident_per_sm(k_reduce_full_sinadd), occ_linear = resident_per_sm(k_reduce_full_linear<InterpChain>),
                   occ_rows = resident_per_sm(k_reduce_full_rows<InterpChain>), occ_generic = resident_per_sm(k_reduce_full_generic<InterpChain>);
  const bool vec = P.all_linear && vec_aligned(P);
  const bool sinadd = vec && P.fast_id == FAST_SIN_ADD && code == R_FADD;
  const bool rows2 = !vec && P.rank == 2 && rowvec_ok(P, 0, 1, false);
  const char* family = vec ? "k_reduce_full_linear<rx::SpecChain>" : rows2 ? "k_reduce_full_rows<rx::SpecChain>" : "k_reduce_full_generic<rx::SpecChain>";
  int occ = sinadd ? occ_sinadd : vec ? occ_linear : rows2 ? occ_rows : occ_generic;
  bool ran = false;
  if (!sinadd) {  // a specialised kernel has its own register count, hence its own resident wave
    cudaError_t e = try_specialised(c, P, family, code, n, dim3(1), nullptr, &ran, &occ);
    if (e != cudaSuccess) return e;
  }
  // 16 elements per thread per trip keeps four 128-bit loads in flight per operand
  int blocks = grid_for((n + 15) / 16, c.sm_count, occ);
  if ((size_t)blocks + 1 > c.scratch_words) return cudaErrorInvalidValue;
  uint32_t* partials = c.scratch;
  unsigned* ticket = (unsigned*)(c.scratch + c.scratch_words - 1);  // zeroed at device creation, reset by each launch
  cudaError_t e = cudaSuccess;
  if (sinadd) {
    const float* x = (const float*)P.leaf[0].ptr + P.leaf[0].offset;
    const float* y = (const float*)P.leaf[1].ptr + P.leaf[1].offset;
    e = launch_pdl(k_reduce_full_sinadd, blocks, c.stream, pdl, x, y, n, partials, ticket, init_bits, P.out[0], ar, early);
  } else if (vec) {
    void* args[] = {(void*)&P, (void*)&n, (void*)&code, (void*)&partials, (void*)&ticket, (void*)&init_bits, (void*)&ar, (void*)&early};
    e = try_specialised(c, P, family, code, n, dim3(blocks), args, &ran, nullptr, pdl);
    if (!ran && e == cudaSuccess) e = launch_pdl(k_reduce_full_linear<InterpChain>, blocks, c.stream, pdl, P, n, code, partials, ticket, init_bits, ar, early);
  } else if (rows2) {
    int64_t rows = P.dim[0], cols = P.dim[1];
    void* args[] = {(void*)&P, (void*)&rows, (void*)&cols, (void*)&code, (void*)&partials, (void*)&ticket, (void*)&init_bits, (void*)&ar, (void*)&early};
    e = try_specialised(c, P, family, code, n, dim3(blocks), args, &ran, nullptr, pdl);
    if (!ran && e == cudaSuccess) e = launch_pdl(k_reduce_full_rows<InterpChain>, blocks, c.stream, pdl, P, rows, cols, code, partials, ticket, init_bits, ar, early);
  } else {
    void* args[] = {(void*)&P, (void*)&n, (void*)&code, (void*)&partials, (void*)&ticket, (void*)&init_bits, (void*)&ar, (void*)&early};
    e = try_specialised(c, P, family, code, n, dim3(blocks), args, &ran, nullptr, pdl);
    if (!ran && e == cudaSuccess) e = launch_pdl(k_reduce_full_generic<InterpChain>, blocks, c.stream, pdl, P, n, code, partials, ticket, init_bits, ar, early);
  }
  if (e != cudaSuccess) return e;
  *c.launches += 1;
  return cudaGetLastError();
}

cudaError_t launch_reduce_row(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, int64_t outer, int64_t red_n) {
  if (outer == 0) return cudaSuccess;
  void* args[] = {(void*)&P, (void*)&code, (void*)&init_bits, (void*)&outer, (void*)&red_n};
  bool ran = false;
  cudaError_t e;
  const int64_t work = outer * red_n;
  if (red_n >= 2048) {
    dim3 grid((unsigned)outer);
    e = try_specialised(c, P, "k_reduce_row<rx::SpecChain, 256>", code, work, grid, args, &ran);
    if (!ran && e == cudaSuccess) k_reduce_row<InterpChain, kThreads><<<grid, kThreads, 0, c.stream>>>(P, code, init_bits, outer, red_n);
  } else if (red_n >= 16) {
    dim3 grid((unsigned)((outer + 7) / 8));
    e = try_specialised(c, P, "k_reduce_row<rx::SpecChain, 32>", code, work, grid, args, &ran);
    if (!ran && e == cudaSuccess) k_reduce_row<InterpChain, 32><<<grid, kThreads, 0, c.stream>>>(P, code, init_bits, outer, red_n);
  } else {
    dim3 grid((unsigned)((outer + kThreads - 1) / kThreads));
    e = try_specialised(c, P, "k_reduce_row<rx::SpecChain, 1>", code, work, grid, args, &ran);
    if (!ran && e == cudaSuccess) k_reduce_row<InterpChain, 1><<<grid, kThreads, 0, c.stream>>>(P, code, init_bits, outer, red_n);
  }
  if (e != cudaSuccess) return e;
  ++*c.launches;
  return cudaGetLastError();
}

int reduce_col_splits(int64_t outer, int64_t red_n, int64_t inner, int sm_count) {
  int64_t col_blocks = (inner / 4 + kThreads - 1) / kThreads;
  if (col_blocks < 1) col_blocks = 1;
  int64_t want = ((int64_t)sm_count * 8 + col_blocks * outer - 1) / (col_blocks * outer);
  int64_t ns = std::max<int64_t>(1, std::min<int64_t>(want, std::min<int64_t>(256, (red_n + 15) / 16)));
  return (int)ns;
}

cudaError_t launch_reduce_col(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, int64_t outer, int64_t red_n, int64_t inner, uint32_t* partials, int nsplit) {
  if (outer * inner == 0) return cudaSuccess;
  bool ran = false;
  cudaError_t e;
  const int64_t work = outer * red_n * inner;
  if (outer == 1 && rowvec_ok(P, 1, 2, false)) {
    dim3 grid((unsigned)((inner / 4 + kThreads - 1) / kThreads), (unsigned)nsplit, 1);
    void* args[] = {(void*)&P, (void*)&code, (void*)&red_n, (void*)&inner, (void*)&nsplit, (void*)&partials};
    e = try_specialised(c, P, "k_reduce_col_vec<rx::SpecChain>", code, work, grid, args, &ran);
    if (!ran && e == cudaSuccess) k_reduce_col_vec<InterpChain><<<grid, kThreads, 0, c.stream>>>(P, code, red_n, inner, nsplit, partials);
  } else {
    dim3 grid((unsigned)((inner + kThreads - 1) / kThreads), (unsigned)nsplit, (unsigned)std::min<int64_t>(outer, 65535));
    void* args[] = {(void*)&P, (void*)&code, (void*)&outer, (void*)&red_n, (void*)&inner, (void*)&nsplit, (void*)&partials};
    e = try_specialised(c, P, "k_reduce_col<rx::SpecChain>", code, work, grid, args, &ran);
    if (!ran && e == cudaSuccess) k_reduce_col<InterpChain><<<grid, kThreads, 0, c.stream>>>(P, code, outer, red_n, inner, nsplit, partials);
  }
  if (e != cudaSuccess) return e;
  k_reduce_col_finish<<<(unsigned)(outer * ((inner + 31) / 32)), kThreads, 0, c.stream>>>(partials, code, init_bits, outer, nsplit, inner, P.out[0]);
  *c.launches += 2;
  return cudaGetLastError();
}


template <int CODE>
static cudaError_t launch_scan_with(const LaunchCtx& c, const void* src, void* dst, int64_t outer, int64_t n, int64_t inner) {
  if (outer * n * inner == 0) return cudaSuccess;
  const uint32_t* x = (const uint32_t*)src;
  uint32_t* y = (uint32_t*)dst;
  if (inner > 1 || n <= 32) {
    // (for very short contiguous rows a thread per row is as good as anything)
    const int64_t lines = outer * inner;
    const unsigned blocks = (unsigned)((lines + kThreads - 1) / kThreads);
    // fewer lines than half the threads the GPU holds, and long ones: cut them into segments (two launches)
    const int64_t want_threads = (int64_t)c.sm_count * 1024;
    int64_t nseg = std::min<int64_t>((want_threads + lines - 1) / lines, n / 64);
    nseg = std::min<int64_t>(nseg, 64);
    if (nseg >= 2 && (size_t)(nseg * lines) + 6 <= c.scratch_words) {
      const int64_t seg = ((n + nseg - 1) / nseg + 7) / 8 * 8;
      nseg = (n + seg - 1) / seg;
      dim3 grid(blocks, (unsigned)nseg);
      k_scan_lines_seg<CODE, false><<<grid, kThreads, 0, c.stream>>>(x, y, c.scratch, outer, n, inner, seg);
      k_scan_lines_seg<CODE, true><<<grid, kThreads, 0, c.stream>>>(x, y, c.scratch, outer, n, inner, seg);
      *c.launches += 2;
      return cudaGetLastError();
    }
    k_scan_lines<CODE><<<blocks, kThreads, 0, c.stream>>>(x, y, outer, n, inner);
    ++*c.launches;
    return cudaGetLastError();
  }
  if (outer > 65535) return cudaErrorInvalidValue;
  // enough CTAs to fill the GPU, at least four 1024-element chunks per segment
  int64_t want = std::max<int64_t>(1, (8 * (int64_t)c.sm_count + outer - 1) / outer);
  int64_t max_seg = std::max<int64_t>(1, n / 4096);
  int nseg = (int)std::min<int64_t>(std::min(want, max_seg), 4096);
  int64_t seg = ((n + nseg - 1) / nseg + 1023) / 1024 * 1024;
  nseg = (int)((n + seg - 1) / seg);
  if ((size_t)(outer * nseg) + 6 > c.scratch_words) return cudaErrorInvalidValue;  // the last six words belong to the stencil loop and the reductions
  uint32_t* partial = c.scratch;
  dim3 grid((unsigned)nseg, (unsigned)outer);
  if (nseg > 1) {
    k_scan_row_partials<CODE><<<grid, kThreads, 0, c.stream>>>(x, partial, n, seg, nseg);
    ++*c.launches;
  }
  k_scan_row_apply<CODE><<<grid, kThreads, 0, c.stream>>>(x, y, partial, n, seg, nseg);
  ++*c.launches;
  return cudaGetLastError();
}

cudaError_t launch_scan(const LaunchCtx& c, const void* src, void* dst, int code, int64_t outer, int64_t n, int64_t inner) {
  switch (code) {
    case R_FADD: return launch_scan_with<R_FADD>(c, src, dst, outer, n, inner);
    case R_FMAX: return launch_scan_with<R_FMAX>(c, src, dst, outer, n, inner);
    case R_FMIN: return launch_scan_with<R_FMIN>(c, src, dst, outer, n, inner);
    case R_FMUL: return launch_scan_with<R_FMUL>(c, src, dst, outer, n, inner);
    case R_IADD: return launch_scan_with<R_IADD>(c, src, dst, outer, n, inner);
    case R_IMAX: return launch_scan_with<R_IMAX>(c, src, dst, outer, n, inner);
    case R_IMIN: return launch_scan_with<R_IMIN>(c, src, dst, outer, n, inner);
    case R_IMUL: return launch_scan_with<R_IMUL>(c, src, dst, outer, n, inner);
    case R_OR: return launch_scan_with<R_OR>(c, src, dst, outer, n, inner);
    case R_AND: return launch_scan_with<R_AND>(c, src, dst, outer, n, inner);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_sum_partials(const LaunchCtx& c, const SumPartialsJob* jobs, int n_jobs) {
  if (n_jobs < 1 || n_jobs > 4) return cudaErrorInvalidValue;
  SumJobs all{};
  int64_t widest = 1;
  for (int q = 0; q < n_jobs; ++q) {
    all.j[q] = jobs[q];
    widest = std::max(widest, jobs[q].n);
  }
  dim3 grid((unsigned)((widest + 31) / 32), (unsigned)n_jobs);
  k_sum_partials<<<grid, kThreads, 0, c.stream>>>(all);
  ++*c.launches;
  return cudaGetLastError();
}

cudaError_t launch_logsumexp(const LaunchCtx& c, const float* x, int64_t row_stride, int64_t rows, int64_t cols, float* m, float* s, float* lse) {
  if (rows == 0) return cudaSuccess;
  bool vec = ((uintptr_t)x % 16 == 0) && (row_stride % 4 == 0);
  if (cols >= 2048) {
    if (vec) k_logsumexp<kThreads, true><<<(unsigned)rows, kThreads, 0, c.stream>>>(x, row_stride, rows, cols, m, s, lse);
    else k_logsumexp<kThreads, false><<<(unsigned)rows, kThreads, 0, c.stream>>>(x, row_stride, rows, cols, m, s, lse);
  } else {
    unsigned g = (unsigned)((rows + 7) / 8);
    if (vec) k_logsumexp<32, true><<<g, kThreads, 0, c.stream>>>(x, row_stride, rows, cols, m, s, lse);
    else k_logsumexp<32, false><<<g, kThreads, 0, c.stream>>>(x, row_stride, rows, cols, m, s, lse);
  }
  ++*c.launches;
  return cudaGetLastError();
}

}  // namespace rx
