// Kernel skeletons of the fused map / map-reduce families, templated on a chain policy C that
// says how the fused elementwise chain is evaluated:
//   * InterpChain (rx_kernels.cu, compiled ahead of time) runs the bytecode interpreter;
//   * a generated policy (rx_jit.cpp, compiled at run time for one chain) is straight-line code
//     with compile-time leaf kinds and register numbers, so the register file lives in machine
//     registers and the loops over leaves and outputs unroll.
// The skeletons themselves (access patterns, grid-stride loops, ordered cross-CTA combine) are the
// same for both.  This header must stay free of host includes: it is also compiled by NVRTC.
//
//  * k_map_*           elementwise chains (StableHLO elementwise ops after
//                       Reactant's enzyme-batch pass, src/TracedUtils.jl:1202-1352)
//  * k_reduce_full_*   chain -> stablehlo.reduce to a scalar (src/Ops.jl:3491-3622),
//                       deterministic two-pass combine across CTAs
//  * k_reduce_row/col  chain -> reduce along one axis
#pragma once
#include "rx_device.cuh"

#ifdef RX_CHAIN_SPECIALISED
#define RX_CHAIN_UNROLL _Pragma("unroll")
#else
#define RX_CHAIN_UNROLL
#endif

namespace rx {

constexpr int kThreads = 256;

// 128-bit row write into a register-file row
__device__ __forceinline__ void put4(uint32_t* d, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
#ifdef RX_CHAIN_SPECIALISED
  d[0] = x; d[1] = y; d[2] = z; d[3] = w;  // rows are machine registers
#else
  *(uint4*)d = make_uint4(x, y, z, w);
#endif
}

// Programmatic dependent launch.  A full reduce is launched with the "programmatic stream serialization"
// attribute, so its CTAs may start while the kernel in front of it on the stream is still running; everything it
// shares with that kernel (the partials scratch, the ticket, its output word, a mailbox) is touched only after
// `pdl_wait`, which returns once the kernel in front has completed and its writes are visible.  With `early`
// set by the host -- none of this launch's operands is written by the kernel in front -- the operand loads and
// the arithmetic come before the wait, so the main loop of this launch overlaps the cross-CTA combine and the
// drain of the previous one.  `pdl_release` lets the kernel behind this one start; it comes after this kernel's own
// wait, so at most two kernels of such a chain are ever in flight together.  Launched without the attribute
// both instructions do nothing.  (pdl_wait / pdl_release: rx_device.cuh)

// Second pass of the cross-CTA combine, run by whichever CTA finishes last: it adds
// the per-CTA partials in index order, so the result does not depend on which CTA
// that is.  `ticket` counts finished CTAs and is reset for the next launch.
__device__ __forceinline__ void finish_in_last_block(uint32_t mine, uint32_t* partials, unsigned* ticket, int code, uint32_t init_bits, const VmOut& out,
                                                     uint32_t* sm, const FusedAllReduce& ar) {
  __shared__ bool is_last;
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = mine;
    __threadfence();
    unsigned t = atomicAdd(ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  uint32_t acc = red_identity(code);
  for (int i = threadIdx.x; i < (int)gridDim.x; i += kThreads) acc = red_combine(code, acc, __ldcg(partials + i));
  // block_red<kThreads>, inlined here because this branch is taken by one whole CTA only
  acc = warp_red(code, acc);
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sm[w] = acc;
  __syncthreads();
  if (w == 0) {
    uint32_t x = lane < kThreads / 32 ? sm[lane] : red_identity(code);
    x = warp_red(code, x);
    x = red_combine(code, init_bits, x);
    if (ar.n > 1) {
      // sharded reduce: exchange this device's partial with the mesh before storing (f32 sum only)
      float total;
      if (!mailbox_allreduce_warp(ar, u2f(x), &total)) total = u2f(x);
      x = f2u(total);
    }
    if (lane == 0) {
      out_store(out, out.offset, x);
      *ticket = 0;
    }
  }
}

// ---- vector leaf access (4 consecutive elements, 4-element aligned) ----------
__device__ __forceinline__ void load4(const VmLeaf& l, int64_t i, uint32_t* d) {
  if (l.linear == 2) {
    uint32_t u = leaf_load(l, l.offset);
    put4(d, u, u, u, u);
    return;
  }
  if (!RX_LEAF_OK(l, l.offset + i, 4)) {
    put4(d, 0u, 0u, 0u, 0u);
    return;
  }
  switch (l.elem) {
    case EL_F32:
    case EL_I32: {
      uint4 t = __ldg((const uint4*)((const uint32_t*)l.ptr + l.offset + i));
      put4(d, t.x, t.y, t.z, t.w);
      break;
    }
    case EL_BF16: {
      uint2 v = __ldg((const uint2*)((const uint16_t*)l.ptr + l.offset + i));
      put4(d, v.x << 16, v.x & 0xFFFF0000u, v.y << 16, v.y & 0xFFFF0000u);
      break;
    }
    default: {
      uchar4 v = __ldg((const uchar4*)((const uint8_t*)l.ptr + l.offset + i));
      put4(d, v.x != 0, v.y != 0, v.z != 0, v.w != 0);
      break;
    }
  }
}

__device__ __forceinline__ void store4(const VmOut& o, int64_t i, const uint32_t* s) {
  if (!RX_OUT_OK(o, o.offset + i, 4)) return;
  switch (o.elem) {
    case EL_F32:
    case EL_I32:
      *(uint4*)((uint32_t*)o.ptr + o.offset + i) = make_uint4(s[0], s[1], s[2], s[3]);
      break;
    case EL_BF16: {
      uint2 v;
      v.x = bf16x2_bits(u2f(s[0]), u2f(s[1]));
      v.y = bf16x2_bits(u2f(s[2]), u2f(s[3]));
      *(uint2*)((uint16_t*)o.ptr + o.offset + i) = v;
      break;
    }
    default:
      *(uchar4*)((uint8_t*)o.ptr + o.offset + i) = make_uchar4(s[0] != 0, s[1] != 0, s[2] != 0, s[3] != 0);
      break;
  }
}

// one element through the chain, leaves addressed by multi-index
template <class C>
__device__ __forceinline__ uint32_t vm_eval_at(const VmProgram& P, const int64_t* idx) {
  __align__(16) uint32_t R[C::kRegs][1];
  RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) {
    const auto& l = C::leaf(P, k);
    R[C::leaf_reg(P, k)][0] = leaf_load(l, leaf_offset(l, idx, P.rank));
  }
  C::template exec<1>(P, R, idx);
  return R[C::result_reg(P)][0];
}

// ---- map ----------------------------------------------------------------------
template <class C>
__global__ void __launch_bounds__(kThreads) k_map_linear(const __grid_constant__ VmProgram P, int64_t n) {
  int64_t n4 = n >> 2;
  int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
    __align__(16) uint32_t R[C::kRegs][4];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) load4(C::leaf(P, k), i * 4, R[C::leaf_reg(P, k)]);
    C::template exec<4>(P, R, idx0);
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_outs(P); ++k) store4(C::out(P, k), i * 4, R[C::out_reg(P, k)]);
  }
  // tail
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t i = n4 * 4 + threadIdx.x;
    __align__(16) uint32_t R[C::kRegs][1];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k)
      R[C::leaf_reg(P, k)][0] = leaf_load(C::leaf(P, k), C::leaf(P, k).offset + (C::leaf(P, k).linear == 2 ? 0 : i));
    C::template exec<1>(P, R, idx0);
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_outs(P); ++k) out_store(C::out(P, k), C::out(P, k).offset + i, R[C::out_reg(P, k)][0]);
  }
}

template <class C, bool SMALL>
__global__ void __launch_bounds__(kThreads) k_map_generic(const __grid_constant__ VmProgram P, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t idx[kMaxRank];
    if (SMALL) unravel32(P, (uint32_t)i, idx);
    else unravel(P, i, idx);
    __align__(16) uint32_t R[C::kRegs][1];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) R[C::leaf_reg(P, k)][0] = leaf_load(C::leaf(P, k), leaf_offset(C::leaf(P, k), idx, P.rank));
    C::template exec<1>(P, R, idx);
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_outs(P); ++k) out_store(C::out(P, k), out_offset(C::out(P, k), idx, P.rank), R[C::out_reg(P, k)][0]);
  }
}

// Any strides, no alignment: the space is [rows][inner] (rows = all dims but the last, flattened), and a thread takes
// V elements of one row that lie W apart, W lanes side by side on the row (W: a power of two between 32 and 256
// picked by the launcher from the row length; a CTA covers 256 / W rows' chunks at once).  The index arithmetic --
// unravelling the row, one offset per operand -- is done once per V elements, a warp's accesses stay consecutive
// whatever the operands' offsets (shifted windows of one array are never 16-byte aligned all at once), and V
// independent chains and V loads per operand are in flight (V = 4, or 8 for chains with few registers).  Not for
// programs that read the index (iota): element v is not at inner + v.
template <class C, int V>
__global__ void __launch_bounds__(kThreads) k_map_runs(const __grid_constant__ VmProgram P, int64_t rows, int64_t inner, int log2w, int64_t chunks_per_row) {
  const int W = 1 << log2w, rank = C::rank(P), last = rank - 1;
  const int sub = (int)threadIdx.x >> log2w, lane = (int)threadIdx.x & (W - 1), per_cta = kThreads >> log2w;
  const int64_t total = rows * chunks_per_row;
  const bool small = total < ((int64_t)1 << 31) && rows < ((int64_t)1 << 31);
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  for (int64_t g = (int64_t)blockIdx.x * per_cta + sub; g < total; g += (int64_t)gridDim.x * per_cta) {
    int64_t row, cc;
    if (small) { const uint32_t r = (uint32_t)g / (uint32_t)chunks_per_row; row = r; cc = (uint32_t)g - r * (uint32_t)chunks_per_row; }
    else { row = g / chunks_per_row; cc = g - row * chunks_per_row; }
    const int64_t col = cc * (V * W) + lane;
    int64_t idx[kMaxRank] = {0, 0, 0, 0};
    {
      int64_t lin = row;
#pragma unroll
      for (int d = kMaxRank - 2; d >= 0; --d) {
        if (d < last) {
          if (small) { const uint32_t dm = (uint32_t)C::dim(P, d), q = (uint32_t)lin / dm; idx[d] = (uint32_t)lin - q * dm; lin = q; }
          else { const int64_t q = lin / C::dim(P, d); idx[d] = lin - q * C::dim(P, d); lin = q; }
        }
      }
    }
#pragma unroll
    for (int d = 0; d < kMaxRank; ++d)
      if (d == last) idx[d] = col;
    // what is left of the row from this thread's first element on, and the steps between a thread's elements, as
    // 32-bit numbers (the launcher checks that V steps fit): per element only one widening add is left
    const int rem = (int)min(inner - col, (int64_t)0x7FFFFFFF);
    __align__(16) uint32_t R[C::kRegs][V];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) {
      const VmLeaf l = C::leaf(P, k);
      const int64_t off = leaf_offset(l, idx, rank);
      int st = 0;
#pragma unroll
      for (int d = 0; d < kMaxRank; ++d)
        if (d == last) st = (int)l.stride[d] * W;
#pragma unroll
      for (int v = 0; v < V; ++v) R[C::leaf_reg(P, k)][v] = v * W < rem ? leaf_load(l, off + v * st) : 0u;
    }
    C::template exec<V>(P, R, idx0);
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_outs(P); ++k) {
      const VmOut o = C::out(P, k);
      const int64_t off = out_offset(o, idx, rank);
      int st = 0;
#pragma unroll
      for (int d = 0; d < kMaxRank; ++d)
        if (d == last) st = (int)o.stride[d] * W;
#pragma unroll
      for (int v = 0; v < V; ++v)
        if (v * W < rem) out_store(o, off + v * st, R[C::out_reg(P, k)][v]);
    }
  }
}

// ---- 2-D "row-vector" access: 4 consecutive elements of the innermost dim, operands either
// contiguous along it (stride 1) or broadcast along it (stride 0); any stride along the row dim.
__device__ __forceinline__ void load4_rowvec(const VmLeaf& l, int64_t row, int64_t col, int drow, int dcol, uint32_t* d) {
  int64_t off = l.offset + row * l.stride[drow];
  if (l.stride[dcol] == 0) {
    uint32_t u = leaf_load(l, off);
    put4(d, u, u, u, u);
    return;
  }
  off += col;
  if (!RX_LEAF_OK(l, off, 4)) {
    put4(d, 0u, 0u, 0u, 0u);
    return;
  }
  switch (l.elem) {
    case EL_F32:
    case EL_I32: {
      uint4 t = __ldg((const uint4*)((const uint32_t*)l.ptr + off));
      put4(d, t.x, t.y, t.z, t.w);
      break;
    }
    case EL_BF16: {
      uint2 v = __ldg((const uint2*)((const uint16_t*)l.ptr + off));
      put4(d, v.x << 16, v.x & 0xFFFF0000u, v.y << 16, v.y & 0xFFFF0000u);
      break;
    }
    default: {
      uchar4 v = __ldg((const uchar4*)((const uint8_t*)l.ptr + off));
      put4(d, v.x != 0, v.y != 0, v.z != 0, v.w != 0);
      break;
    }
  }
}

__device__ __forceinline__ void store4_rowvec(const VmOut& o, int64_t row, int64_t col, int drow, const uint32_t* s) {
  VmOut t = o;
  t.offset = o.offset + row * o.stride[drow] + col;
  store4(t, 0, s);
}

// map over [rows][cols], 4*U columns per thread (U = 2 halves the interpreter's per-lane dispatch cost)
template <class C, int U>
__global__ void __launch_bounds__(kThreads) k_map_rows(const __grid_constant__ VmProgram P, int64_t rows, int64_t cols) {
  constexpr int V = 4 * U;
  const int64_t cv = cols / V, total = rows * cv;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    int64_t row, col;
    if (total < ((int64_t)1 << 31)) { uint32_t r = (uint32_t)i / (uint32_t)cv; row = r; col = (int64_t)((uint32_t)i - r * (uint32_t)cv) * V; }
    else { row = i / cv; col = (i - row * cv) * V; }
    __align__(16) uint32_t R[C::kRegs][V];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k)
#pragma unroll
      for (int u = 0; u < U; ++u) load4_rowvec(C::leaf(P, k), row, col + 4 * u, 0, 1, R[C::leaf_reg(P, k)] + 4 * u);
    C::template exec<V>(P, R, idx0);
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_outs(P); ++k)
#pragma unroll
      for (int u = 0; u < U; ++u) store4_rowvec(C::out(P, k), row, col + 4 * u, 0, R[C::out_reg(P, k)] + 4 * u);
  }
}

// full reduce over [rows][cols], 4 columns per thread
template <class C>
__global__ void __launch_bounds__(kThreads) k_reduce_full_rows(const __grid_constant__ VmProgram P, int64_t rows, int64_t cols, int code_arg, uint32_t* __restrict__ partials,
                                                               unsigned* ticket, uint32_t init_bits, const __grid_constant__ FusedAllReduce ar, int early) {
  const int code = C::red_code(code_arg);
  if (!early) {
    pdl_wait();
    pdl_release();
  }
  __shared__ uint32_t sm[kThreads / 32];
  const int64_t c4 = cols >> 2, total = rows * c4;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  uint32_t acc[4];
  for (int v = 0; v < 4; ++v) acc[v] = red_identity(code);
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    int64_t row, col;
    if (total < ((int64_t)1 << 31)) { uint32_t r = (uint32_t)i / (uint32_t)c4; row = r; col = ((uint32_t)i - r * (uint32_t)c4) * 4; }
    else { row = i / c4; col = (i - row * c4) * 4; }
    __align__(16) uint32_t R[C::kRegs][4];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) load4_rowvec(C::leaf(P, k), row, col, 0, 1, R[C::leaf_reg(P, k)]);
    C::template exec<4>(P, R, idx0);
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = red_combine(code, acc[v], R[C::result_reg(P)][v]);
  }
  uint32_t v = red_combine(code, red_combine(code, acc[0], acc[1]), red_combine(code, acc[2], acc[3]));
  v = block_red<kThreads>(code, v, sm);
  if (early) {
    pdl_wait();
    pdl_release();
  }
  finish_in_last_block(v, partials, ticket, code, init_bits, C::out(P, 0), sm, ar);
}

// column reduce over [red][inner] (outer == 1): each thread owns 4 adjacent columns and a slice of rows
template <class C>
__global__ void __launch_bounds__(kThreads) k_reduce_col_vec(const __grid_constant__ VmProgram P, int code_arg, int64_t red_n, int64_t inner, int nsplit,
                                                             uint32_t* __restrict__ partials) {
  const int code = C::red_code(code_arg);
  const int64_t b4 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * 4;
  if (b4 >= inner) return;
  const int split = blockIdx.y;
  const int64_t chunk = (red_n + nsplit - 1) / nsplit;
  const int64_t r0 = split * chunk, r1 = min(red_n, r0 + chunk);
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  uint32_t acc[4];
  for (int v = 0; v < 4; ++v) acc[v] = red_identity(code);
  for (int64_t r = r0; r < r1; ++r) {
    __align__(16) uint32_t R[C::kRegs][4];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) load4_rowvec(C::leaf(P, k), r, b4, 1, 2, R[C::leaf_reg(P, k)]);
    C::template exec<4>(P, R, idx0);
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = red_combine(code, acc[v], R[C::result_reg(P)][v]);
  }
  *(uint4*)(partials + (int64_t)split * inner + b4) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
}

// Generic chain, all operands contiguous: interpreter on 4 lanes.
template <class C>
__global__ void __launch_bounds__(kThreads) k_reduce_full_linear(const __grid_constant__ VmProgram P, int64_t n, int code_arg, uint32_t* __restrict__ partials,
                                                                 unsigned* ticket, uint32_t init_bits, const __grid_constant__ FusedAllReduce ar, int early) {
  const int code = C::red_code(code_arg);
  if (!early) {
    pdl_wait();
    pdl_release();
  }
  __shared__ uint32_t sm[kThreads / 32];
  int64_t n4 = n >> 2;
  int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  uint32_t acc[4];
  for (int v = 0; v < 4; ++v) acc[v] = red_identity(code);
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
    __align__(16) uint32_t R[C::kRegs][4];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k) load4(C::leaf(P, k), i * 4, R[C::leaf_reg(P, k)]);
    C::template exec<4>(P, R, idx0);
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = red_combine(code, acc[v], R[C::result_reg(P)][v]);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t i = n4 * 4 + threadIdx.x;
    __align__(16) uint32_t R[C::kRegs][1];
    RX_CHAIN_UNROLL for (int k = 0; k < C::n_leaves(P); ++k)
      R[C::leaf_reg(P, k)][0] = leaf_load(C::leaf(P, k), C::leaf(P, k).offset + (C::leaf(P, k).linear == 2 ? 0 : i));
    C::template exec<1>(P, R, idx0);
    acc[0] = red_combine(code, acc[0], R[C::result_reg(P)][0]);
  }
  uint32_t v = red_combine(code, red_combine(code, acc[0], acc[1]), red_combine(code, acc[2], acc[3]));
  v = block_red<kThreads>(code, v, sm);
  if (early) {
    pdl_wait();
    pdl_release();
  }
  finish_in_last_block(v, partials, ticket, code, init_bits, C::out(P, 0), sm, ar);
}

// Generic chain, strided operands.
template <class C>
__global__ void __launch_bounds__(kThreads) k_reduce_full_generic(const __grid_constant__ VmProgram P, int64_t n, int code_arg, uint32_t* __restrict__ partials,
                                                                  unsigned* ticket, uint32_t init_bits, const __grid_constant__ FusedAllReduce ar, int early) {
  const int code = C::red_code(code_arg);
  if (!early) {
    pdl_wait();
    pdl_release();
  }
  __shared__ uint32_t sm[kThreads / 32];
  int64_t stride = (int64_t)gridDim.x * kThreads;
  uint32_t acc = red_identity(code);
  const bool small = n < ((int64_t)1 << 31);
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t idx[kMaxRank];
    if (small) unravel32(P, (uint32_t)i, idx);
    else unravel(P, i, idx);
    acc = red_combine(code, acc, vm_eval_at<C>(P, idx));
  }
  acc = block_red<kThreads>(code, acc, sm);
  if (early) {
    pdl_wait();
    pdl_release();
  }
  finish_in_last_block(acc, partials, ticket, code, init_bits, C::out(P, 0), sm, ar);
}

// ---- reduce along one axis: [outer][red] with TPR threads per row --------------------
template <class C, int TPR>
__global__ void __launch_bounds__(kThreads) k_reduce_row(const __grid_constant__ VmProgram P, int code_arg, uint32_t init_bits, int64_t outer, int64_t red_n) {
  const int code = C::red_code(code_arg);
  __shared__ uint32_t sm[kThreads / 32];
  constexpr int RPB = kThreads / TPR;
  int64_t row = (int64_t)blockIdx.x * RPB + threadIdx.x / TPR;
  int lane = threadIdx.x % TPR;
  uint32_t acc = red_identity(code);
  if (row < outer) {
    int64_t idx[kMaxRank] = {row, 0, 0, 0};
    for (int64_t r = lane; r < red_n; r += TPR) {
      idx[1] = r;
      acc = red_combine(code, acc, vm_eval_at<C>(P, idx));
    }
  }
  if (TPR == kThreads) acc = block_red<kThreads>(code, acc, sm);
  else if (TPR == 32) acc = warp_red(code, acc);
  if (lane == 0 && row < outer) out_store(C::out(P, 0), C::out(P, 0).offset + row * C::out(P, 0).stride[0], red_combine(code, init_bits, acc));
}

// ---- reduce along a strided axis: [outer][red][inner], threads along inner -----------
template <class C>
__global__ void __launch_bounds__(kThreads) k_reduce_col(const __grid_constant__ VmProgram P, int code_arg, int64_t outer, int64_t red_n, int64_t inner, int nsplit, uint32_t* __restrict__ partials) {
  const int code = C::red_code(code_arg);
  int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (b >= inner) return;
  int split = blockIdx.y;
  int64_t chunk = (red_n + nsplit - 1) / nsplit;
  int64_t r0 = split * chunk, r1 = min(red_n, r0 + chunk);
  for (int64_t o = blockIdx.z; o < outer; o += gridDim.z) {
    int64_t idx[kMaxRank] = {o, 0, b, 0};
    uint32_t acc = red_identity(code);
    for (int64_t r = r0; r < r1; ++r) {
      idx[1] = r;
      acc = red_combine(code, acc, vm_eval_at<C>(P, idx));
    }
    partials[(o * nsplit + split) * inner + b] = acc;
  }
}


}  // namespace rx
