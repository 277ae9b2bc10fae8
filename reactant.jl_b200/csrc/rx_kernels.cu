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
#include "rx_kernels.h"

#include <stdio.h>
#include <algorithm>

#include "rx_device.cuh"

namespace rx {

namespace {

constexpr int kThreads = 256;

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
      store_elem(out.ptr, out.offset, out.elem, x);
      *ticket = 0;
    }
  }
}

// ---- vector leaf access (4 consecutive elements, 4-element aligned) ----------
__device__ __forceinline__ void load4(const VmLeaf& l, int64_t i, uint32_t* d) {
  if (l.linear == 2) {
    uint32_t u = load_elem(l.ptr, l.offset, l.elem);
    *(uint4*)d = make_uint4(u, u, u, u);
    return;
  }
  switch (l.elem) {
    case EL_F32:
    case EL_I32: {
      *(uint4*)d = __ldg((const uint4*)((const uint32_t*)l.ptr + l.offset + i));
      break;
    }
    case EL_BF16: {
      uint2 v = __ldg((const uint2*)((const uint16_t*)l.ptr + l.offset + i));
      *(uint4*)d = make_uint4(v.x << 16, v.x & 0xFFFF0000u, v.y << 16, v.y & 0xFFFF0000u);
      break;
    }
    default: {
      uchar4 v = __ldg((const uchar4*)((const uint8_t*)l.ptr + l.offset + i));
      *(uint4*)d = make_uint4(v.x != 0, v.y != 0, v.z != 0, v.w != 0);
      break;
    }
  }
}

__device__ __forceinline__ void store4(const VmOut& o, int64_t i, const uint32_t* s) {
  switch (o.elem) {
    case EL_F32:
    case EL_I32:
      *(uint4*)((uint32_t*)o.ptr + o.offset + i) = make_uint4(s[0], s[1], s[2], s[3]);
      break;
    case EL_BF16: {
      __nv_bfloat162 a = __floats2bfloat162_rn(u2f(s[0]), u2f(s[1]));
      __nv_bfloat162 b = __floats2bfloat162_rn(u2f(s[2]), u2f(s[3]));
      uint2 v;
      v.x = *(uint32_t*)&a;
      v.y = *(uint32_t*)&b;
      *(uint2*)((uint16_t*)o.ptr + o.offset + i) = v;
      break;
    }
    default:
      *(uchar4*)((uint8_t*)o.ptr + o.offset + i) = make_uchar4(s[0] != 0, s[1] != 0, s[2] != 0, s[3] != 0);
      break;
  }
}

// ---- map ----------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) k_map_linear(const __grid_constant__ VmProgram P, int64_t n) {
  int64_t n4 = n >> 2;
  int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
    __align__(16) uint32_t R[kVmMaxRegs][4];
    for (int k = 0; k < P.n_leaves; ++k) load4(P.leaf[k], i * 4, R[P.leaf[k].reg]);
    vm_exec<4>(P, R, idx0);
    for (int k = 0; k < P.n_outs; ++k) store4(P.out[k], i * 4, R[P.out[k].reg]);
  }
  // tail
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t i = n4 * 4 + threadIdx.x;
    __align__(16) uint32_t R[kVmMaxRegs][1];
    for (int k = 0; k < P.n_leaves; ++k)
      R[P.leaf[k].reg][0] = load_elem(P.leaf[k].ptr, P.leaf[k].offset + (P.leaf[k].linear == 2 ? 0 : i), P.leaf[k].elem);
    vm_exec<1>(P, R, idx0);
    for (int k = 0; k < P.n_outs; ++k) store_elem(P.out[k].ptr, P.out[k].offset + i, P.out[k].elem, R[P.out[k].reg][0]);
  }
}

template <bool SMALL>
__global__ void __launch_bounds__(kThreads) k_map_generic(const __grid_constant__ VmProgram P, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t idx[kMaxRank];
    if (SMALL) unravel32(P, (uint32_t)i, idx);
    else unravel(P, i, idx);
    __align__(16) uint32_t R[kVmMaxRegs][1];
    for (int k = 0; k < P.n_leaves; ++k) R[P.leaf[k].reg][0] = load_elem(P.leaf[k].ptr, leaf_offset(P.leaf[k], idx, P.rank), P.leaf[k].elem);
    vm_exec<1>(P, R, idx);
    for (int k = 0; k < P.n_outs; ++k) store_elem(P.out[k].ptr, out_offset(P.out[k], idx, P.rank), P.out[k].elem, R[P.out[k].reg][0]);
  }
}


// ---- 2-D "row-vector" access: 4 consecutive elements of the innermost dim, operands either
// contiguous along it (stride 1) or broadcast along it (stride 0); any stride along the row dim.
__device__ __forceinline__ void load4_rowvec(const VmLeaf& l, int64_t row, int64_t col, int drow, int dcol, uint32_t* d) {
  int64_t off = l.offset + row * l.stride[drow];
  if (l.stride[dcol] == 0) {
    uint32_t u = load_elem(l.ptr, off, l.elem);
    *(uint4*)d = make_uint4(u, u, u, u);
    return;
  }
  off += col;
  switch (l.elem) {
    case EL_F32:
    case EL_I32: {
      *(uint4*)d = __ldg((const uint4*)((const uint32_t*)l.ptr + off));
      break;
    }
    case EL_BF16: {
      uint2 v = __ldg((const uint2*)((const uint16_t*)l.ptr + off));
      *(uint4*)d = make_uint4(v.x << 16, v.x & 0xFFFF0000u, v.y << 16, v.y & 0xFFFF0000u);
      break;
    }
    default: {
      uchar4 v = __ldg((const uchar4*)((const uint8_t*)l.ptr + off));
      *(uint4*)d = make_uint4(v.x != 0, v.y != 0, v.z != 0, v.w != 0);
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
template <int U>
__global__ void __launch_bounds__(kThreads) k_map_rows(const __grid_constant__ VmProgram P, int64_t rows, int64_t cols) {
  constexpr int V = 4 * U;
  const int64_t cv = cols / V, total = rows * cv;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    int64_t row, col;
    if (total < ((int64_t)1 << 31)) { uint32_t r = (uint32_t)i / (uint32_t)cv; row = r; col = (int64_t)((uint32_t)i - r * (uint32_t)cv) * V; }
    else { row = i / cv; col = (i - row * cv) * V; }
    __align__(16) uint32_t R[kVmMaxRegs][V];
    for (int k = 0; k < P.n_leaves; ++k)
#pragma unroll
      for (int u = 0; u < U; ++u) load4_rowvec(P.leaf[k], row, col + 4 * u, 0, 1, R[P.leaf[k].reg] + 4 * u);
    vm_exec<V>(P, R, idx0);
    for (int k = 0; k < P.n_outs; ++k)
#pragma unroll
      for (int u = 0; u < U; ++u) store4_rowvec(P.out[k], row, col + 4 * u, 0, R[P.out[k].reg] + 4 * u);
  }
}

// full reduce over [rows][cols], 4 columns per thread
__global__ void __launch_bounds__(kThreads) k_reduce_full_rows(const __grid_constant__ VmProgram P, int64_t rows, int64_t cols, int code, uint32_t* __restrict__ partials,
                                                               unsigned* ticket, uint32_t init_bits, const __grid_constant__ FusedAllReduce ar) {
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
    __align__(16) uint32_t R[kVmMaxRegs][4];
    for (int k = 0; k < P.n_leaves; ++k) load4_rowvec(P.leaf[k], row, col, 0, 1, R[P.leaf[k].reg]);
    vm_exec<4>(P, R, idx0);
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = red_combine(code, acc[v], R[P.result_reg][v]);
  }
  uint32_t v = red_combine(code, red_combine(code, acc[0], acc[1]), red_combine(code, acc[2], acc[3]));
  v = block_red<kThreads>(code, v, sm);
  finish_in_last_block(v, partials, ticket, code, init_bits, P.out[0], sm, ar);
}

// column reduce over [red][inner] (outer == 1): each thread owns 4 adjacent columns and a slice of rows
__global__ void __launch_bounds__(kThreads) k_reduce_col_vec(const __grid_constant__ VmProgram P, int code, int64_t red_n, int64_t inner, int nsplit,
                                                             uint32_t* __restrict__ partials) {
  const int64_t b4 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * 4;
  if (b4 >= inner) return;
  const int split = blockIdx.y;
  const int64_t chunk = (red_n + nsplit - 1) / nsplit;
  const int64_t r0 = split * chunk, r1 = min(red_n, r0 + chunk);
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  uint32_t acc[4];
  for (int v = 0; v < 4; ++v) acc[v] = red_identity(code);
  for (int64_t r = r0; r < r1; ++r) {
    __align__(16) uint32_t R[kVmMaxRegs][4];
    for (int k = 0; k < P.n_leaves; ++k) load4_rowvec(P.leaf[k], r, b4, 1, 2, R[P.leaf[k].reg]);
    vm_exec<4>(P, R, idx0);
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = red_combine(code, acc[v], R[P.result_reg][v]);
  }
  *(uint4*)(partials + (int64_t)split * inner + b4) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
}

// ---- full reduce: pass 1 ---------------------------------------------------------
// FAST_SIN_ADD: sum(sin(x) + y) with x = leaf 0, y = leaf 1, both contiguous f32.
__global__ void __launch_bounds__(kThreads) k_reduce_full_sinadd(const float* __restrict__ x, const float* __restrict__ y, int64_t n, uint32_t* __restrict__ partials,
                                                                 unsigned* ticket, uint32_t init_bits, VmOut out, const __grid_constant__ FusedAllReduce ar) {
  __shared__ uint32_t sm[kThreads / 32];
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
  finish_in_last_block(r, partials, ticket, R_FADD, init_bits, out, sm, ar);
}

// Generic chain, all operands contiguous: interpreter on 4 lanes.
__global__ void __launch_bounds__(kThreads) k_reduce_full_linear(const __grid_constant__ VmProgram P, int64_t n, int code, uint32_t* __restrict__ partials,
                                                                 unsigned* ticket, uint32_t init_bits, const __grid_constant__ FusedAllReduce ar) {
  __shared__ uint32_t sm[kThreads / 32];
  int64_t n4 = n >> 2;
  int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t idx0[kMaxRank] = {0, 0, 0, 0};
  uint32_t acc[4];
  for (int v = 0; v < 4; ++v) acc[v] = red_identity(code);
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
    __align__(16) uint32_t R[kVmMaxRegs][4];
    for (int k = 0; k < P.n_leaves; ++k) load4(P.leaf[k], i * 4, R[P.leaf[k].reg]);
    vm_exec<4>(P, R, idx0);
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = red_combine(code, acc[v], R[P.result_reg][v]);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t i = n4 * 4 + threadIdx.x;
    __align__(16) uint32_t R[kVmMaxRegs][1];
    for (int k = 0; k < P.n_leaves; ++k)
      R[P.leaf[k].reg][0] = load_elem(P.leaf[k].ptr, P.leaf[k].offset + (P.leaf[k].linear == 2 ? 0 : i), P.leaf[k].elem);
    vm_exec<1>(P, R, idx0);
    acc[0] = red_combine(code, acc[0], R[P.result_reg][0]);
  }
  uint32_t v = red_combine(code, red_combine(code, acc[0], acc[1]), red_combine(code, acc[2], acc[3]));
  v = block_red<kThreads>(code, v, sm);
  finish_in_last_block(v, partials, ticket, code, init_bits, P.out[0], sm, ar);
}

// Generic chain, strided operands.
__global__ void __launch_bounds__(kThreads) k_reduce_full_generic(const __grid_constant__ VmProgram P, int64_t n, int code, uint32_t* __restrict__ partials,
                                                                  unsigned* ticket, uint32_t init_bits, const __grid_constant__ FusedAllReduce ar) {
  __shared__ uint32_t sm[kThreads / 32];
  int64_t stride = (int64_t)gridDim.x * kThreads;
  uint32_t acc = red_identity(code);
  const bool small = n < ((int64_t)1 << 31);
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t idx[kMaxRank];
    if (small) unravel32(P, (uint32_t)i, idx);
    else unravel(P, i, idx);
    acc = red_combine(code, acc, vm_eval_at(P, idx));
  }
  acc = block_red<kThreads>(code, acc, sm);
  finish_in_last_block(acc, partials, ticket, code, init_bits, P.out[0], sm, ar);
}

// ---- reduce along one axis: [outer][red] with TPR threads per row --------------------
template <int TPR>
__global__ void __launch_bounds__(kThreads) k_reduce_row(const __grid_constant__ VmProgram P, int code, uint32_t init_bits, int64_t outer, int64_t red_n) {
  __shared__ uint32_t sm[kThreads / 32];
  constexpr int RPB = kThreads / TPR;
  int64_t row = (int64_t)blockIdx.x * RPB + threadIdx.x / TPR;
  int lane = threadIdx.x % TPR;
  uint32_t acc = red_identity(code);
  if (row < outer) {
    int64_t idx[kMaxRank] = {row, 0, 0, 0};
    for (int64_t r = lane; r < red_n; r += TPR) {
      idx[1] = r;
      acc = red_combine(code, acc, vm_eval_at(P, idx));
    }
  }
  if (TPR == kThreads) acc = block_red<kThreads>(code, acc, sm);
  else if (TPR == 32) acc = warp_red(code, acc);
  if (lane == 0 && row < outer) store_elem(P.out[0].ptr, P.out[0].offset + row * P.out[0].stride[0], P.out[0].elem, red_combine(code, init_bits, acc));
}

// ---- reduce along a strided axis: [outer][red][inner], threads along inner -----------
__global__ void __launch_bounds__(kThreads) k_reduce_col(const __grid_constant__ VmProgram P, int code, int64_t outer, int64_t red_n, int64_t inner, int nsplit, uint32_t* __restrict__ partials) {
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
      acc = red_combine(code, acc, vm_eval_at(P, idx));
    }
    partials[(o * nsplit + split) * inner + b] = acc;
  }
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
    store_elem(out.ptr, out.offset + o * out.stride[0] + b * out.stride[2], out.elem, red_combine(code, init_bits, t));
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
  bool f = dt == DT::F32 || dt == DT::BF16;
  switch (k) {
    case RedK::Add: return f ? R_FADD : R_IADD;
    case RedK::Max: return f ? R_FMAX : R_IMAX;
    case RedK::Min: return f ? R_FMIN : R_IMIN;
    case RedK::Mul: return f ? R_FMUL : R_IMUL;
    case RedK::Or: return R_OR;
    default: return R_AND;
  }
}

cudaError_t launch_map(const LaunchCtx& c, const VmProgram& P) {
  int64_t n = total_of(P);
  if (n == 0) return cudaSuccess;
  if (P.all_linear && vec_aligned(P)) {
    k_map_linear<<<grid_for((n + 3) / 4, c.sm_count, 8), kThreads, 0, c.stream>>>(P, n);
  } else if (P.rank == 2 && rowvec_ok(P, 0, 1, true)) {
    static const int per_sm = getenv("RX_MAP_CTAS") ? atoi(getenv("RX_MAP_CTAS")) : 8;
    static const int lanes = getenv("RX_MAP_LANES") ? atoi(getenv("RX_MAP_LANES")) : 8;
    if (P.dim[1] % 8 == 0 && lanes == 8) k_map_rows<2><<<grid_for(n / 8, c.sm_count, per_sm), kThreads, 0, c.stream>>>(P, P.dim[0], P.dim[1]);
    else k_map_rows<1><<<grid_for(n / 4, c.sm_count, per_sm), kThreads, 0, c.stream>>>(P, P.dim[0], P.dim[1]);
  } else {
    if (n < ((int64_t)1 << 31)) k_map_generic<true><<<grid_for(n, c.sm_count, 8), kThreads, 0, c.stream>>>(P, n);
    else k_map_generic<false><<<grid_for(n, c.sm_count, 8), kThreads, 0, c.stream>>>(P, n);
  }
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

cudaError_t launch_reduce_full(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, const FusedAllReduce* fused) {
  FusedAllReduce ar{};
  if (fused) ar = *fused;
  int64_t n = total_of(P);
  static const int occ_sinadd = resident_per_sm(k_reduce_full_sinadd), occ_linear = resident_per_sm(k_reduce_full_linear),
                   occ_rows = resident_per_sm(k_reduce_full_rows), occ_generic = resident_per_sm(k_reduce_full_generic);
  const bool vec0 = P.all_linear && vec_aligned(P);
  const int occ = (vec0 && P.fast_id == FAST_SIN_ADD && code == R_FADD) ? occ_sinadd : vec0 ? occ_linear : (P.rank == 2 && rowvec_ok(P, 0, 1, false)) ? occ_rows : occ_generic;
  // 16 elements per thread per trip keeps four 128-bit loads in flight per operand
  int blocks = grid_for((n + 15) / 16, c.sm_count, occ);
  if ((size_t)blocks + 1 > c.scratch_words) return cudaErrorInvalidValue;
  uint32_t* partials = c.scratch;
  unsigned* ticket = (unsigned*)(c.scratch + c.scratch_words - 1);  // zeroed at device creation, reset by each launch
  bool vec = P.all_linear && vec_aligned(P);
  if (vec && P.fast_id == FAST_SIN_ADD && code == R_FADD) {
    const float* x = (const float*)P.leaf[0].ptr + P.leaf[0].offset;
    const float* y = (const float*)P.leaf[1].ptr + P.leaf[1].offset;
    k_reduce_full_sinadd<<<blocks, kThreads, 0, c.stream>>>(x, y, n, partials, ticket, init_bits, P.out[0], ar);
  } else if (vec) {
    k_reduce_full_linear<<<blocks, kThreads, 0, c.stream>>>(P, n, code, partials, ticket, init_bits, ar);
  } else if (P.rank == 2 && rowvec_ok(P, 0, 1, false)) {
    k_reduce_full_rows<<<blocks, kThreads, 0, c.stream>>>(P, P.dim[0], P.dim[1], code, partials, ticket, init_bits, ar);
  } else {
    k_reduce_full_generic<<<blocks, kThreads, 0, c.stream>>>(P, n, code, partials, ticket, init_bits, ar);
  }
  *c.launches += 1;
  return cudaGetLastError();
}

cudaError_t launch_reduce_row(const LaunchCtx& c, const VmProgram& P, int code, uint32_t init_bits, int64_t outer, int64_t red_n) {
  if (outer == 0) return cudaSuccess;
  if (red_n >= 2048) {
    k_reduce_row<kThreads><<<(unsigned)outer, kThreads, 0, c.stream>>>(P, code, init_bits, outer, red_n);
  } else if (red_n >= 16) {
    k_reduce_row<32><<<(unsigned)((outer + 7) / 8), kThreads, 0, c.stream>>>(P, code, init_bits, outer, red_n);
  } else {
    k_reduce_row<1><<<(unsigned)((outer + kThreads - 1) / kThreads), kThreads, 0, c.stream>>>(P, code, init_bits, outer, red_n);
  }
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
  if (outer == 1 && rowvec_ok(P, 1, 2, false)) {
    dim3 grid((unsigned)((inner / 4 + kThreads - 1) / kThreads), (unsigned)nsplit, 1);
    k_reduce_col_vec<<<grid, kThreads, 0, c.stream>>>(P, code, red_n, inner, nsplit, partials);
  } else {
    dim3 grid((unsigned)((inner + kThreads - 1) / kThreads), (unsigned)nsplit, (unsigned)std::min<int64_t>(outer, 65535));
    k_reduce_col<<<grid, kThreads, 0, c.stream>>>(P, code, outer, red_n, inner, nsplit, partials);
  }
  k_reduce_col_finish<<<(unsigned)(outer * ((inner + 31) / 32)), kThreads, 0, c.stream>>>(partials, code, init_bits, outer, nsplit, inner, P.out[0]);
  *c.launches += 2;
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
