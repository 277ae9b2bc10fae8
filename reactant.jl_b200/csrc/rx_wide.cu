// Float64 on the device.  Reactant's own tests run mostly on Float64 arrays (test/core/map_reduction.jl:8-19); the
// engine's fast kernels are 32-bit.  A fusion group that touches an f64 value is lowered to the same bytecode with the
// `wide` flag set (rx_vm.h) and runs here: a 64-bit-register interpreter in which every floating-point op is the
// IEEE double operation (libdevice's double functions for the transcendental ones), integer and predicate ops keep
// the 32-bit semantics of the narrow interpreter in the low word, f32 / bf16 operands are widened on load and
// f32 results rounded once on store.  Kernels: map, the three reduce shapes (deterministic: fixed strided partials
// and fixed-order trees), scan along one dim, and a plain dot_general.  These are correctness paths -- one element
// per thread, generic indexing, no run-time specialisation -- for the f64 programs Reactant users run as a check,
// not for throughput.
#include "rx_kernels.h"

#include "rx_device.cuh"

namespace rx {

namespace {

constexpr int kWideThreads = 256;

__device__ __forceinline__ double u2d(uint64_t u) { return __longlong_as_double((long long)u); }
__device__ __forceinline__ uint64_t d2u(double d) { return (uint64_t)__double_as_longlong(d); }

__device__ __forceinline__ double nan_maxd(double a, double b) { return (a != a) ? a : (b != b) ? b : fmax(a, b); }
__device__ __forceinline__ double nan_mind(double a, double b) { return (a != a) ? a : (b != b) ? b : fmin(a, b); }

__device__ __forceinline__ uint32_t cmp_d(int dir, double a, double b) {
  switch (dir) {
    case CMP_EQ: return a == b;
    case CMP_NE: return a != b;
    case CMP_LT: return a < b;
    case CMP_LE: return a <= b;
    case CMP_GT: return a > b;
    default: return a >= b;
  }
}

// load one element of any storage kind into a 64-bit register: floats as the double of the same value
__device__ __forceinline__ uint64_t wide_load(const VmLeaf& l, int64_t i) {
  if (!RX_LEAF_OK(l, i, 1)) return 0;
  switch (l.elem) {
    case EL_F64: return (uint64_t)__ldg((const unsigned long long*)l.ptr + i);
    case EL_F32: return d2u((double)__uint_as_float(__ldg((const uint32_t*)l.ptr + i)));
    case EL_BF16: return d2u((double)__uint_as_float(((uint32_t)__ldg((const uint16_t*)l.ptr + i)) << 16));
    case EL_I32: return (uint64_t)__ldg((const uint32_t*)l.ptr + i);
    default: return __ldg((const uint8_t*)l.ptr + i) ? 1u : 0u;
  }
}
__device__ __forceinline__ void wide_store(const VmOut& o, int64_t i, uint64_t v) {
  if (!RX_OUT_OK(o, i, 1)) return;
  switch (o.elem) {
    case EL_F64: ((unsigned long long*)o.ptr)[i] = v; break;
    case EL_F32: ((float*)o.ptr)[i] = (float)u2d(v); break;   // one rounding: the conversion
    case EL_BF16: ((uint16_t*)o.ptr)[i] = bf16_bits((float)u2d(v)); break;
    case EL_I32: ((uint32_t*)o.ptr)[i] = (uint32_t)v; break;
    default: ((uint8_t*)o.ptr)[i] = v ? 1 : 0; break;
  }
}

// ops whose operands / results are floating point in the narrow machine: here they are doubles
__device__ __forceinline__ bool is_float_op(int op) {
  switch (op) {
    case VM_NEG: case VM_SIN: case VM_COS: case VM_EXP: case VM_LOG: case VM_TANH: case VM_SQRT: case VM_RSQRT: case VM_ABS: case VM_LOG1P:
    case VM_EXPM1: case VM_FLOOR: case VM_CEIL: case VM_SIGN: case VM_LOGISTIC: case VM_SQR: case VM_I2F: case VM_F2I: case VM_P2F: case VM_F2P:
    case VM_TAN: case VM_CBRT: case VM_RINT: case VM_ROUND: case VM_ISFINITE: case VM_ADD: case VM_SUB: case VM_RSUB: case VM_MUL: case VM_DIV:
    case VM_RDIV: case VM_MAX: case VM_MIN: case VM_POW: case VM_FCMP: case VM_ATAN2: case VM_REM: case VM_MULADD: case VM_MULADD_C:
      return true;
    default: return false;
  }
}

// The chain at one index.  R: the register file (leaf registers already loaded).
__device__ __forceinline__ void vm_exec64(const VmProgram& P, uint64_t* R, const int64_t* idx) {
  uint64_t acc = 0;
  for (int pc = 0; pc < P.n_instr; ++pc) {
    const VmInstr in = P.ins[pc];
    const int op = in.op;
    if (op == VM_LD) {
      acc = R[in.b];
    } else if (op == VM_CONST) {
      acc = in.c == 1 ? P.wconst[in.imm] : (uint64_t)in.imm;  // table entry (a double), or an integer / predicate
    } else if (op == VM_MOV) {
    } else if (op == VM_IOTA) {
      acc = (uint64_t)(uint32_t)(int32_t)idx[in.a];
    } else if (op == VM_SELECT) {
      acc = (uint32_t)acc ? R[in.b] : R[in.c];
    } else if (is_float_op(op)) {
      const double a = u2d(acc), b = u2d(R[in.b]);
      const int32_t ia = (int32_t)(uint32_t)acc;
      double r = 0.0;
      bool is_double = true;
      uint32_t w = 0;
      switch (op) {
        case VM_NEG: r = -a; break;
        case VM_SIN: r = sin(a); break;
        case VM_COS: r = cos(a); break;
        case VM_EXP: r = exp(a); break;
        case VM_LOG: r = log(a); break;
        case VM_TANH: r = tanh(a); break;
        case VM_SQRT: r = sqrt(a); break;
        case VM_RSQRT: r = 1.0 / sqrt(a); break;
        case VM_ABS: r = fabs(a); break;
        case VM_LOG1P: r = log1p(a); break;
        case VM_EXPM1: r = expm1(a); break;
        case VM_FLOOR: r = floor(a); break;
        case VM_CEIL: r = ceil(a); break;
        case VM_SIGN: r = (a != a) ? a : (double)((a > 0.0) - (a < 0.0)); break;
        case VM_LOGISTIC: r = 1.0 / (1.0 + exp(-a)); break;
        case VM_SQR: r = __dmul_rn(a, a); break;
        case VM_TAN: r = tan(a); break;
        case VM_CBRT: r = cbrt(a); break;
        case VM_RINT: r = rint(a); break;
        case VM_ROUND: r = round(a); break;
        case VM_I2F: r = (double)ia; break;
        case VM_P2F: r = (uint32_t)acc ? 1.0 : 0.0; break;
        case VM_F2I: is_double = false; w = (a != a) ? 0u : (a >= 2147483648.0 ? 0x7FFFFFFFu : (uint32_t)(int32_t)fmax(trunc(a), -2147483648.0)); break;
        case VM_F2P: is_double = false; w = (uint32_t)(a != 0.0); break;
        case VM_ISFINITE: is_double = false; w = (uint32_t)(fabs(a) <= 1.7976931348623157e308); break;
        case VM_ADD: r = __dadd_rn(a, b); break;
        case VM_SUB: r = __dsub_rn(a, b); break;
        case VM_RSUB: r = __dsub_rn(b, a); break;
        case VM_MUL: r = __dmul_rn(a, b); break;
        case VM_DIV: r = a / b; break;
        case VM_RDIV: r = b / a; break;
        case VM_MAX: r = nan_maxd(a, b); break;
        case VM_MIN: r = nan_mind(a, b); break;
        case VM_POW: r = pow(a, b); break;
        case VM_ATAN2: r = atan2(a, b); break;
        case VM_REM: r = fmod(a, b); break;
        case VM_FCMP: is_double = false; w = cmp_d(in.c, a, b); break;
        case VM_MULADD: r = __dadd_rn(__dmul_rn(a, b), u2d(R[in.c])); break;           // two roundings, as separate ops
        case VM_MULADD_C: r = __dadd_rn(__dmul_rn(b, u2d(R[in.c])), a); break;
        default: break;
      }
      acc = is_double ? d2u(r) : (uint64_t)w;
    } else {
      // integer and predicate ops: the narrow machine's semantics on the low words
      const uint32_t ua = (uint32_t)acc, ub = (uint32_t)R[in.b];
      const int32_t ia = (int32_t)ua, ib = (int32_t)ub;
      uint32_t w = 0;
      switch (op) {
        case VM_INEG: w = 0u - ua; break;
        case VM_IABS: w = ia < 0 ? 0u - ua : ua; break;
        case VM_NOT: w = ~ua; break;
        case VM_LNOT: w = ua ? 0u : 1u; break;
        case VM_I2P: w = (uint32_t)(ia != 0); break;
        case VM_IADD: w = ua + ub; break;
        case VM_ISUB: w = ua - ub; break;
        case VM_IMUL: w = ua * ub; break;
        case VM_IDIV: w = ib == 0 ? 0xFFFFFFFFu : ((ia == INT32_MIN && ib == -1) ? (uint32_t)INT32_MIN : (uint32_t)(ia / ib)); break;
        case VM_IMAX: w = (uint32_t)smax32(ia, ib); break;
        case VM_IMIN: w = (uint32_t)smin32(ia, ib); break;
        case VM_AND: w = ua & ub; break;
        case VM_OR: w = ua | ub; break;
        case VM_XOR: w = ua ^ ub; break;
        case VM_ICMP: w = vm_cmp_i(in.c, ia, ib); break;
        default: break;
      }
      acc = (uint64_t)w;
    }
    if (in.flags & VMF_STORE) R[in.dst] = acc;
  }
}

__device__ __forceinline__ uint64_t wide_eval_at(const VmProgram& P, const int64_t* idx) {
  uint64_t R[kVmMaxRegs];
  for (int k = 0; k < P.n_leaves; ++k) R[P.leaf[k].reg] = wide_load(P.leaf[k], leaf_offset(P.leaf[k], idx, P.rank));
  vm_exec64(P, R, idx);
  return R[P.result_reg];
}

// reductions: `f64` says whether the reduced values are doubles; otherwise the 32-bit combine of the narrow kernels
__device__ __forceinline__ uint64_t wide_identity(int code, bool f64) {
  if (!f64) return red_identity(code);
  switch (code) {
    case R_FADD: return d2u(0.0);
    case R_FMAX: return d2u(-INFINITY);
    case R_FMIN: return d2u(INFINITY);
    default: return d2u(1.0);
  }
}
__device__ __forceinline__ uint64_t wide_combine(int code, bool f64, uint64_t a, uint64_t b) {
  if (!f64) return red_combine(code, (uint32_t)a, (uint32_t)b);
  switch (code) {
    case R_FADD: return d2u(__dadd_rn(u2d(a), u2d(b)));
    case R_FMAX: return d2u(nan_maxd(u2d(a), u2d(b)));
    case R_FMIN: return d2u(nan_mind(u2d(a), u2d(b)));
    default: return d2u(__dmul_rn(u2d(a), u2d(b)));
  }
}
// block-wide combine in a fixed order (thread 0 ends with the result)
__device__ __forceinline__ uint64_t wide_block_red(int code, bool f64, uint64_t v, uint64_t* sm) {
  sm[threadIdx.x] = v;
  __syncthreads();
  for (int s = kWideThreads / 2; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) sm[threadIdx.x] = wide_combine(code, f64, sm[threadIdx.x], sm[threadIdx.x + s]);
    __syncthreads();
  }
  return sm[0];
}

__global__ void __launch_bounds__(kWideThreads) k_wide_map(const __grid_constant__ VmProgram P, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * kWideThreads;
  for (int64_t i = (int64_t)blockIdx.x * kWideThreads + threadIdx.x; i < n; i += stride) {
    int64_t idx[kMaxRank];
    unravel(P, i, idx);
    uint64_t R[kVmMaxRegs];
    for (int k = 0; k < P.n_leaves; ++k) R[P.leaf[k].reg] = wide_load(P.leaf[k], leaf_offset(P.leaf[k], idx, P.rank));
    vm_exec64(P, R, idx);
    for (int k = 0; k < P.n_outs; ++k) wide_store(P.out[k], out_offset(P.out[k], idx, P.rank), R[P.out[k].reg]);
  }
}

// whole space -> one value: every CTA folds a strided share of the elements (strided partials per thread, fixed tree),
// the CTA that finishes last folds the CTAs' values in index order.  The grid depends only on the element count and
// the device, so the order of combination, and with it the result, is the same from run to run.
__global__ void __launch_bounds__(kWideThreads) k_wide_reduce_full(const __grid_constant__ VmProgram P, int64_t n, int code, int f64, uint64_t init, uint64_t* partials,
                                                                   unsigned* ticket) {
  __shared__ uint64_t sm[kWideThreads];
  __shared__ int last_cta;
  uint64_t acc = wide_identity(code, f64);
  for (int64_t i = (int64_t)blockIdx.x * kWideThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kWideThreads) {
    int64_t idx[kMaxRank];
    unravel(P, i, idx);
    acc = wide_combine(code, f64, acc, wide_eval_at(P, idx));
  }
  acc = wide_block_red(code, f64, acc, sm);
  if (gridDim.x == 1) {
    if (threadIdx.x == 0) wide_store(P.out[0], P.out[0].offset, wide_combine(code, f64, init, acc));
    return;
  }
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = acc;
    __threadfence();
    last_cta = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last_cta) return;
  __threadfence();
  acc = wide_identity(code, f64);
  for (int j = threadIdx.x; j < (int)gridDim.x; j += kWideThreads) acc = wide_combine(code, f64, acc, __ldcg(partials + j));
  acc = wide_block_red(code, f64, acc, sm);
  if (threadIdx.x == 0) {
    wide_store(P.out[0], P.out[0].offset, wide_combine(code, f64, init, acc));
    *ticket = 0;  // for the next launch that counts finished CTAs in it
  }
}

// [outer][red]: one CTA per row
__global__ void __launch_bounds__(kWideThreads) k_wide_reduce_row(const __grid_constant__ VmProgram P, int64_t outer, int64_t red_n, int code, int f64, uint64_t init) {
  __shared__ uint64_t sm[kWideThreads];
  for (int64_t row = blockIdx.x; row < outer; row += gridDim.x) {
    int64_t idx[kMaxRank] = {row, 0, 0, 0};
    uint64_t acc = wide_identity(code, f64);
    for (int64_t r = threadIdx.x; r < red_n; r += kWideThreads) {
      idx[1] = r;
      acc = wide_combine(code, f64, acc, wide_eval_at(P, idx));
    }
    acc = wide_block_red(code, f64, acc, sm);
    if (threadIdx.x == 0) wide_store(P.out[0], P.out[0].offset + row * P.out[0].stride[0], wide_combine(code, f64, init, acc));
    __syncthreads();
  }
}

// [outer][red][inner]: one thread per (outer, inner), the reduced dim walked in order
__global__ void __launch_bounds__(kWideThreads) k_wide_reduce_col(const __grid_constant__ VmProgram P, int64_t outer, int64_t red_n, int64_t inner, int code, int f64,
                                                                  uint64_t init) {
  const int64_t total = outer * inner, stride = (int64_t)gridDim.x * kWideThreads;
  for (int64_t q = (int64_t)blockIdx.x * kWideThreads + threadIdx.x; q < total; q += stride) {
    const int64_t o = q / inner, b = q - o * inner;
    int64_t idx[kMaxRank] = {o, 0, b, 0};
    uint64_t acc = wide_identity(code, f64);
    for (int64_t r = 0; r < red_n; ++r) {
      idx[1] = r;
      acc = wide_combine(code, f64, acc, wide_eval_at(P, idx));
    }
    wide_store(P.out[0], P.out[0].offset + o * P.out[0].stride[0] + b * P.out[0].stride[2], wide_combine(code, f64, init, acc));
  }
}

// inclusive scan along the middle dim of a dense [outer][n][inner] array of doubles: one thread per line
__global__ void __launch_bounds__(kWideThreads) k_wide_scan(const double* __restrict__ src, double* __restrict__ dst, int code, int64_t outer, int64_t n, int64_t inner) {
  const int64_t total = outer * inner, stride = (int64_t)gridDim.x * kWideThreads;
  for (int64_t q = (int64_t)blockIdx.x * kWideThreads + threadIdx.x; q < total; q += stride) {
    const int64_t o = q / inner, b = q - o * inner;
    const double* s = src + o * n * inner + b;
    double* d = dst + o * n * inner + b;
    uint64_t acc = wide_identity(code, true);
    for (int64_t r = 0; r < n; ++r) {
      acc = wide_combine(code, true, acc, d2u(s[r * inner]));
      d[r * inner] = u2d(acc);
    }
  }
}

// D[m][n] = sum_k A(m,k) B(k,n) in doubles, one thread per element, k in order
__global__ void __launch_bounds__(kWideThreads) k_wide_gemm(const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ D, int64_t M, int64_t N, int64_t K,
                                                            int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t a_sb, int64_t b_sb, int64_t d_sb) {
  A += blockIdx.y * a_sb;
  B += blockIdx.y * b_sb;
  D += blockIdx.y * d_sb;
  const int64_t total = M * N, stride = (int64_t)gridDim.x * kWideThreads;
  for (int64_t q = (int64_t)blockIdx.x * kWideThreads + threadIdx.x; q < total; q += stride) {
    const int64_t mm = q / N, nn = q - mm * N;
    double acc = 0.0;
    for (int64_t k = 0; k < K; ++k) acc = fma(A[mm * a_sm + k * a_sk], B[k * b_sk + nn * b_sn], acc);
    D[q] = acc;
  }
}

int grid_for(const LaunchCtx& c, int64_t n) { return (int)std::max<int64_t>(1, std::min<int64_t>((n + kWideThreads - 1) / kWideThreads, (int64_t)c.sm_count * 8)); }

}  // namespace

cudaError_t launch_wide_map(const LaunchCtx& c, const VmProgram& P) {
  int64_t n = 1;
  for (int d = 0; d < P.rank; ++d) n *= P.dim[d];
  if (n == 0) return cudaSuccess;
  k_wide_map<<<grid_for(c, n), kWideThreads, 0, c.stream>>>(P, n);
  if (c.launches) ++*c.launches;
  return cudaGetLastError();
}

cudaError_t launch_wide_reduce(const LaunchCtx& c, const VmProgram& P, int shape, int code, bool f64, uint64_t init, int64_t outer, int64_t red_n, int64_t inner) {
  if (shape == 0) {
    int64_t n = 1;
    for (int d = 0; d < P.rank; ++d) n *= P.dim[d];
    // at least 8 elements per thread; the partials sit at the start of the device's scratch words, the ticket in the
    // last one (shared, in stream order, with the 32-bit reductions)
    int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((n + 8 * kWideThreads - 1) / (8 * kWideThreads), (int64_t)c.sm_count * 8));
    if ((size_t)blocks * 2 + 8 > c.scratch_words) blocks = 1;
    k_wide_reduce_full<<<blocks, kWideThreads, 0, c.stream>>>(P, n, code, f64 ? 1 : 0, init, (uint64_t*)c.scratch, (unsigned*)(c.scratch + c.scratch_words - 1));
  } else if (shape == 1) {
    if (outer == 0) return cudaSuccess;
    k_wide_reduce_row<<<(int)std::min<int64_t>(outer, (int64_t)c.sm_count * 8), kWideThreads, 0, c.stream>>>(P, outer, red_n, code, f64 ? 1 : 0, init);
  } else {
    if (outer * inner == 0) return cudaSuccess;
    k_wide_reduce_col<<<grid_for(c, outer * inner), kWideThreads, 0, c.stream>>>(P, outer, red_n, inner, code, f64 ? 1 : 0, init);
  }
  if (c.launches) ++*c.launches;
  return cudaGetLastError();
}

cudaError_t launch_wide_scan(const LaunchCtx& c, const void* src, void* dst, int code, int64_t outer, int64_t n, int64_t inner) {
  if (outer * inner * n == 0) return cudaSuccess;
  k_wide_scan<<<grid_for(c, outer * inner), kWideThreads, 0, c.stream>>>((const double*)src, (double*)dst, code, outer, n, inner);
  if (c.launches) ++*c.launches;
  return cudaGetLastError();
}

cudaError_t launch_wide_gemm(const LaunchCtx& c, const void* a, const void* b, void* d, int64_t M, int64_t N, int64_t K, int64_t batch, int64_t a_sm, int64_t a_sk, int64_t b_sk,
                             int64_t b_sn, int64_t a_sb, int64_t b_sb, int64_t d_sb) {
  if (M * N * batch == 0) return cudaSuccess;
  dim3 grid((unsigned)grid_for(c, M * N), (unsigned)batch);
  k_wide_gemm<<<grid, kWideThreads, 0, c.stream>>>((const double*)a, (const double*)b, (double*)d, M, N, K, a_sm, a_sk, b_sk, b_sn, a_sb, b_sb, d_sb);
  if (c.launches) ++*c.launches;
  return cudaGetLastError();
}

}  // namespace rx
