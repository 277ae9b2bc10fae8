// Device-side helpers shared by the kernels: element loads/stores, the
// fused-chain interpreter, and warp/block combine primitives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rx_vm.h"

namespace rx {

// reduction kinds on raw 32-bit lanes
enum RedCode : int { R_FADD = 0, R_FMAX, R_FMIN, R_FMUL, R_IADD, R_IMAX, R_IMIN, R_IMUL, R_OR, R_AND };

__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }

// StableHLO maximum/minimum propagate NaN.
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a) ? a : ((b != b) ? b : fmaxf(a, b)); }
__device__ __forceinline__ float nan_min(float a, float b) { return (a != a) ? a : ((b != b) ? b : fminf(a, b)); }

__device__ __forceinline__ uint32_t red_combine(int code, uint32_t a, uint32_t b) {
  switch (code) {
    case R_FADD: return f2u(u2f(a) + u2f(b));
    case R_FMAX: return f2u(nan_max(u2f(a), u2f(b)));
    case R_FMIN: return f2u(nan_min(u2f(a), u2f(b)));
    case R_FMUL: return f2u(u2f(a) * u2f(b));
    case R_IADD: return (uint32_t)((int32_t)a + (int32_t)b);
    case R_IMAX: return (uint32_t)max((int32_t)a, (int32_t)b);
    case R_IMIN: return (uint32_t)min((int32_t)a, (int32_t)b);
    case R_IMUL: return (uint32_t)((int32_t)a * (int32_t)b);
    case R_OR: return a | b;
    default: return a & b;
  }
}

__host__ __device__ __forceinline__ uint32_t red_identity(int code) {
  switch (code) {
    case R_FADD: return 0u;
    case R_FMAX: return 0xFF800000u;
    case R_FMIN: return 0x7F800000u;
    case R_FMUL: return 0x3F800000u;
    case R_IADD: return 0u;
    case R_IMAX: return 0x80000000u;
    case R_IMIN: return 0x7FFFFFFFu;
    case R_IMUL: return 1u;
    case R_OR: return 0u;
    default: return 0xFFFFFFFFu;
  }
}

__device__ __forceinline__ uint32_t load_elem(const void* p, int64_t i, int elem) {
  switch (elem) {
    case EL_F32: return __ldg((const uint32_t*)p + i);
    case EL_BF16: return ((uint32_t)__ldg((const uint16_t*)p + i)) << 16;
    case EL_I32: return __ldg((const uint32_t*)p + i);
    default: return __ldg((const uint8_t*)p + i) ? 1u : 0u;
  }
}

__device__ __forceinline__ void store_elem(void* p, int64_t i, int elem, uint32_t v) {
  switch (elem) {
    case EL_F32: ((uint32_t*)p)[i] = v; break;
    case EL_BF16: ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(u2f(v)); break;
    case EL_I32: ((uint32_t*)p)[i] = v; break;
    default: ((uint8_t*)p)[i] = v ? 1 : 0; break;
  }
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t vm_cmp_f(int dir, float a, float b) {
  switch (dir) {
    case CMP_EQ: return a == b;
    case CMP_NE: return a != b;
    case CMP_LT: return a < b;
    case CMP_LE: return a <= b;
    case CMP_GT: return a > b;
    default: return a >= b;
  }
}
__device__ __forceinline__ uint32_t vm_cmp_i(int dir, int32_t a, int32_t b) {
  switch (dir) {
    case CMP_EQ: return a == b;
    case CMP_NE: return a != b;
    case CMP_LT: return a < b;
    case CMP_LE: return a <= b;
    case CMP_GT: return a > b;
    default: return a >= b;
  }
}

// Evaluate the instruction list on V lanes.  R holds the registers; leaves have
// already been loaded into their registers.  `idx` is the root multi-index of
// lane 0 (only read by VM_IOTA, which the planner never vectorises).
template <int V>
__device__ __forceinline__ void vm_exec(const VmProgram& P, uint32_t (*R)[V], const int64_t* idx) {
  for (int pc = 0; pc < P.n_instr; ++pc) {
    const VmInstr in = P.ins[pc];
    const uint32_t* A = R[in.a];
    const uint32_t* B = R[in.b];
    const uint32_t* C = R[in.c];
    uint32_t out[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      float a = u2f(A[v]), b = u2f(B[v]);
      int32_t ia = (int32_t)A[v], ib = (int32_t)B[v];
      uint32_t r;
      switch (in.op) {
        case VM_CONST: r = in.imm; break;
        case VM_MOV: r = A[v]; break;
        case VM_NEG: r = f2u(-a); break;
        case VM_SIN: r = f2u(sinf(a)); break;
        case VM_COS: r = f2u(cosf(a)); break;
        case VM_EXP: r = f2u(expf(a)); break;
        case VM_LOG: r = f2u(logf(a)); break;
        case VM_TANH: r = f2u(tanhf(a)); break;
        case VM_SQRT: r = f2u(sqrtf(a)); break;
        case VM_RSQRT: r = f2u(1.0f / sqrtf(a)); break;
        case VM_ABS: r = f2u(fabsf(a)); break;
        case VM_LOG1P: r = f2u(log1pf(a)); break;
        case VM_EXPM1: r = f2u(expm1f(a)); break;
        case VM_FLOOR: r = f2u(floorf(a)); break;
        case VM_CEIL: r = f2u(ceilf(a)); break;
        case VM_SIGN: r = f2u((a != a) ? a : (float)((a > 0.f) - (a < 0.f))); break;
        case VM_LOGISTIC: r = f2u(1.0f / (1.0f + expf(-a))); break;
        case VM_RBF16: r = f2u(round_bf16(a)); break;
        case VM_ADD: r = f2u(a + b); break;
        case VM_SUB: r = f2u(a - b); break;
        case VM_MUL: r = f2u(a * b); break;
        case VM_DIV: r = f2u(a / b); break;
        case VM_MAX: r = f2u(nan_max(a, b)); break;
        case VM_MIN: r = f2u(nan_min(a, b)); break;
        case VM_POW: r = f2u(powf(a, b)); break;
        case VM_IADD: r = (uint32_t)(ia + ib); break;
        case VM_ISUB: r = (uint32_t)(ia - ib); break;
        case VM_IMUL: r = (uint32_t)(ia * ib); break;
        case VM_IDIV: r = ib == 0 ? 0xFFFFFFFFu : ((ia == INT32_MIN && ib == -1) ? (uint32_t)INT32_MIN : (uint32_t)(ia / ib)); break;
        case VM_IMAX: r = (uint32_t)max(ia, ib); break;
        case VM_IMIN: r = (uint32_t)min(ia, ib); break;
        case VM_INEG: r = (uint32_t)(-ia); break;
        case VM_IABS: r = (uint32_t)abs(ia); break;
        case VM_AND: r = A[v] & B[v]; break;
        case VM_OR: r = A[v] | B[v]; break;
        case VM_XOR: r = A[v] ^ B[v]; break;
        case VM_NOT: r = ~A[v]; break;
        case VM_LNOT: r = A[v] ? 0u : 1u; break;
        case VM_FCMP: r = vm_cmp_f(in.c, a, b); break;
        case VM_ICMP: r = vm_cmp_i(in.c, ia, ib); break;
        case VM_SELECT: r = A[v] ? B[v] : C[v]; break;
        case VM_I2F: r = f2u((float)ia); break;
        case VM_F2I: r = (a != a) ? 0u : (uint32_t)(int32_t)fminf(fmaxf(truncf(a), -2147483648.f), 2147483520.f); break;
        case VM_P2F: r = f2u(A[v] ? 1.f : 0.f); break;
        case VM_F2P: r = a != 0.f; break;
        case VM_I2P: r = ia != 0; break;
        case VM_IOTA: r = (uint32_t)(int32_t)(idx[in.a] + (in.a == P.rank - 1 ? v : 0)); break;
        default: r = 0; break;
      }
      out[v] = r;
    }
#pragma unroll
    for (int v = 0; v < V; ++v) R[in.dst][v] = out[v];
  }
}

// linear index -> multi-index over P.dim[0..rank)
__device__ __forceinline__ void unravel(const VmProgram& P, int64_t lin, int64_t* idx) {
#pragma unroll
  for (int d = kMaxRank - 1; d >= 0; --d) {
    if (d < P.rank) {
      int64_t q = lin / P.dim[d];
      idx[d] = lin - q * P.dim[d];
      lin = q;
    } else {
      idx[d] = 0;
    }
  }
}

// same for spaces of fewer than 2^31 points: 32-bit divisions
__device__ __forceinline__ void unravel32(const VmProgram& P, uint32_t lin, int64_t* idx) {
#pragma unroll
  for (int d = kMaxRank - 1; d >= 0; --d) {
    if (d < P.rank) {
      uint32_t dm = (uint32_t)P.dim[d];
      uint32_t q = lin / dm;
      idx[d] = lin - q * dm;
      lin = q;
    } else {
      idx[d] = 0;
    }
  }
}

__device__ __forceinline__ int64_t leaf_offset(const VmLeaf& l, const int64_t* idx, int rank) {
  int64_t o = l.offset;
#pragma unroll
  for (int d = 0; d < kMaxRank; ++d)
    if (d < rank) o += idx[d] * l.stride[d];
  return o;
}
__device__ __forceinline__ int64_t out_offset(const VmOut& l, const int64_t* idx, int rank) {
  int64_t o = l.offset;
#pragma unroll
  for (int d = 0; d < kMaxRank; ++d)
    if (d < rank) o += idx[d] * l.stride[d];
  return o;
}

// one element through the interpreter, leaves addressed by multi-index
__device__ __forceinline__ uint32_t vm_eval_at(const VmProgram& P, const int64_t* idx) {
  uint32_t R[kVmMaxRegs][1];
  for (int k = 0; k < P.n_leaves; ++k) R[P.leaf[k].reg][0] = load_elem(P.leaf[k].ptr, leaf_offset(P.leaf[k], idx, P.rank), P.leaf[k].elem);
  vm_exec<1>(P, R, idx);
  return R[P.result_reg][0];
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ uint32_t warp_red(int code, uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine(code, v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// Block-wide combine in a fixed order (warp shuffles, then one warp over the
// per-warp partials in shared memory): the result does not depend on timing.
template <int THREADS>
__device__ __forceinline__ uint32_t block_red(int code, uint32_t v, uint32_t* smem /* >= THREADS/32 words */) {
  v = warp_red(code, v);
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) smem[w] = v;
  __syncthreads();
  if (w == 0) {
    uint32_t x = lane < THREADS / 32 ? smem[lane] : red_identity(code);
    x = warp_red(code, x);
    if (lane == 0) smem[0] = x;
  }
  __syncthreads();
  return smem[0];
}

// All-reduce(sum) of one f32 across the mesh through peer mailboxes, executed by one
// warp (lane r talks to rank r).  Every rank stores {epoch, value} as a single 64-bit
// word into its slot of every peer's mailbox, then polls its own mailbox -- bounded --
// and adds the words in rank order, so all ranks return the same bits.  Returns false
// (and sets *status) if a peer's word did not arrive within the limit.
__device__ __forceinline__ bool mailbox_allreduce_warp(const FusedAllReduce& ar, float mine, float* result) {
  const int lane = threadIdx.x & 31;
  const unsigned long long word = ((unsigned long long)ar.epoch << 32) | (unsigned long long)__float_as_uint(mine);
  const int set = (ar.epoch & 1) * kMailRanks;
  if (lane < ar.n) {
    volatile unsigned long long* dst = ar.peer[lane] + set + ar.rank;
    *dst = word;
  }
  __threadfence_system();
  float got = 0.f;
  int failed = 0;
  if (lane < ar.n) {
    volatile unsigned long long* src = ar.peer[ar.rank] + set + lane;
    unsigned long long w = *src;
    long long spins = 0;
    while ((unsigned)(w >> 32) != ar.epoch) {
      if (++spins > 4000000) { failed = 1; break; }
      __nanosleep(100);
      w = *src;
    }
    got = __uint_as_float((unsigned)w);
  }
  failed = __any_sync(0xFFFFFFFFu, failed);
  float sum = 0.f;
  for (int r = 0; r < ar.n; ++r) sum += __shfl_sync(0xFFFFFFFFu, got, r);
  if (failed) {
    if (lane == 0) *ar.status = 1;
    return false;
  }
  *result = sum;
  return true;
}

}  // namespace rx
