// Device-side helpers shared by the kernels: element loads/stores, the
// fused-chain interpreter, and warp/block combine primitives.
#pragma once
#ifndef __CUDACC_RTC__
#include <cuda_runtime.h>
#include <stdint.h>
#endif

#include "rx_vm.h"

namespace rx {

// reduction kinds on raw 32-bit lanes
enum RedCode : int { R_FADD = 0, R_FMAX, R_FMIN, R_FMUL, R_IADD, R_IMAX, R_IMIN, R_IMUL, R_OR, R_AND };

__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }

// NaN-propagating maximum / minimum (stablehlo.maximum / minimum semantics) as the single hardware instruction.
// Written as PTX rather than as selects around fmaxf: nested select forms of min(min(x, c), x * c) crashed the
// run-time compiler's optimiser, and the instruction is what the selects should become anyway.
__device__ __forceinline__ float nan_max(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float nan_min(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// Signed 32-bit minimum / maximum, computed as an unsigned min / max of sign-biased values inside one asm block.
// With CUDA 12.9 for sm_100a, a signed integer min / max whose operand or result is negated came out wrong in
// three shapes (min(acc, x * -256), min(acc, min(-x, t)) in a reduction loop, -max(a, max(a, b))): the negation
// of one operand was lost, with the C++ min() / max() and with a plain min.s32 / max.s32 alike, so the fault is
// below PTX.  In the biased form no negation is ever an operand or a user of the min / max instruction.
__device__ __forceinline__ int32_t smin32(int32_t a, int32_t b) {
  int32_t r;
  asm("{ .reg .b32 x, y;\n\t"
      "xor.b32 x, %1, 0x80000000;\n\t"
      "xor.b32 y, %2, 0x80000000;\n\t"
      "min.u32 x, x, y;\n\t"
      "xor.b32 %0, x, 0x80000000; }"
      : "=r"(r)
      : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ int32_t smax32(int32_t a, int32_t b) {
  int32_t r;
  asm("{ .reg .b32 x, y;\n\t"
      "xor.b32 x, %1, 0x80000000;\n\t"
      "xor.b32 y, %2, 0x80000000;\n\t"
      "max.u32 x, x, y;\n\t"
      "xor.b32 %0, x, 0x80000000; }"
      : "=r"(r)
      : "r"(a), "r"(b));
  return r;
}

__device__ __forceinline__ uint32_t red_combine(int code, uint32_t a, uint32_t b) {
  switch (code) {
    case R_FADD: return f2u(u2f(a) + u2f(b));
    case R_FMAX: return f2u(nan_max(u2f(a), u2f(b)));
    case R_FMIN: return f2u(nan_min(u2f(a), u2f(b)));
    case R_FMUL: return f2u(u2f(a) * u2f(b));
    case R_IADD: return a + b;  // two's-complement wrap-around
    case R_IMAX: return (uint32_t)smax32((int32_t)a, (int32_t)b);
    case R_IMIN: return (uint32_t)smin32((int32_t)a, (int32_t)b);
    case R_IMUL: return a * b;
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

// f32 -> bf16, round to nearest even (cvt.rn), as a 16-bit pattern; two at once packed lo | hi << 16
__device__ __forceinline__ uint16_t bf16_bits(float x) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_bits(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float round_bf16(float x) { return __uint_as_float((uint32_t)bf16_bits(x) << 16); }

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
    case EL_BF16: ((uint16_t*)p)[i] = bf16_bits(u2f(v)); break;
    case EL_I32: ((uint32_t*)p)[i] = v; break;
    default: ((uint8_t*)p)[i] = v ? 1 : 0; break;
  }
}

// ---- bounds-checked build ---------------------------------------------------------------------------------
// With -DRX_BOUNDS=1 (build.py --bounds; the run-time compiler is given the same definition) every element access a
// chain kernel makes through an operand or result descriptor is checked against the extent of the buffer behind it.
// A miss is recorded once per execution in the device's status block -- {what, index low / high word, extent} -- and
// the access is skipped (loads give 0): nothing traps, the host reports the record at its next synchronising call.
// It stands in for compute-sanitizer's memcheck, which is not available where this engine is developed: an access
// that strays inside mapped memory changes no test result but does show up here.
#ifndef RX_BOUNDS
#define RX_BOUNDS 0
#endif
#if RX_BOUNDS
static __device__ __noinline__ void rx_bounds_miss(int* rec, int64_t extent, int64_t first, int what) {
  if (rec && atomicCAS(rec, 0, what) == 0) {
    rec[1] = (int)(first & 0xFFFFFFFFll);
    rec[2] = (int)(first >> 32);
    rec[3] = (int)(extent > 0x7FFFFFFF ? 0x7FFFFFFF : extent);
    __threadfence_system();
  }
}
__device__ __forceinline__ bool rx_in_bounds(int* rec, int64_t extent, int64_t first, int count, int what) {
  if (!rec || (first >= 0 && first + count <= extent)) return true;  // no record word: the descriptor was not bound for checking
  rx_bounds_miss(rec, extent, first, what);
  return false;
}
#define RX_LEAF_OK(l, first, count) rx_in_bounds((l).bounds, (l).extent, (first), (count), 100 + (l).reg)
#define RX_OUT_OK(o, first, count) rx_in_bounds((o).bounds, (o).extent, (first), (count), 200 + (o).reg)
#else
#define RX_LEAF_OK(l, first, count) true
#define RX_OUT_OK(o, first, count) true
#endif
// one element of an operand / result at element index i of its buffer
__device__ __forceinline__ uint32_t leaf_load(const VmLeaf& l, int64_t i) { return RX_LEAF_OK(l, i, 1) ? load_elem(l.ptr, i, l.elem) : 0u; }
__device__ __forceinline__ void out_store(const VmOut& o, int64_t i, uint32_t v) {
  if (RX_OUT_OK(o, i, 1)) store_elem(o.ptr, i, o.elem, v);
}


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
// Register-file rows are moved 128 bits at a time (the rows are 16-byte aligned local memory).
template <int V>
__device__ __forceinline__ void vm_ldrow(const uint32_t* src, uint32_t* dst) {
  if constexpr (V % 4 == 0) {
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const uint4 t = *reinterpret_cast<const uint4*>(src + 4 * q);
      dst[4 * q] = t.x; dst[4 * q + 1] = t.y; dst[4 * q + 2] = t.z; dst[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int v = 0; v < V; ++v) dst[v] = src[v];
  }
}
template <int V>
__device__ __forceinline__ void vm_strow(uint32_t* dst, const uint32_t* src) {
  if constexpr (V % 4 == 0) {
#pragma unroll
    for (int q = 0; q < V / 4; ++q) *reinterpret_cast<uint4*>(dst + 4 * q) = make_uint4(src[4 * q], src[4 * q + 1], src[4 * q + 2], src[4 * q + 3]);
  } else {
#pragma unroll
    for (int v = 0; v < V; ++v) dst[v] = src[v];
  }
}

template <int V>
__device__ __forceinline__ void vm_exec(const VmProgram& P, uint32_t (*R)[V], const int64_t* idx) {
  uint32_t acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0;
  for (int pc = 0; pc < P.n_instr; ++pc) {
    const VmInstr in = P.ins[pc];
    const uint32_t imm = in.imm;
    const float fimm = u2f(imm);
    const int cdir = in.c;
    (void)fimm; (void)cdir;
    // one dispatch per instruction; the lane loop lives inside each case
#define RX_UN(expr)                                  \
  {                                                  \
    _Pragma("unroll") for (int v = 0; v < V; ++v) {  \
      const uint32_t ua = acc[v];                    \
      const float a = u2f(ua);                       \
      const int32_t ia = (int32_t)ua;                \
      (void)a; (void)ia;                             \
      acc[v] = (expr);                               \
    }                                                \
  }                                                  \
  break
#define RX_BIN(expr)                                 \
  {                                                  \
    uint32_t B[V];                                   \
    vm_ldrow<V>(R[in.b], B);                         \
    _Pragma("unroll") for (int v = 0; v < V; ++v) {  \
      const uint32_t ua = acc[v], ub = B[v];         \
      const float a = u2f(ua), b = u2f(ub);          \
      const int32_t ia = (int32_t)ua, ib = (int32_t)ub; \
      (void)a; (void)b; (void)ia; (void)ib;          \
      acc[v] = (expr);                               \
    }                                                \
  }                                                  \
  break
    switch (in.op) {
      case VM_LD: vm_ldrow<V>(R[in.b], acc); break;
#define RX_X(op, expr) case op: RX_UN(expr);
      RX_VM_UNARY_OPS(RX_X)
#undef RX_X
#define RX_X(op, expr) case op: RX_BIN(expr);
      RX_VM_BINARY_OPS(RX_X)
#undef RX_X
      case VM_IOTA: {
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = (uint32_t)(int32_t)(idx[in.a] + (in.a == P.rank - 1 ? v : 0));
        break;
      }
      case VM_SELECT:
      case VM_MULADD:
      case VM_MULADD_C: {
        uint32_t B[V], C[V];
        vm_ldrow<V>(R[in.b], B);
        vm_ldrow<V>(R[in.c], C);
        if (in.op == VM_SELECT) {
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] = acc[v] ? B[v] : C[v];
        } else if (in.op == VM_MULADD) {
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] = f2u(__fadd_rn(__fmul_rn(u2f(acc[v]), u2f(B[v])), u2f(C[v])));
        } else {
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] = f2u(__fadd_rn(__fmul_rn(u2f(B[v]), u2f(C[v])), u2f(acc[v])));
        }
        break;
      }
      default: break;
    }
#undef RX_UN
#undef RX_BIN
    if (in.flags & VMF_STORE) vm_strow<V>(R[in.dst], acc);
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

// Programmatic dependent launch: wait until the kernel in front on the stream has completed and its writes are
// visible / allow the kernel behind to start.  No-ops in a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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
      if (++spins > ar.poll_limit) { failed = 1; break; }
      __nanosleep(kPeerPollNs);
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
