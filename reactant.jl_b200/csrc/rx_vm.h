// Fused-elementwise micro-program: the planner compiles a chain of StableHLO
// elementwise ops (the body of a fusion group) into this register bytecode and
// every map / map-reduce / stencil / GEMM-epilogue kernel evaluates it per
// element.  Well-known chains are additionally recognised by `fast_id` and run
// through compile-time-fused functors instead of the interpreter.
//
// The op set mirrors the scalar emitters of Reactant (src/Ops.jl:398-460 unary,
// :536-589 binary, :1865-1961 select/compare/convert).
#pragma once
#ifdef __CUDACC_RTC__
// run-time compilation of specialised chains: no host headers are available
typedef unsigned char uint8_t;
typedef unsigned short uint16_t;
typedef unsigned int uint32_t;
typedef int int32_t;
typedef long long int64_t;
typedef unsigned long long uint64_t;
#define INT32_MIN (-2147483647 - 1)
#else
#include <stdint.h>
#endif

namespace rx {

enum VmOp : uint8_t {
  VM_NOP = 0,
  VM_CONST,   // dst = imm (raw 32 bits)
  VM_MOV,
  // f32 unary
  VM_NEG, VM_SIN, VM_COS, VM_EXP, VM_LOG, VM_TANH, VM_SQRT, VM_RSQRT, VM_ABS,
  VM_LOG1P, VM_EXPM1, VM_FLOOR, VM_CEIL, VM_SIGN, VM_LOGISTIC,
  VM_RBF16,   // round f32 to the nearest bf16 value (ties to even)
  // f32 binary
  VM_ADD, VM_SUB, VM_MUL, VM_DIV, VM_MAX, VM_MIN, VM_POW,
  // i32 arithmetic
  VM_IADD, VM_ISUB, VM_IMUL, VM_IDIV, VM_IMAX, VM_IMIN, VM_INEG, VM_IABS,
  VM_AND, VM_OR, VM_XOR, VM_NOT,   // bitwise on raw 32 bits
  VM_LNOT,                          // logical not on a 0/1 predicate
  // comparisons -> 0/1 ; `c` = direction
  VM_FCMP, VM_ICMP,
  VM_SELECT,  // dst = a ? b : c
  // conversions
  VM_I2F, VM_F2I, VM_P2F /* pred->f32 */, VM_F2P /* f32 != 0 */, VM_I2P,
  VM_IOTA,    // dst = index along root dim `a` (as i32)
  // f32 forms with an immediate operand (imm = raw bits) and the two-rounding multiply-add;
  // produced by the planner's peephole pass, never by the parser
  VM_ADDI, VM_SUBI /* a - imm */, VM_RSUBI /* imm - a */, VM_MULI, VM_DIVI /* a / imm */, VM_RDIVI /* imm / a */, VM_MAXI, VM_MINI,
  VM_MULADD,  // acc = round(round(acc * R[b]) + R[c]): same roundings as separate multiply and add
  VM_MULADD_C,  // acc = round(round(R[b] * R[c]) + acc)
  VM_LD,      // acc = R[b]
  VM_SQR,     // acc = acc * acc
  VM_RSUB,    // acc = R[b] - acc
  VM_RDIV,    // acc = R[b] / acc
  // more f32 ops (src/Ops.jl:398-460, 536-589 emitters for tan, cbrt, round, isfinite, atan, rem)
  VM_TAN, VM_CBRT, VM_RINT /* ties to even */, VM_ROUND /* ties away from zero */, VM_ISFINITE /* -> 0/1 */,
  VM_ATAN2, VM_REM,
  VM_NUM_OPS
};

// Scalar semantics of the ops, written once: the interpreter expands the tables into its
// switch, and the chain specialiser pastes the same expression text into generated code.
// Names available to an expression: ua / a / ia = the accumulator as raw bits / f32 / i32,
// ub / b / ib = the register operand, imm / fimm = the immediate as raw bits / f32,
// cdir = comparison direction.
#define RX_VM_UNARY_OPS(X)                                                                     \
  X(VM_CONST, imm)                                                                             \
  X(VM_MOV, ua)                                                                                \
  X(VM_NEG, f2u(-a))                                                                           \
  X(VM_SIN, f2u(sinf(a)))                                                                      \
  X(VM_COS, f2u(cosf(a)))                                                                      \
  X(VM_EXP, f2u(expf(a)))                                                                      \
  X(VM_LOG, f2u(logf(a)))                                                                      \
  X(VM_TANH, f2u(tanhf(a)))                                                                    \
  X(VM_SQRT, f2u(sqrtf(a)))                                                                    \
  X(VM_RSQRT, f2u(1.0f / sqrtf(a)))                                                            \
  X(VM_ABS, f2u(fabsf(a)))                                                                     \
  X(VM_LOG1P, f2u(log1pf(a)))                                                                  \
  X(VM_EXPM1, f2u(expm1f(a)))                                                                  \
  X(VM_FLOOR, f2u(floorf(a)))                                                                  \
  X(VM_CEIL, f2u(ceilf(a)))                                                                    \
  X(VM_SIGN, f2u((a != a) ? a : (float)((a > 0.f) - (a < 0.f))))                               \
  X(VM_LOGISTIC, f2u(1.0f / (1.0f + expf(-a))))                                                \
  X(VM_RBF16, f2u(round_bf16(a)))                                                              \
  X(VM_SQR, f2u(__fmul_rn(a, a)))                                                              \
  X(VM_ADDI, f2u(__fadd_rn(a, fimm)))                                                          \
  X(VM_SUBI, f2u(__fsub_rn(a, fimm)))                                                          \
  X(VM_RSUBI, f2u(__fsub_rn(fimm, a)))                                                         \
  X(VM_MULI, f2u(__fmul_rn(a, fimm)))                                                          \
  X(VM_DIVI, f2u(a / fimm))                                                                    \
  X(VM_RDIVI, f2u(fimm / a))                                                                   \
  X(VM_MAXI, f2u(nan_max(a, fimm)))                                                            \
  X(VM_MINI, f2u(nan_min(a, fimm)))                                                            \
  X(VM_INEG, 0u - ua)                                                                  \
  X(VM_IABS, ia < 0 ? 0u - ua : ua)                                                                \
  X(VM_NOT, ~ua)                                                                               \
  X(VM_LNOT, ua ? 0u : 1u)                                                                     \
  X(VM_I2F, f2u((float)ia))                                                                    \
  X(VM_F2I, (a != a) ? 0u : (a >= 2147483648.f ? 0x7FFFFFFFu : (uint32_t)(int32_t)fmaxf(truncf(a), -2147483648.f))) \
  X(VM_P2F, f2u(ua ? 1.f : 0.f))                                                               \
  X(VM_F2P, (uint32_t)(a != 0.f))                                                              \
  X(VM_I2P, (uint32_t)(ia != 0))                                                              \
  X(VM_TAN, f2u(tanf(a)))                                                                      \
  X(VM_CBRT, f2u(cbrtf(a)))                                                                    \
  X(VM_RINT, f2u(rintf(a)))                                                                    \
  X(VM_ROUND, f2u(roundf(a)))                                                                  \
  X(VM_ISFINITE, (uint32_t)(fabsf(a) <= 3.402823466e+38f))
#define RX_VM_BINARY_OPS(X)                                                                    \
  X(VM_ADD, f2u(__fadd_rn(a, b)))                                                              \
  X(VM_SUB, f2u(__fsub_rn(a, b)))                                                              \
  X(VM_RSUB, f2u(__fsub_rn(b, a)))                                                             \
  X(VM_MUL, f2u(__fmul_rn(a, b)))                                                              \
  X(VM_DIV, f2u(a / b))                                                                        \
  X(VM_RDIV, f2u(b / a))                                                                       \
  X(VM_MAX, f2u(nan_max(a, b)))                                                                \
  X(VM_MIN, f2u(nan_min(a, b)))                                                                \
  X(VM_POW, f2u(powf(a, b)))                                                                   \
  X(VM_IADD, ua + ub)                                                              \
  X(VM_ISUB, ua - ub)                                                              \
  X(VM_IMUL, ua * ub)                                                              \
  X(VM_IDIV, ib == 0 ? 0xFFFFFFFFu : ((ia == INT32_MIN && ib == -1) ? (uint32_t)INT32_MIN : (uint32_t)(ia / ib))) \
  X(VM_IMAX, (uint32_t)smax32(ia, ib))                                                         \
  X(VM_IMIN, (uint32_t)smin32(ia, ib))                                                         \
  X(VM_AND, ua & ub)                                                                           \
  X(VM_OR, ua | ub)                                                                            \
  X(VM_XOR, ua ^ ub)                                                                           \
  X(VM_FCMP, vm_cmp_f(cdir, a, b))                                                             \
  X(VM_ICMP, vm_cmp_i(cdir, ia, ib))                                                          \
  X(VM_ATAN2, f2u(atan2f(a, b)))                                                               \
  X(VM_REM, f2u(fmodf(a, b)))

enum VmCmp : uint8_t { CMP_EQ = 0, CMP_NE, CMP_LT, CMP_LE, CMP_GT, CMP_GE };

// storage element kinds a kernel can load/store
enum VmElem : uint8_t { EL_F32 = 0, EL_BF16, EL_I32, EL_PRED /* 1 byte */, EL_I64, EL_F64 };

// Accumulator machine: every instruction computes acc = f(acc, R[b], R[c] | imm), where acc
// (the previous instruction's result) lives in machine registers and R is the per-thread
// register file in local memory.  The result is copied to R[dst] only when VMF_STORE is set
// (it has a later, non-adjacent use or is an output).  For the chain-shaped programs that
// fusion produces, most instructions touch the register file once or not at all.
enum VmFlags : uint8_t { VMF_STORE = 8 };

struct VmInstr {
  uint8_t op, dst, a /* root dim for VM_IOTA */, b, c /* register, or comparison direction */, flags, pad[2];
  uint32_t imm;
};

constexpr int kVmMaxInstr = 48;
constexpr int kVmMaxRegs = 24;
constexpr int kVmMaxLeaves = 8;
constexpr int kVmMaxOuts = 4;
constexpr int kMaxRank = 4;
constexpr int kVmMaxWideConsts = 8;

// Known chains with compile-time-fused implementations.
enum FastId : int32_t {
  FAST_NONE = 0,
  FAST_SIN_ADD,        // sin(l0) + l1          (README sinsum_add)
  FAST_IDENTITY,       // l0
  FAST_EXP_SUB,        // exp(l0 - l1)
  FAST_STENCIL5_MUL,   // ((((l0+l1)+l2)+l3)+l4) * c   (Jacobi-2D)
};

struct VmLeaf {
  const void* ptr;
  int64_t offset;             // in elements
  int64_t stride[kMaxRank];   // in elements, per collapsed root dim
  uint8_t elem;               // VmElem
  uint8_t reg;                // destination register
  uint8_t linear;             // 1: contiguous in the root linear index; 2: scalar broadcast
  uint8_t pad[5];
  // Bounds-checked builds (RX_BOUNDS): elements in the buffer behind `ptr`, and where a miss is recorded.
  int64_t extent;
  int* bounds;
};

struct VmOut {
  void* ptr;
  int64_t offset;
  int64_t stride[kMaxRank];
  uint8_t elem;
  uint8_t reg;                // register holding the value
  uint8_t linear;
  uint8_t pad[5];
  int64_t extent;             // as in VmLeaf
  int* bounds;
};

struct VmProgram {
  int32_t n_instr, n_leaves, n_outs, fast_id;
  int32_t rank;               // collapsed root rank (<= kMaxRank)
  int32_t all_linear;         // every leaf/out is linear or scalar
  int64_t dim[kMaxRank];      // collapsed root dims, row-major
  float fast_c;               // constant of the fast chain, if any
  int32_t result_reg;         // register reduced / handed to an epilogue
  VmLeaf leaf[kVmMaxLeaves];
  VmOut out[kVmMaxOuts];
  VmInstr ins[kVmMaxInstr];
  // Wide programs: every floating-point value of the chain is an f64 (f32 / bf16 operands are widened when loaded,
  // f32 results rounded when stored), registers are 64 bits, integers and predicates keep their 32-bit semantics in
  // the low word.  Constants do not fit an instruction's 32-bit immediate: VM_CONST with c == 1 reads wconst[imm].
  // Such programs run on the interpreter kernels of rx_wide.cu only.
  int32_t wide;
  int32_t n_wconst;
  uint64_t wconst[kVmMaxWideConsts];
};

// Arguments of the NVLink mailbox all-reduce when it is fused into the tail of a
// full reduce (n == 0: no all-reduce).  peer[r] points at rank r's mailbox:
// 2 x kMailRanks 64-bit slots, indexed [epoch parity][sender rank].
constexpr int kMailRanks = 32;
constexpr unsigned kPeerPollNs = 200;  // sleep between two polls of a mailbox word (a poll costs about 0.25 us in all)
struct FusedAllReduce {
  unsigned long long* peer[kMailRanks];
  int rank, n;
  unsigned epoch;
  int* status;
  long long poll_limit;  // polls of a peer's word before the wait is given up (RxClient::peer_wait_polls)
};

}  // namespace rx
