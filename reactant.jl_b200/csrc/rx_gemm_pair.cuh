// The two-CTA tcgen05 GEMM kernel (bf16 operands, fp32 accumulation in TMEM) as a template on its epilogue, in a
// header free of host includes: rx_gemm_tc.cu instantiates it ahead of time with the plain epilogue (round once,
// store), and the chain specialiser (rx_jit.cpp) compiles it at run time with an epilogue that evaluates a fused
// elementwise chain on the accumulator -- bias add, activation, casts, gradients of the loss -- writes several
// results, and accumulates column sums and full sums of chain values, so that the elementwise and reduction work
// that follows a stablehlo.dot_general (src/stdlibs/LinearAlgebra.jl:274-330 with NNlib activations,
// ext/ReactantNNlibExt/Implementations.jl:12-25, and what Enzyme's reverse pass adds around it) costs no pass over
// HBM of its own.
//
// A cluster of two CTAs (two SMs) computes one 256 x 256 tile with tcgen05.mma.cta_group::2 (M256 N256 K16).  Each
// CTA stages its own 128 rows of A and *half* of the B slab (128 of the 256 N rows), so per SM the shared-memory fill
// and the L2->SM traffic per FLOP drop by a third against a one-CTA kernel.  The leader CTA (cluster rank 0) issues
// every MMA; the TMA loads of both CTAs complete on the leader's `full` barrier (cta_group::2 loads, no
// multicast); tcgen05.commit with a two-CTA mask releases slabs / publishes accumulators in both CTAs; both CTAs'
// epilogue warps arrive on the leader's `acc_empty` barrier.  Each CTA's TMEM holds its 128 accumulator rows x 256
// columns, double buffered, so the epilogue of one tile runs under the MMAs of the next.
// Every mbarrier wait is bounded; a wait that runs out sets a status word, all roles drain, TMEM is released and
// the kernel returns.
#pragma once
#include "rx_device.cuh"
#include "rx_tma_device.cuh"

namespace rx {

constexpr int kGemmThreads = 192;
constexpr int kEpiWarps = 4;
constexpr long long kGemmWaitLimit = 4000000;
constexpr int UMMA_K = 16;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;        // 1: operand is MN-major in memory (contiguous along M resp. N)
  void* D;
  long long ldd;
  int out_bf16;
  int tiles_m, tiles_n;
  int* status;
  int tma_store;         // pair kernel, plain epilogue: through shared memory and tiled bulk stores
};

// ---- tcgen05 wrappers ------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
        "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
        "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (SWIZZLE_128B): start address, leading / stride
// byte offsets in 16-byte units, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}



// One plain epilogue step: 32 consecutive columns of row m, rounded once to the output type.
__device__ __forceinline__ void store_row32(const GemmParams& p, long long m, long long n, const uint32_t* v) {
  if (m >= p.M) return;
  if (p.out_bf16) {
    uint16_t* row = (uint16_t*)p.D + m * p.ldd + n;
    if (n + 32 <= p.N && (((unsigned long long)row & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = bf16x2_bits(u2f(v[8 * q + 0]), u2f(v[8 * q + 1]));
        o.y = bf16x2_bits(u2f(v[8 * q + 2]), u2f(v[8 * q + 3]));
        o.z = bf16x2_bits(u2f(v[8 * q + 4]), u2f(v[8 * q + 5]));
        o.w = bf16x2_bits(u2f(v[8 * q + 6]), u2f(v[8 * q + 7]));
        *(uint4*)(row + 8 * q) = o;
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (n + j < p.N) row[j] = bf16_bits(u2f(v[j]));
    }
  } else {
    float* row = (float*)p.D + m * p.ldd + n;
    if (n + 32 <= p.N && (((unsigned long long)row & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < 8; ++q) *(uint4*)(row + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
      for (int j = 0; j < 32; ++j)
        if (n + j < p.N) row[j] = u2f(v[j]);
    }
  }
}

// ---- epilogue policies -------------------------------------------------------------------------------------
// The plain epilogue: nothing but the store (the kernel's own code paths).
struct EpiPlain {
  static constexpr bool kPlain = true;
  static constexpr int kWarps = kEpiWarps;  // epilogue warps per CTA
  struct Params { int unused; };
  struct Tile {};
  static __device__ __forceinline__ void begin_tile(Tile&, unsigned char*) {}
  static __device__ __forceinline__ void piece(Tile&, const Params&, const GemmParams&, long long, long long, uint32_t*) {}
  static __device__ __forceinline__ void end_tile(Tile&, const Params&, int, bool) {}
};

// Fused epilogue.  `C` is a chain policy generated for one fused chain (the same kind rx_chain_kernels.cuh takes),
// extended with: kAccLeaf (which leaf of the program is the accumulator: it is not read from memory but taken
// from TMEM, rounded to the dot_general's result type first, exactly as if the product had been stored and read
// back), kNumCol / col_reg(q) (registers whose column sums over all rows are wanted) and kNumFull / full_reg(q)
// (registers summed over the whole matrix).  The program's root space is [M][N]; operands other than the
// accumulator are addressed as base + offset + m * stride[0] + n * stride[1] with stride[1] in {0, 1}; results
// are dense [M][N] arrays.
// Sums are deterministic: a column's partial over a block of 32 rows is formed by a fixed butterfly over the warp's
// lanes and written to col_partial[row block][column]; a full sum's partial per (tile, CTA, warp) is written to
// full_partial[(tile * 2 + cta) * kWarps + warp]; a small kernel adds the partials in index order afterwards.
struct alignas(64) EpiChainParams {
  // Results leave through shared memory: every epilogue warp owns a 4 KiB buffer in which it lays out its 32 x 32
  // block of each result (2 KiB for bf16, 4 KiB for f32, as many results as fit), and the copy engine writes the
  // block to global memory with one tiled bulk store per result -- whole 64- or 128-byte row pieces instead of 32
  // scattered 16-byte stores per instruction.  stage_off[k] is the byte offset of result k's block in the buffer,
  // or -1 for a result that is stored straight from registers.
  CUtensorMap tm_out[kVmMaxOuts];
  int stage_off[kVmMaxOuts];
  VmProgram P;
  float* col_partial[2];   // [M / 32][N]
  float* full_partial[2];  // [tiles * 2 * EpiChain::kWarps]
  int vec_ok;              // every operand and result allows aligned V-element accesses
};

template <class C>
struct EpiChain {
  static constexpr bool kPlain = false;
  // Eight epilogue warps, two per TMEM lane quadrant, each taking half of the tile's 256 columns: the chain's
  // arithmetic and the latency of its operand loads are spread over two warps per scheduler instead of one.
  static constexpr int kWarps = 8;
  using Params = EpiChainParams;
  static constexpr int V = 8;
  static constexpr int NF = C::kNumFull > 0 ? C::kNumFull : 1;
  static constexpr int NC = C::kNumCol > 0 ? C::kNumCol : 1;

  struct Tile {
    float full[NF];
    unsigned char* stage;
  };
  static __device__ __forceinline__ void begin_tile(Tile& ts, unsigned char* stage) {
    ts.stage = stage;
#pragma unroll
    for (int q = 0; q < NF; ++q) ts.full[q] = 0.f;
  }

  // V consecutive elements of operand l at (m, n): n is a multiple of V (V = 4 or 8)
  static __device__ __forceinline__ void load_v(const VmLeaf& l, long long m, long long n, bool vec, uint32_t* d) {
    const long long base = l.offset + m * l.stride[0];
    if (l.stride[1] == 0) {
      const uint32_t u = leaf_load(l, base);
#pragma unroll
      for (int j = 0; j < V; ++j) d[j] = u;
      return;
    }
    if (!RX_LEAF_OK(l, base + n, V)) {
#pragma unroll
      for (int j = 0; j < V; ++j) d[j] = 0u;
      return;
    }
    if (vec && l.elem == EL_F32) {
      const uint4* q = (const uint4*)((const uint32_t*)l.ptr + base + n);
#pragma unroll
      for (int h = 0; h < V / 4; ++h) {
        const uint4 a = __ldg(q + h);
        d[4 * h] = a.x; d[4 * h + 1] = a.y; d[4 * h + 2] = a.z; d[4 * h + 3] = a.w;
      }
    } else if (vec && l.elem == EL_BF16) {
      if constexpr (V == 8) {
        const uint4 a = __ldg((const uint4*)((const uint16_t*)l.ptr + base + n));
        d[0] = a.x << 16; d[1] = a.x & 0xFFFF0000u; d[2] = a.y << 16; d[3] = a.y & 0xFFFF0000u;
        d[4] = a.z << 16; d[5] = a.z & 0xFFFF0000u; d[6] = a.w << 16; d[7] = a.w & 0xFFFF0000u;
      } else {
        const uint2 a = __ldg((const uint2*)((const uint16_t*)l.ptr + base + n));
        d[0] = a.x << 16; d[1] = a.x & 0xFFFF0000u; d[2] = a.y << 16; d[3] = a.y & 0xFFFF0000u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) d[j] = load_elem(l.ptr, base + n + j, l.elem);
    }
  }
  static __device__ __forceinline__ void store_v(const VmOut& o, long long m, long long n, bool vec, const uint32_t* s) {
    const long long at = o.offset + m * o.stride[0] + n;
    if (!RX_OUT_OK(o, at, V)) return;
    if (vec && o.elem == EL_F32) {
      uint4* q = (uint4*)((uint32_t*)o.ptr + at);
#pragma unroll
      for (int h = 0; h < V / 4; ++h) q[h] = make_uint4(s[4 * h], s[4 * h + 1], s[4 * h + 2], s[4 * h + 3]);
    } else if (vec && o.elem == EL_BF16) {
      if constexpr (V == 8) {
        uint4 w;
        w.x = bf16x2_bits(u2f(s[0]), u2f(s[1]));
        w.y = bf16x2_bits(u2f(s[2]), u2f(s[3]));
        w.z = bf16x2_bits(u2f(s[4]), u2f(s[5]));
        w.w = bf16x2_bits(u2f(s[6]), u2f(s[7]));
        *(uint4*)((uint16_t*)o.ptr + at) = w;
      } else {
        uint2 w;
        w.x = bf16x2_bits(u2f(s[0]), u2f(s[1]));
        w.y = bf16x2_bits(u2f(s[2]), u2f(s[3]));
        *(uint2*)((uint16_t*)o.ptr + at) = w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) store_elem(o.ptr, at + j, o.elem, s[j]);
    }
  }

  // 32 columns n0 .. n0 + 31 of row m; v = the accumulator values from TMEM
  static __device__ __forceinline__ void piece(Tile& ts, const Params& ep, const GemmParams& p, long long m, long long n0, uint32_t* v) {
    const VmProgram& P = ep.P;
    const bool vec = ep.vec_ok != 0;
    const int64_t idx0[kMaxRank] = {0, 0, 0, 0};
    const int lane = threadIdx.x & 31;
    float cs[NC][32];
    // every operand of the piece is requested before the chain starts, so that the loads of all groups of V columns
    // are in flight together (read-only loads: the compiler could not move them above the stores otherwise)
    uint32_t L[C::kLeaves > 0 ? C::kLeaves : 1][32];
#pragma unroll
    for (int k = 0; k < C::n_leaves(P); ++k) {
      if (k == C::kAccLeaf) continue;
#pragma unroll
      for (int sub = 0; sub < 32; sub += V) load_v(C::leaf(P, k), m, n0 + sub, vec, &L[k][sub]);
    }
    tmem_ld_wait();  // the accumulators (requested by the caller) and the operands above arrive together
#pragma unroll
    for (int sub = 0; sub < 32; sub += V) {
      uint32_t R[C::kRegs][V];
#pragma unroll
      for (int k = 0; k < C::n_leaves(P); ++k) {
        if (k == C::kAccLeaf) {
#pragma unroll
          for (int j = 0; j < V; ++j) R[C::leaf_reg(P, k)][j] = C::leaf(P, k).elem == EL_BF16 ? f2u(round_bf16(u2f(v[sub + j]))) : v[sub + j];
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) R[C::leaf_reg(P, k)][j] = L[k][sub + j];
        }
      }
      C::template exec<V>(P, R, idx0);
      if (sub == 0) {
        // the staging buffer is free again once the bulk stores of the previous block have read it; asked for as late
        // as possible, after this block's operand loads and first group of chain values
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int k = 0; k < C::n_outs(P); ++k) {
        const uint32_t* sv = R[C::out_reg(P, k)];
        if (ep.stage_off[k] < 0) {
          store_v(C::out(P, k), m, n0 + sub, vec, sv);
        } else if (C::out(P, k).elem == EL_BF16) {
          // row = lane, 64 bytes per row, 16-byte chunks swizzled as the 64-byte tensor-map swizzle expects
          // (chunk ^= (row / 2) % 4): the 32 lanes' stores spread over all banks
          const int chunk = (sub >> 3) ^ ((lane >> 1) & 3);
          *(uint4*)(ts.stage + ep.stage_off[k] + lane * 64 + chunk * 16) =
              make_uint4(bf16x2_bits(u2f(sv[0]), u2f(sv[1])), bf16x2_bits(u2f(sv[2]), u2f(sv[3])), bf16x2_bits(u2f(sv[4]), u2f(sv[5])), bf16x2_bits(u2f(sv[6]), u2f(sv[7])));
        } else {
          // f32: 128 bytes per row, 128-byte swizzle (chunk ^= row % 8)
          unsigned char* row = ts.stage + ep.stage_off[k] + lane * 128;
#pragma unroll
          for (int h = 0; h < 2; ++h) *(uint4*)(row + ((((sub >> 2) + h) ^ (lane & 7)) << 4)) = make_uint4(sv[4 * h], sv[4 * h + 1], sv[4 * h + 2], sv[4 * h + 3]);
        }
      }
#pragma unroll
      for (int q = 0; q < C::kNumCol; ++q)
#pragma unroll
        for (int j = 0; j < V; ++j) cs[q][sub + j] = u2f(R[C::col_reg(q)][j]);
#pragma unroll
      for (int q = 0; q < C::kNumFull; ++q)
#pragma unroll
        for (int j = 0; j < V; ++j) ts.full[q] += u2f(R[C::full_reg(q)][j]);
    }
    // hand the staged blocks to the copy engine
    fence_async_shared();
    __syncwarp();
    if (lane == 0) {
      bool any = false;
#pragma unroll
      for (int k = 0; k < C::n_outs(P); ++k)
        if (ep.stage_off[k] >= 0) {
          tma_store_2d(&ep.tm_out[k], ts.stage + ep.stage_off[k], (int)n0, (int)(m - lane));
          any = true;
        }
      if (any) tma_store_commit();
    }
    // column sums over the 32 rows this warp holds: a butterfly that halves the register count at every step,
    // lane j ending with the sum of column n0 + j; then one coalesced 128-byte store per sum
#pragma unroll
    for (int q = 0; q < C::kNumCol; ++q) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < o; ++i) {
          const float keep = up ? cs[q][i + o] : cs[q][i];
          const float send = up ? cs[q][i] : cs[q][i + o];
          cs[q][i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
        }
      }
      ep.col_partial[q][(m >> 5) * (long long)p.N + n0 + lane] = cs[q][0];
    }
  }

  static __device__ __forceinline__ void end_tile(Tile& ts, const Params& ep, int slot, bool row_valid) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int q = 0; q < C::kNumFull; ++q) {
      float s = row_valid ? ts.full[q] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
      if (lane == 0) ep.full_partial[q][slot] = s;
    }
  }
};

template <bool WIDE>
struct Slab2 {
  static constexpr int kBK = WIDE ? 128 : 64;
  static constexpr int kStages = WIDE ? 3 : 6;
  static constexpr int kABytes = 128 * kBK * 2;   // this CTA's rows of A
  static constexpr int kBBytes = 128 * kBK * 2;   // this CTA's half of B
  static constexpr int kStageBytes = kABytes + kBBytes;
};
constexpr int kRing2Bytes = 6 * 32768;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// commit -> the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit2(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void tc_mma2(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// TMA load of this CTA's box whose completion is counted on the *leader's* barrier
// (same offset, CTA-rank bit of the shared::cluster address cleared).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
               "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar) & 0xFEFFFFFFu)
               : "memory");
}
// arrive on the barrier at this offset in the leader CTA
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* tmap, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(smem_dst)),
               "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar) & 0xFEFFFFFFu)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile(
      "{\n"
      ".reg .b32 ra;\n"
      "mapa.shared::cluster.u32 ra, %0, 0;\n"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n"
      "}\n" ::"r"(smem_u32(bar))
      : "memory");
}


// Epilogue staging of the pair kernel: per epilogue warp two 4 KiB buffers (32 rows x 128 bytes, 128-byte swizzle).
// Each lane owns an accumulator row after tcgen05.ld, so direct global stores touch 32 different lines per
// instruction (the last tile's epilogue, which nothing overlaps, took 3.4 us that way); through shared memory the
// copy engine writes whole 128-byte row pieces and the warp only issues conflict-free 16-byte shared stores.
constexpr int kOutStageBytes = kEpiWarps * 2 * 4096;

template <bool WIDE, class Epi>
__global__ void __launch_bounds__(64 + 32 * Epi::kWarps, 1) k_gemm_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                              const __grid_constant__ CUtensorMap tmD, const __grid_constant__ GemmParams p,
                                                              const __grid_constant__ typename Epi::Params ep) {
  using S = Slab2<WIDE>;
  constexpr int STAGES2 = S::kStages, STAGE2_BYTES = S::kStageBytes, A2_BYTES = S::kABytes, BK = S::kBK;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[STAGES2], empty[STAGES2], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  unsigned char* smem = (unsigned char*)(((unsigned long long)smem_raw + 1023) & ~(unsigned long long)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int ntiles = p.tiles_m * p.tiles_n;     // 256 x 256 tiles
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");  // the first copies wait for the descriptors otherwise
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    for (int s = 0; s < STAGES2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * Epi::kWarps); }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc2(&tmem_base_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  // Launched with programmatic stream serialization, the CTAs get here (barriers, TMEM, descriptors ready) while the
  // kernel in front on the stream may still be running; every global read and write comes after this wait.
  pdl_wait();
  pdl_release();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_p = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < ntiles && !*abort_p; t += npairs) {
        const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
        const int m0 = tm * 256 + (int)rank * 128, n0 = tn * 256 + (int)rank * 128;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, kGemmWaitLimit, abort_p)) { *abort_p = 1; *p.status = 13; break; }
          unsigned char* sa = smem + stage * STAGE2_BYTES;
          unsigned char* sb = sa + A2_BYTES;
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * STAGE2_BYTES);  // both CTAs' boxes land on the leader's barrier
          const int k0 = kb * BK;
          if (WIDE) {
            // one 32 KiB copy per operand half: {64, 128 rows, 2 groups}
            if (p.a_mn) tma_load_3d_pair(sa, &tmA, 0, k0, m0 >> 6, &full[stage]);
            else tma_load_3d_pair(sa, &tmA, 0, m0, k0 >> 6, &full[stage]);
            if (p.b_mn) tma_load_3d_pair(sb, &tmB, 0, k0, n0 >> 6, &full[stage]);
            else tma_load_3d_pair(sb, &tmB, 0, n0, k0 >> 6, &full[stage]);
          } else {
            if (p.a_mn) {
              tma_load_2d_pair(sa, &tmA, m0, k0, &full[stage]);
              tma_load_2d_pair(sa + 8192, &tmA, m0 + 64, k0, &full[stage]);
            } else {
              tma_load_2d_pair(sa, &tmA, k0, m0, &full[stage]);
            }
            if (p.b_mn) {
              tma_load_2d_pair(sb, &tmB, n0, k0, &full[stage]);
              tma_load_2d_pair(sb + 8192, &tmB, n0 + 64, k0, &full[stage]);
            } else {
              tma_load_2d_pair(sb, &tmB, k0, n0, &full[stage]);
            }
          }
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) | ((uint32_t)(256 >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = pair; t < ntiles && !*abort_p; t += npairs, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, kGemmWaitLimit, abort_p)) { *abort_p = 1; *p.status = 14; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, kGemmWaitLimit, abort_p)) { *abort_p = 1; *p.status = 15; ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE2_BYTES);
          const uint32_t sb = sa + A2_BYTES;
          // MN-major: the two 64-wide groups of the 128 rows are one slab-height apart (8 KiB for 64 k-rows,
          // 16 KiB for 128), and 16 k-rows are 2 KiB.  K-major: 16 k-columns are 32 bytes inside a 64-column
          // group; the wide slab's second group starts 16 KiB further on.
          constexpr uint32_t kGroupBytes = 128 * BK;
          const uint64_t adesc0 = p.a_mn ? smem_desc(sa, kGroupBytes, 1024) : smem_desc(sa, 16, 1024);
          const uint64_t bdesc0 = p.b_mn ? smem_desc(sb, kGroupBytes, 1024) : smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t aoff = p.a_mn ? k * 2048 : ((k >> 2) * 16384 + (k & 3) * 32);
            const uint32_t boff = p.b_mn ? k * 2048 : ((k >> 2) * 16384 + (k & 3) * 32);
            tc_mma2(tmem_d, adesc0 + (aoff >> 4), bdesc0 + (boff >> 4), idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit2(&empty[stage]);
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit2(&acc_full[buf]);
      }
    }
  } else {
    const int quad = warp & 3;
    int it = 0;
    for (int t = pair; t < ntiles && !*abort_p; t += npairs, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase, kGemmWaitLimit, abort_p)) { *abort_p = 1; *p.status = 16; break; }
      tc_fence_after();
      const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
      const long long m = (long long)tm * 256 + rank * 128 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * 256;
      if constexpr (!Epi::kPlain) {
        // fused epilogue: every 32-column piece of this lane's accumulator row goes through the chain
        typename Epi::Tile ts;
        Epi::begin_tile(ts, smem + kRing2Bytes + (warp - 2) * 4096);
        const bool row_ok = m < p.M;
#pragma unroll 1
        constexpr int kColsPerWarp = 256 / (Epi::kWarps / 4);
        const int c0 = ((warp - 2) >> 2) * kColsPerWarp;
        for (int c = c0; c < c0 + kColsPerWarp; c += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + c, v);
          // rows and columns come in whole groups of 32 (the launcher checks M % 32 == 0 and N % 32 == 0); piece()
          // waits for the accumulators itself, after it has asked for its other operands
          if (row_ok && (long long)tn * 256 + c < p.N) Epi::piece(ts, ep, p, m, (long long)tn * 256 + c, v);
          else tmem_ld_wait();
        }
        Epi::end_tile(ts, ep, (t * 2 + (int)rank) * Epi::kWarps + (warp - 2), row_ok);
      } else if (p.tma_store) {
        unsigned char* ob = smem + kRing2Bytes + (warp - 2) * 8192;
        const int row0 = tm * 256 + (int)rank * 128 + quad * 32;   // row of lane 0
        const int sw = lane & 7;
        if (p.out_bf16) {
#pragma unroll 1
          for (int c = 0; c < 256; c += 64) {   // 64 bf16 columns = 128 bytes per row
            uint32_t v[32], w[32];
            tmem_ld32(taddr + c, v);
            tmem_ld32(taddr + c + 32, w);
            if (lane == 0) tma_store_wait_read<1>();  // the buffer written two chunks ago has been read
            __syncwarp();
            tmem_ld_wait();
            unsigned char* dst = ob + ((c >> 6) & 1) * 4096 + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t* q = j < 4 ? v + 8 * j : w + 8 * (j - 4);
              uint4 o;
              o.x = bf16x2_bits(u2f(q[0]), u2f(q[1]));
              o.y = bf16x2_bits(u2f(q[2]), u2f(q[3]));
              o.z = bf16x2_bits(u2f(q[4]), u2f(q[5]));
              o.w = bf16x2_bits(u2f(q[6]), u2f(q[7]));
              *(uint4*)(dst + ((j ^ sw) << 4)) = o;
            }
            fence_async_shared();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, ob + ((c >> 6) & 1) * 4096, tn * 256 + c, row0);
              tma_store_commit();
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < 256; c += 32) {   // 32 f32 columns = 128 bytes per row
            uint32_t v[32];
            tmem_ld32(taddr + c, v);
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
            tmem_ld_wait();
            unsigned char* dst = ob + ((c >> 5) & 1) * 4096 + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) *(uint4*)(dst + ((j ^ sw) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            fence_async_shared();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, ob + ((c >> 5) & 1) * 4096, tn * 256 + c, row0);
              tma_store_commit();
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + c, v);
          tmem_ld_wait();
          store_row32(p, m, (long long)tn * 256 + c, v);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
    }
    if ((p.tma_store || !Epi::kPlain) && lane == 0) tma_store_wait<0>();  // this thread's bulk stores have been written
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or exits while its peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}


}  // namespace rx
