// bf16 dot_general on the 5th-generation tensor cores (tcgen05 + TMEM), fp32
// accumulation -- the contraction Reactant emits for `W * X`
// (src/stdlibs/LinearAlgebra.jl:274-330 -> src/Ops.jl:1075-1200) and the three
// transposed-operand contractions Enzyme's reverse pass adds for its gradient.
//
// Persistent kernel, one CTA per SM, 128 x 256 output tiles:
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte
//               swizzle) of the A (128 x 64) and B (256 x 64) k-slabs into a
//               4-stage shared-memory ring, completion on `full` mbarriers;
//   warp 1      allocates TMEM (512 columns = two 128 x 256 fp32 accumulators);
//               one lane issues tcgen05.mma (M128 N256 K16, cta_group::1) four
//               times per slab, releases the slab with tcgen05.commit -> `empty`,
//               and hands a finished accumulator over with tcgen05.commit ->
//               `acc_full`;
//   warps 2..5  epilogue: tcgen05.ld the accumulator (32 lanes x 32 columns per
//               instruction), round once to the output type, store; then free the
//               accumulator (`acc_empty`) so the next tile's MMAs overlap it.
// Operands may be K-major or MN-major in memory (any of the four combinations):
// the transposes of the reverse pass are expressed in the shared-memory and
// instruction descriptors, never materialised.  No multicast, one CTA per tile.
// Every mbarrier wait is bounded; a wait that runs out sets a status word and
// all roles drain, TMEM is released and the kernel returns.
#include <cuda_bf16.h>

#include "rx_gemm.h"
#include "rx_tma.h"

namespace rx {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr long long kWaitLimit = 4000000;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;        // 1: operand is MN-major in memory (contiguous along M resp. N)
  void* D;
  long long ldd;
  int out_bf16;
  int tiles_m, tiles_n;
  int* status;
  int tma_store;         // pair kernel: epilogue goes through shared memory and tiled bulk stores
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


// One epilogue step: 32 consecutive columns of row m, rounded once to the output type.
__device__ __forceinline__ void store_row32(const GemmParams& p, long long m, long long n, const uint32_t* v) {
  if (m >= p.M) return;
  if (p.out_bf16) {
    __nv_bfloat16* row = (__nv_bfloat16*)p.D + m * p.ldd + n;
    if (n + 32 <= p.N && (((uintptr_t)row & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
        __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
        __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
        __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
        o.x = *(uint32_t*)&b0; o.y = *(uint32_t*)&b1; o.z = *(uint32_t*)&b2; o.w = *(uint32_t*)&b3;
        *(uint4*)(row + 8 * q) = o;
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (n + j < p.N) row[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
    }
  } else {
    float* row = (float*)p.D + m * p.ldd + n;
    if (n + 32 <= p.N && (((uintptr_t)row & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < 8; ++q) *(uint4*)(row + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
      for (int j = 0; j < 32; ++j)
        if (n + j < p.N) row[j] = __uint_as_float(v[j]);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) k_gemm_tc(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                         const __grid_constant__ GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzle atoms are 1 KiB aligned
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kEpiWarps); }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_p = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < ntiles && !*abort_p; t += gridDim.x) {
        const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 3; break; }
          unsigned char* sa = smem + stage * STAGE_BYTES;
          unsigned char* sb = sa + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if (p.a_mn) {
            tma_load_2d(sa, &tmA, m0, k0, &full[stage]);
            tma_load_2d(sa + 8192, &tmA, m0 + 64, k0, &full[stage]);
          } else {
            tma_load_2d(sa, &tmA, k0, m0, &full[stage]);
          }
          if (p.b_mn) {
#pragma unroll
            for (int j = 0; j < 4; ++j) tma_load_2d(sb + j * 8192, &tmB, n0 + 64 * j, k0, &full[stage]);
          } else {
            tma_load_2d(sb, &tmB, k0, n0, &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=bf16, majors, N>>3, M>>4
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn << 15) | ((uint32_t)p.b_mn << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < ntiles && !*abort_p; t += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 4; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 5; ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          // K-major: rows of 128 B, 8-row groups 1 KiB apart; a K=16 step is 32 B inside the row.
          // MN-major: 64-element blocks of 8 KiB (LBO), 8-k groups 1 KiB apart (SBO); a K=16 step is 2 KiB.
          const uint64_t adesc0 = p.a_mn ? smem_desc(sa, 8192, 1024) : smem_desc(sa, 16, 1024);
          const uint64_t bdesc0 = p.b_mn ? smem_desc(sb, 8192, 1024) : smem_desc(sb, 16, 1024);
          const uint64_t astep = p.a_mn ? (2048 >> 4) : (32 >> 4);
          const uint64_t bstep = p.b_mn ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) tc_mma(tmem_d, adesc0 + k * astep, bdesc0 + k * bstep, idesc, (kb | k) ? 1u : 0u);
          tc_commit(&empty[stage]);  // slab may be refilled once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&acc_full[buf]);
      }
    }
  } else {
    // epilogue warps: TMEM lane quadrant is warp % 4
    const int quad = warp & 3;
    int it = 0;
    for (int t = blockIdx.x; t < ntiles && !*abort_p; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 6; break; }
      tc_fence_after();
      const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
      const long long m = (long long)tm * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld32(taddr + c, v);
        tmem_ld_wait();
        store_row32(p, m, (long long)tn * BN + c, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// =======================================================================================
// Two-CTA variant: a cluster of two CTAs (two SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2 (M256 N256 K16).  Each CTA stages its own 128 rows of A and
// *half* of the B slab (128 of the 256 N rows), so per SM the shared-memory fill and the
// L2->SM traffic per FLOP drop by a third against the one-CTA kernel, which is what its
// mainloop is bound by.  The leader CTA (cluster rank 0) issues every MMA; the TMA loads of
// both CTAs complete on the leader's `full` barrier (cta_group::2 loads, no multicast);
// tcgen05.commit with a two-CTA mask releases slabs / publishes accumulators in both CTAs;
// both CTAs' epilogue warps arrive on the leader's `acc_empty` barrier.  Each CTA's TMEM
// holds its 128 accumulator rows x 256 columns, double buffered.
// =======================================================================================
// Two slab geometries with the same 192 KiB ring.  WIDE (operand extents that are multiples of 64 along their
// contiguous dimension): 128-deep k-slabs, three stages, each operand half fetched by ONE 32 KiB copy through a
// 3-D "grouped" tensor map.  Otherwise: 64-deep slabs, six stages, 2-D maps (one 16 KiB copy for a K-major half,
// two 8 KiB copies for an MN-major half) with zero fill past the edges.  Measured on B200, the per-SM copy engine
// moves 56 / 68 / 78 bytes per clock with 8 / 16 / 32 KiB copies whatever the ring depth or the number of busy SMs,
// and the MMAs of a 256 x 256 pair tile consume 64 bytes per clock per SM -- so only the wide form keeps ahead.
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

template <bool WIDE>
__global__ void __launch_bounds__(kThreads, 1) k_gemm_tc2(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                          const __grid_constant__ CUtensorMap tmD, const __grid_constant__ GemmParams p) {
  using S = Slab2<WIDE>;
  constexpr int STAGES2 = S::kStages, STAGE2_BYTES = S::kStageBytes, A2_BYTES = S::kABytes, BK = S::kBK;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[STAGES2], empty[STAGES2], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int ntiles = p.tiles_m * p.tiles_n;     // 256 x 256 tiles
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");  // the first copies wait for the descriptors otherwise
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    for (int s = 0; s < STAGES2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * kEpiWarps); }
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
          if (!mbar_wait(&empty[stage], phase ^ 1, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 13; break; }
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
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 14; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 15; ok = false; break; }
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
      if (!mbar_wait(&acc_full[buf], acc_phase, kWaitLimit, abort_p)) { *abort_p = 1; *p.status = 16; break; }
      tc_fence_after();
      const int tm = t / p.tiles_n, tn = t - tm * p.tiles_n;
      const long long m = (long long)tm * 256 + rank * 128 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * 256;
      if (p.tma_store) {
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
              __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(q[0]), __uint_as_float(q[1]));
              __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(q[2]), __uint_as_float(q[3]));
              __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(q[4]), __uint_as_float(q[5]));
              __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(q[6]), __uint_as_float(q[7]));
              o.x = *(uint32_t*)&b0; o.y = *(uint32_t*)&b1; o.z = *(uint32_t*)&b2; o.w = *(uint32_t*)&b3;
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
    if (p.tma_store && lane == 0) tma_store_wait<0>();  // this thread's bulk stores have been written
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or exits while its peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

bool make_operand_map(CUtensorMap* m, const __nv_bfloat16* base, bool mn_major, long long mn_extent, long long k_extent, long long pitch_elems, int box_mn) {
  // K-major: inner dim = K (contiguous), rows = MN with pitch; box 64 (K) x box_mn
  // MN-major: inner dim = MN (contiguous), rows = K with pitch; box 64 (MN) x 64 (K)
  if (mn_major) return tma_make_2d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)mn_extent, (uint64_t)k_extent, (uint64_t)pitch_elems * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  return tma_make_2d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)k_extent, (uint64_t)mn_extent, (uint64_t)pitch_elems * 2, 64, (uint32_t)box_mn, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <bool WIDE>
cudaError_t launch_pair_kernel(RxDevice* d, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const GemmParams& p) {
  const size_t smem2 = (size_t)Slab2<WIDE>::kStages * Slab2<WIDE>::kStageBytes + kOutStageBytes + 1024;
  static_assert(Slab2<WIDE>::kStages * Slab2<WIDE>::kStageBytes == kRing2Bytes, "both slab geometries use the same ring");
  static bool attr2_dev[64] = {};          // function attributes are per device
  static int max_clusters_dev[64] = {};
  bool& attr2 = attr2_dev[d->ordinal & 63];
  int& max_clusters = max_clusters_dev[d->ordinal & 63];
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem2;
  cfg.stream = d->stream;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  if (!attr2) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_tc2<WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return e;
    cfg.gridDim = dim3(d->sm_count & ~1);
    if (cudaOccupancyMaxActiveClusters(&max_clusters, k_gemm_tc2<WIDE>, &cfg) != cudaSuccess || max_clusters < 1) {
      cudaGetLastError();
      max_clusters = d->sm_count / 2;
    }
    attr2 = true;
  }
  int pairs = std::min(p.tiles_m * p.tiles_n, std::min(max_clusters, d->sm_count / 2));
  cfg.gridDim = dim3(2 * pairs);
  return cudaLaunchKernelEx(&cfg, k_gemm_tc2<WIDE>, tmA, tmB, tmD, p);
}

}  // namespace

cudaError_t run_gemm_tc(RxDevice* d, const Step& st, const void* a, const void* b, void* out, bool* handled) {
  *handled = false;
  const GemmDesc& g = st.gemm;
  if (getenv("RX_GEMM_SIMT")) return cudaSuccess;
  if (g.in_dt != DT::BF16 || g.batch != 1) return cudaSuccess;
  if (!(g.out_dt == DT::BF16 || g.out_dt == DT::F32)) return cudaSuccess;
  const bool a_k = g.a_sk == 1, a_m = g.a_sm == 1, b_k = g.b_sk == 1, b_n = g.b_sn == 1;
  if (!(a_k || a_m) || !(b_k || b_n)) return cudaSuccess;
  const bool a_mn = !a_k, b_mn = !b_k;  // prefer K-major when a dimension has extent 1
  const long long a_pitch = a_mn ? g.a_sk : g.a_sm, b_pitch = b_mn ? g.b_sk : g.b_sn;
  const __nv_bfloat16* A = (const __nv_bfloat16*)a + st.prog.leaf[0].offset;
  const __nv_bfloat16* B = (const __nv_bfloat16*)b + st.prog.leaf[1].offset;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15) || (a_pitch % 8) || (b_pitch % 8) || a_pitch <= 0 || b_pitch <= 0) return cudaSuccess;
  if (g.M < 1 || g.N < 1 || g.K < 1 || g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX) return cudaSuccess;
  // two-CTA tiles (256 x 256 per SM pair) when the problem is large enough to fill them
  const bool two_cta = !getenv("RX_GEMM_1CTA") && g.M >= 256 && g.N >= 256;
  CUtensorMap tmA, tmB;
  if (!make_operand_map(&tmA, A, a_mn, g.M, g.K, a_pitch, BM)) return cudaSuccess;
  if (!make_operand_map(&tmB, B, b_mn, g.N, g.K, b_pitch, two_cta ? 128 : BN)) return cudaSuccess;
  GemmParams p{};
  p.M = (int)g.M;
  p.N = (int)g.N;
  p.K = (int)g.K;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.D = out;
  p.ldd = g.N;
  p.out_bf16 = g.out_dt == DT::BF16;
  p.tiles_m = (int)((g.M + BM - 1) / BM);
  p.tiles_n = (int)((g.N + BN - 1) / BN);
  int* dstatus = nullptr;
  cudaHostGetDevicePointer(&dstatus, d->status, 0);
  p.status = dstatus + 2;
  if (two_cta) {
    p.tiles_m = (int)((g.M + 255) / 256);
    p.tiles_n = (int)((g.N + 255) / 256);
    // wide slabs need whole 64-element groups along each operand's contiguous dimension
    bool wide = !getenv("RX_GEMM_NARROW") && ((a_mn ? g.M : g.K) % 64 == 0) && ((b_mn ? g.N : g.K) % 64 == 0);
    if (wide) {
      CUtensorMap wa, wb;
      wide = tma_make_grouped(&wa, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, a_mn ? g.M : g.K, a_mn ? g.K : g.M, (uint64_t)a_pitch * 2, 128, 2) &&
             tma_make_grouped(&wb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, B, b_mn ? g.N : g.K, b_mn ? g.K : g.N, (uint64_t)b_pitch * 2, 128, 2);
      if (wide) {
        tmA = wa;
        tmB = wb;
      }
    }
    // output tensor map for the staged epilogue: boxes of 32 rows x 128 bytes, 128-byte swizzle
    CUtensorMap tmD{};
    const size_t esz = p.out_bf16 ? 2 : 4;
    p.tma_store = !getenv("RX_GEMM_DIRECT_STORE") && ((uintptr_t)out % 16 == 0) && ((size_t)p.ldd * esz % 16 == 0) &&
                  tma_make_2d(&tmD, p.out_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, out, (uint64_t)g.N, (uint64_t)g.M,
                              (uint64_t)p.ldd * esz, (uint32_t)(128 / esz), 32, CU_TENSOR_MAP_SWIZZLE_128B);
    cudaError_t e = wide ? launch_pair_kernel<true>(d, tmA, tmB, tmD, p) : launch_pair_kernel<false>(d, tmA, tmB, tmD, p);
    ++d->launches;
    *handled = true;
    return e != cudaSuccess ? e : cudaGetLastError();
  }
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  static bool attr_dev[64] = {};
  bool& attr = attr_dev[d->ordinal & 63];
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  int grid = std::min(p.tiles_m * p.tiles_n, d->sm_count);
  k_gemm_tc<<<grid, kThreads, smem, d->stream>>>(tmA, tmB, p);
  ++d->launches;
  *handled = true;
  return cudaGetLastError();
}

}  // namespace rx
