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

#include <string>

#include "rx_gemm.h"
#include "rx_gemm_pair.cuh"
#include "rx_jit.h"
#include "rx_tma.h"

namespace rx {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kThreads = kGemmThreads;
constexpr long long kWaitLimit = kGemmWaitLimit;

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
  static const bool pdl = !(getenv("RX_PDL") && atoi(getenv("RX_PDL")) == 0);
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel waits (griddepcontrol) before it touches global memory
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem2;
  cfg.stream = d->stream;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 2 : 1;
  if (!attr2) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_pair<WIDE, EpiPlain>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return e;
    cfg.gridDim = dim3(d->sm_count & ~1);
    if (cudaOccupancyMaxActiveClusters(&max_clusters, k_gemm_pair<WIDE, EpiPlain>, &cfg) != cudaSuccess || max_clusters < 1) {
      cudaGetLastError();
      max_clusters = d->sm_count / 2;
    }
    attr2 = true;
  }
  int pairs = std::min(p.tiles_m * p.tiles_n, std::min(max_clusters, d->sm_count / 2));
  cfg.gridDim = dim3(2 * pairs);
  return cudaLaunchKernelEx(&cfg, k_gemm_pair<WIDE, EpiPlain>, tmA, tmB, tmD, p, EpiPlain::Params{0});
}

}  // namespace

constexpr int kFusedEpiWarps = 8;  // EpiChain::kWarps

// What the generated chain policy of a fused epilogue carries besides the chain itself.
std::string gemm_epilogue_members(const GemmDesc& g) {
  std::string extra = "  static constexpr int kLeaves = " + std::to_string(g.n_leaves) + ";\n  static constexpr int kAccLeaf = " + std::to_string(g.acc_leaf) + ";\n  static constexpr int kNumCol = " + std::to_string(g.n_col) +
                      ";\n  static constexpr int kNumFull = " + std::to_string(g.n_full) + ";\n";
  auto regs = [](const char* name, const int* r, int n) {
    std::string t = std::string("  static __device__ __forceinline__ int ") + name + "(int q) {\n    switch (q) {\n";
    for (int q = 0; q < n; ++q) t += "      case " + std::to_string(q) + ": return " + std::to_string(r[q]) + ";\n";
    return t + "    }\n    return 0;\n  }\n";
  };
  return extra + regs("col_reg", g.col_reg, g.n_col) + regs("full_reg", g.full_reg, g.n_full);
}
const char* gemm_epilogue_family(bool wide) { return wide ? "k_gemm_pair<true, rx::EpiChain<rx::SpecChain>>" : "k_gemm_pair<false, rx::EpiChain<rx::SpecChain>>"; }

// The pair kernel compiled at run time around the step's fused chain.
static cudaError_t launch_fused(RxDevice* d, const GemmDesc& g, bool wide, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                const GemmEpilogueArgs& ea) {
  EpiChainParams ep{};
  ep.P = *ea.prog;
  for (int q = 0; q < 2; ++q) {
    ep.col_partial[q] = ea.col_partial[q];
    ep.full_partial[q] = ea.full_partial[q];
  }
  // 8 consecutive elements per access: 16 bytes of bf16, two 16-byte halves of f32
  bool vec = true;
  auto esz = [](int e) { return e == EL_BF16 ? 2 : 4; };
  for (int k = 0; k < ep.P.n_leaves; ++k) {
    const VmLeaf& l = ep.P.leaf[k];
    if (k == g.acc_leaf || l.stride[1] == 0) continue;
    vec = vec && ((uintptr_t)l.ptr + (uintptr_t)l.offset * esz(l.elem)) % 16 == 0 && ((size_t)l.stride[0] * esz(l.elem)) % 16 == 0;
  }
  for (int k = 0; k < ep.P.n_outs; ++k) {
    const VmOut& o = ep.P.out[k];
    vec = vec && ((uintptr_t)o.ptr + (uintptr_t)o.offset * esz(o.elem)) % 16 == 0 && ((size_t)o.stride[0] * esz(o.elem)) % 16 == 0;
  }
  ep.vec_ok = vec ? 1 : 0;
  // results that can go through the shared-memory staging buffer and tiled bulk stores (as many as fit in 4 KiB)
  int used = 0;
  for (int k = 0; k < kVmMaxOuts; ++k) ep.stage_off[k] = -1;
  for (int k = 0; k < ep.P.n_outs && !getenv("RX_EPI_DIRECT_STORE"); ++k) {
    const VmOut& o = ep.P.out[k];
    const int es = esz(o.elem), need = 32 * 32 * es;
    const char* base = (const char*)o.ptr + (size_t)o.offset * es;
    if (used + need > 4096 || (uintptr_t)base % 16 || ((size_t)o.stride[0] * es) % 16) continue;
    if (!tma_make_2d(&ep.tm_out[k], o.elem == EL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, (uint64_t)p.N, (uint64_t)p.M,
                     (uint64_t)o.stride[0] * es, 32, 32, o.elem == EL_BF16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B))
      continue;
    ep.stage_off[k] = used;
    used += need;
  }
  const std::string extra = gemm_epilogue_members(g);
  const char* family = gemm_epilogue_family(wide);
  bool failed = false;
  const JitKernel* k = jit_chain_kernel(d->ordinal, ep.P, family, -1, INT64_MAX, &failed, extra.c_str(), true);
  if (!k) return failed ? cudaErrorUnknown : cudaErrorNotSupported;
  CUtensorMap tmD{};  // the fused epilogue stores from registers
  GemmParams pp = p;
  pp.tma_store = 0;
  const size_t smem2 = (size_t)kRing2Bytes + kOutStageBytes + 1024;
  const int pairs = std::min(pp.tiles_m * pp.tiles_n, d->sm_count / 2);
  void* args[] = {(void*)&tmA, (void*)&tmB, (void*)&tmD, (void*)&pp, (void*)&ep};
  static const bool pdl = !(getenv("RX_PDL") && atoi(getenv("RX_PDL")) == 0);
  return jit_launch_cluster(k, 2u * (unsigned)pairs, 64u + 32u * (unsigned)kFusedEpiWarps, 2, smem2, args, d->stream, pdl);
}

cudaError_t run_gemm_tc(RxDevice* d, const Step& st, const void* a, const void* b, void* out, const GemmEpilogueArgs* epilogue, bool* handled) {
  *handled = false;
  const GemmDesc& g = st.gemm;
  if (getenv("RX_GEMM_SIMT")) return cudaSuccess;
  if (g.in_dt != DT::BF16 || g.batch != 1) return cudaSuccess;
  if (!(g.out_dt == DT::BF16 || g.out_dt == DT::F32)) return cudaSuccess;
  const bool a_k = g.a_sk == 1, a_m = g.a_sm == 1, b_k = g.b_sk == 1, b_n = g.b_sn == 1;
  if (!(a_k || a_m) || !(b_k || b_n)) return cudaSuccess;
  const bool a_mn = !a_k, b_mn = !b_k;  // prefer K-major when a dimension has extent 1
  const long long a_pitch = a_mn ? g.a_sk : g.a_sm, b_pitch = b_mn ? g.b_sk : g.b_sn;
  const __nv_bfloat16* A = (const __nv_bfloat16*)a + g.a_off;
  const __nv_bfloat16* B = (const __nv_bfloat16*)b + g.b_off;
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
    p.tma_store = !g.has_epilogue && !getenv("RX_GEMM_DIRECT_STORE") && ((uintptr_t)out % 16 == 0) && ((size_t)p.ldd * esz % 16 == 0) &&
                  tma_make_2d(&tmD, p.out_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, out, (uint64_t)g.N, (uint64_t)g.M,
                              (uint64_t)p.ldd * esz, (uint32_t)(128 / esz), 32, CU_TENSOR_MAP_SWIZZLE_128B);
    cudaError_t e;
    if (g.has_epilogue) {
      if (!epilogue || !epilogue->prog) return cudaErrorInvalidValue;
      e = launch_fused(d, g, wide, tmA, tmB, p, *epilogue);
    } else {
      e = wide ? launch_pair_kernel<true>(d, tmA, tmB, tmD, p) : launch_pair_kernel<false>(d, tmA, tmB, tmD, p);
    }
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
