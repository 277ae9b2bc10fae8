// dot_general on the device (src/Ops.jl:1075-1200; matmul lowering
// src/stdlibs/LinearAlgebra.jl:274-330): D[m][n] = sum_k A(m,k) B(k,n), operands
// addressed through element strides so that the transposes Reactant folds into
// dimension numbers never get materialised.  bf16 or f32 inputs, fp32
// accumulation, output rounded once to the result type.
//
// k_gemm_simt is the shape-agnostic CUDA-core path (any strides, any sizes).
#include "rx_gemm.h"

#include <cuda_bf16.h>

namespace rx {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TIn>
__device__ __forceinline__ float ldf(const TIn* p, int64_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __uint_as_float(((uint32_t)__ldg((const uint16_t*)p + i)) << 16);
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) k_gemm_simt(const TIn* __restrict__ A, const TIn* __restrict__ B, TOut* __restrict__ D, int64_t M, int64_t N, int64_t K,
                                                   int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t a_sb, int64_t b_sb, int64_t d_sb) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  A += blockIdx.z * a_sb;
  B += blockIdx.z * b_sb;
  D += blockIdx.z * d_sb;
  int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      // walk the contiguous operand dim fastest
      int mi, ki;
      if (a_sk == 1) { ki = e % TK; mi = e / TK; } else { mi = e % TM; ki = e / TM; }
      int64_t m = m0 + mi, k = k0 + ki;
      As[ki][mi] = (m < M && k < K) ? ldf<TIn>(A, m * a_sm + k * a_sk) : 0.f;
    }
    for (int e = threadIdx.x; e < TN * TK; e += 256) {
      int ni, ki;
      if (b_sk == 1) { ki = e % TK; ni = e / TK; } else { ni = e % TN; ki = e / TN; }
      int64_t n = n0 + ni, k = k0 + ki;
      Bs[ki][ni] = (n < N && k < K) ? ldf<TIn>(B, k * b_sk + n * b_sn) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) {
        if constexpr (sizeof(TOut) == 2) D[m * N + n] = __float2bfloat16_rn(acc[i][j]);
        else D[m * N + n] = acc[i][j];
      }
    }
}

}  // namespace

cudaError_t run_gemm_tc(RxDevice* d, const Step& st, const void* a, const void* b, void* out, const GemmEpilogueArgs* epilogue, bool* handled);

cudaError_t run_gemm(RxDevice* d, const Step& st, const void* a, const void* b, void* out, const GemmEpilogueArgs* epilogue) {
  const GemmDesc& g = st.gemm;
  bool handled = false;
  cudaError_t e = run_gemm_tc(d, st, a, b, out, epilogue, &handled);
  d->last_gemm_tc = handled;
  if (handled) return e;
  // a step planned with a fused epilogue exists only in the tensor-core kernel (the planner checked the shape)
  if (g.has_epilogue) return cudaErrorNotSupported;
  dim3 grid((unsigned)((g.N + TN - 1) / TN), (unsigned)((g.M + TM - 1) / TM), (unsigned)g.batch);
  int64_t ao = g.a_off, bo = g.b_off;
  if (g.in_dt == DT::BF16) {
    auto* A = (const __nv_bfloat16*)a + ao;
    auto* B = (const __nv_bfloat16*)b + bo;
    if (g.out_dt == DT::BF16)
      k_gemm_simt<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, d->stream>>>(A, B, (__nv_bfloat16*)out, g.M, g.N, g.K, g.a_sm, g.a_sk, g.b_sk, g.b_sn, g.a_sb, g.b_sb, g.d_sb);
    else
      k_gemm_simt<__nv_bfloat16, float><<<grid, 256, 0, d->stream>>>(A, B, (float*)out, g.M, g.N, g.K, g.a_sm, g.a_sk, g.b_sk, g.b_sn, g.a_sb, g.b_sb, g.d_sb);
  } else {
    auto* A = (const float*)a + ao;
    auto* B = (const float*)b + bo;
    if (g.out_dt == DT::BF16)
      k_gemm_simt<float, __nv_bfloat16><<<grid, 256, 0, d->stream>>>(A, B, (__nv_bfloat16*)out, g.M, g.N, g.K, g.a_sm, g.a_sk, g.b_sk, g.b_sn, g.a_sb, g.b_sb, g.d_sb);
    else
      k_gemm_simt<float, float><<<grid, 256, 0, d->stream>>>(A, B, (float*)out, g.M, g.N, g.K, g.a_sm, g.a_sk, g.b_sk, g.b_sn, g.a_sb, g.b_sb, g.d_sb);
  }
  ++d->launches;
  return cudaGetLastError();
}

}  // namespace rx
