// Tensor-map construction and the TMA / mbarrier PTX wrappers shared by the
// stencil and GEMM kernels.  The driver entry point is looked up at run time so
// that the library carries no link-time dependency on libcuda (it must load on
// machines without a GPU).  Every wait is bounded.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rx {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tma_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
    cudaGetLastError();
  }
  return fn;
}

// 2-D map over a row-major array: dim0 (inner, contiguous) x dim1, row pitch in bytes.
inline bool tma_make_2d(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                        uint32_t box_outer, CUtensorMapSwizzle swz) {
  EncodeTiledFn enc = tma_encode_fn();
  if (!enc) return false;
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, dt, 2, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D map that fetches `groups` adjacent 64-element (128-byte) column groups of a row-major 16-bit matrix with ONE
// copy: dim0 = the 64 elements of a group, dim1 = the rows (pitch), dim2 = the groups (128 bytes apart).  A box
// {64, box_rows, box_groups} lands in shared memory as box_groups consecutive [box_rows][128 B] blocks -- the layout
// the 128-byte-swizzled UMMA descriptors expect -- and a copy of 32 KiB moves more bytes per clock than two of
// 16 KiB or four of 8 KiB (the copy engine has a fixed cost per copy).  `cols` must be a multiple of 64.
inline bool tma_make_grouped(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows,
                             uint32_t box_groups) {
  EncodeTiledFn enc = tma_encode_fn();
  if (!enc || cols % 64) return false;
  cuuint64_t gdim[3] = {64, rows, cols / 64};
  cuuint64_t gstride[2] = {pitch_bytes, 128};
  cuuint32_t box[3] = {64, box_rows, box_groups};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(m, dt, 3, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if the phase did not complete within `limit` polls, or as
// soon as *abort becomes non-zero (another role of the CTA gave up).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit, volatile int* abort = nullptr) {
  for (long long i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (abort && (i & 255) == 255 && *abort) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
               "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
// Tiled store shared -> global (bulk async group).  Rows and columns outside the tensor are clipped by the copy
// engine; x * element size must be a multiple of 16 bytes and never negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's store groups still read their shared-memory source / are still in flight
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// generic-proxy writes to shared memory become visible to the async proxy (the copy engine)
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
#endif

}  // namespace rx
