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
}  // namespace rx
#include "rx_tma_device.cuh"
namespace rx {
#endif

}  // namespace rx
