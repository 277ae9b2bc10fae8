// RxSinSumAddNoAlloc: sum(sin.(x) .+ y) for callers that must not allocate.
//
// Some hosts cannot let a library call cudaMalloc on their behalf: a runtime
// that has already claimed (almost) all device memory for its own arena, the
// way Reactant's stock GPU client preallocates a fraction of the device
// (XLA_REACTANT_GPU_MEM_FRACTION / XLA_REACTANT_GPU_PREALLOCATE,
// src/xla/XLA.jl:211-235), would see the allocation fail or eat into its
// budget; a latency-critical loop cannot afford the device-wide
// synchronisation that cudaMalloc / cudaFree imply; and a host that audits its
// memory budget wants every byte to be its own.  For them this one entry point
// runs the fused map-reduce with no allocation at all: inputs and the output
// are the caller's device pointers, and the cross-CTA scratch (one partial sum
// per 65536-element chunk plus a counter) lives in a fixed array that is part
// of the library image.
//
// What that implies for the caller:
//  * Size limit.  The array holds 16384 partials, so n may be at most
//    16384 * 65536 = 2^30 elements; larger n is refused with RX_ERR_TOO_LARGE
//    and nothing is launched.  The array costs 64 KiB + 256 B of device memory
//    on every GPU that loads the library, for the life of the process.
//  * First call per device.  The first call made with a given device current
//    looks up the array's device address (cudaGetSymbolAddress) and the SM
//    count, once.  Make that first call outside any stream capture.
//  * One call at a time per device.  All calls share the array, and it keeps
//    whatever the previous call left in it.  The counter is cleared on the
//    caller's stream before every launch; partials are always written before
//    they are read.  Two calls whose kernels overlap on the GPU (different
//    streams, or different host threads) race on the array: serialise them.
//  * x and y must be 16-byte aligned device pointers on the current device.
//
// The partial of chunk c depends only on the data, not on the grid, and the
// last CTA to finish adds the partials in index order, so the result is the
// same from run to run and from device to device.
//
// This entry point has no counterpart in the reference.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "rx_device.cuh"
#include "rx_runtime.h"

namespace rx {
void set_last_error(int code, const std::string& msg);
void clear_last_error();
}  // namespace rx

namespace {

constexpr int kThreads = 256;
constexpr int64_t kChunk = 1 << 16;       // elements per partial
constexpr int kMaxPartials = 16384;       // => at most 2^30 elements
constexpr int64_t kMaxElems = kChunk * kMaxPartials;
constexpr int kTicketWord = kMaxPartials; // one counter after the partials

// Host code may name this array only as a handle for cudaGetSymbolAddress: the
// identifier is not a device address on the host side.
static __device__ __align__(256) unsigned int g_noalloc_scratch[kMaxPartials + 64];

__global__ void __launch_bounds__(kThreads) k_sinsum_noalloc(const float* __restrict__ x, const float* __restrict__ y, long long n, float* __restrict__ out,
                                                             unsigned int* __restrict__ scratch) {
  __shared__ uint32_t sm[kThreads / 32];
  __shared__ bool is_last;
  const long long nchunks = (n + kChunk - 1) / kChunk;
  for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const long long lo = c * kChunk;
    const long long hi = min(n, lo + kChunk);
    const long long n4 = (hi - lo) >> 2;
    const float4* x4 = (const float4*)(x + lo);
    const float4* y4 = (const float4*)(y + lo);
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    long long i = threadIdx.x;
    for (; i + 3 * kThreads < n4; i += 4 * kThreads) {
      float4 p0 = __ldcs(x4 + i), p1 = __ldcs(x4 + i + kThreads), p2 = __ldcs(x4 + i + 2 * kThreads), p3 = __ldcs(x4 + i + 3 * kThreads);
      float4 q0 = __ldcs(y4 + i), q1 = __ldcs(y4 + i + kThreads), q2 = __ldcs(y4 + i + 2 * kThreads), q3 = __ldcs(y4 + i + 3 * kThreads);
      a0 += sinf(p0.x) + q0.x; a1 += sinf(p0.y) + q0.y; a2 += sinf(p0.z) + q0.z; a3 += sinf(p0.w) + q0.w;
      a0 += sinf(p1.x) + q1.x; a1 += sinf(p1.y) + q1.y; a2 += sinf(p1.z) + q1.z; a3 += sinf(p1.w) + q1.w;
      a0 += sinf(p2.x) + q2.x; a1 += sinf(p2.y) + q2.y; a2 += sinf(p2.z) + q2.z; a3 += sinf(p2.w) + q2.w;
      a0 += sinf(p3.x) + q3.x; a1 += sinf(p3.y) + q3.y; a2 += sinf(p3.z) + q3.z; a3 += sinf(p3.w) + q3.w;
    }
    for (; i < n4; i += kThreads) {
      float4 p = __ldcs(x4 + i), q = __ldcs(y4 + i);
      a0 += sinf(p.x) + q.x; a1 += sinf(p.y) + q.y; a2 += sinf(p.z) + q.z; a3 += sinf(p.w) + q.w;
    }
    const long long tail = lo + n4 * 4 + threadIdx.x;  // at most 3 elements, last chunk only
    if (tail < hi) a0 += sinf(x[tail]) + y[tail];
    uint32_t r = rx::block_red<kThreads>(rx::R_FADD, rx::f2u((a0 + a1) + (a2 + a3)), sm);
    if (threadIdx.x == 0) scratch[c] = r;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned t = atomicAdd(&scratch[kTicketWord], 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float acc = 0.f;
  for (long long c = threadIdx.x; c < nchunks; c += kThreads) acc += rx::u2f(__ldcg(scratch + c));
  uint32_t total = rx::block_red<kThreads>(rx::R_FADD, rx::f2u(acc), sm);
  if (threadIdx.x == 0) {
    *out = rx::u2f(total);
    scratch[kTicketWord] = 0;
  }
}

struct PerDevice {
  bool ready = false;
  unsigned int* scratch = nullptr;
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;

}  // namespace

extern "C" int RxSinSumAddNoAlloc(const float* x_dev, const float* y_dev, int64_t n, float* out_dev, void* stream) {
  rx::clear_last_error();
  if (n < 0 || !out_dev || (n > 0 && (!x_dev || !y_dev))) {
    rx::set_last_error(RX_ERR_ARG, "RxSinSumAddNoAlloc: null pointer or negative length");
    return RX_ERR_ARG;
  }
  if (n > kMaxElems) {
    rx::set_last_error(RX_ERR_TOO_LARGE, "RxSinSumAddNoAlloc: n = " + std::to_string(n) + " exceeds the " + std::to_string(kMaxElems) +
                                             " elements (2^30) that the fixed scratch array supports");
    return RX_ERR_TOO_LARGE;
  }
  if (((uintptr_t)x_dev | (uintptr_t)y_dev) & 15) {
    rx::set_last_error(RX_ERR_ARG, "RxSinSumAddNoAlloc: x and y must be 16-byte aligned");
    return RX_ERR_ARG;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    rx::set_last_error(RX_ERR_CUDA, std::string("RxSinSumAddNoAlloc: cudaGetDevice: ") + cudaGetErrorString(e));
    return RX_ERR_CUDA;
  }
  PerDevice pd;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev[dev].ready) {
      // once per device, with that device current: resolve the array's device address
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&g_dev[dev].sm_count, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) {
        rx::set_last_error(RX_ERR_CUDA, std::string("RxSinSumAddNoAlloc: set-up failed: ") + cudaGetErrorString(e));
        return RX_ERR_CUDA;
      }
      g_dev[dev].scratch = (unsigned int*)p;
      g_dev[dev].ready = true;
    }
    pd = g_dev[dev];
  }
  cudaStream_t s = (cudaStream_t)stream;
  // the finished-CTA counter must start at zero whatever an earlier (possibly failed) call left behind
  e = cudaMemsetAsync(pd.scratch + kTicketWord, 0, sizeof(unsigned int), s);
  if (e == cudaSuccess) {
    long long nchunks = (n + kChunk - 1) / kChunk;
    long long grid = nchunks < 1 ? 1 : nchunks;
    long long cap = (long long)pd.sm_count * 8;
    if (grid > cap) grid = cap;
    rx::note_foreign_launch();  // executions queued behind this on the same stream must not read early what it writes
    k_sinsum_noalloc<<<(unsigned)grid, kThreads, 0, s>>>(x_dev, y_dev, (long long)n, out_dev, pd.scratch);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    rx::set_last_error(RX_ERR_CUDA, std::string("RxSinSumAddNoAlloc: launch failed: ") + cudaGetErrorString(e));
    return RX_ERR_CUDA;
  }
  return RX_OK;
}
