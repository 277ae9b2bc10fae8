// Entry points that Reactant's compile path calls on every loaded executable and device besides the
// execute / buffer groups: the sharding getters and their OpSharding accessor family, the HLO-module getter,
// and the CUDA device property queries.  Names and argument order are those of deps/ReactantExtra/API.cpp
// (line numbers beside each function), so the Julia wrappers in src/xla/PJRT/LoadedExecutable.jl:34-60,
// src/xla/Sharding.jl:20-120 and src/xla/Device.jl:43-60 bind to them unchanged.
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../../include/rx_b200.h"
#include "rx_runtime.h"

namespace rx {
void set_last_error(int code, const std::string& msg);
void clear_last_error();
}  // namespace rx

// What the reference hands out as an xla::OpSharding*, reduced to the two cases a 1-D mesh produces: a value
// that every device holds in full (REPLICATED) and a value split into equal contiguous chunks along one tensor
// dimension, chunk i on mesh device i (OTHER with a tile assignment that is 1 everywhere except that dimension).
struct RxOpSharding {
  int32_t type = 0;                      // xla::OpSharding::Type: 0 REPLICATED, 3 OTHER (tiled)
  std::vector<int32_t> tile_dims;        // tile_assignment_dimensions, one entry per tensor dim
  std::vector<int32_t> tile_devices;     // tile_assignment_devices, row-major over tile_dims
};

namespace {
RxOpSharding* make_sharding(size_t rank, int sharded_dim, int64_t nparts) {
  auto* s = new RxOpSharding();
  if (sharded_dim < 0 || nparts <= 1) return s;
  s->type = 3;
  s->tile_dims.assign(rank, 1);
  s->tile_dims[sharded_dim] = (int32_t)nparts;
  for (int64_t d = 0; d < nparts; ++d) s->tile_devices.push_back((int32_t)d);
  return s;
}
void fill(RxExecutable* e, RxOpSharding** out, int32_t n, bool params) {
  rx::clear_last_error();
  if (!e || !out) {
    rx::set_last_error(RX_ERR_BAD_HANDLE, "null executable or output array");
    return;
  }
  const rx::Plan& p = *e->plan;
  const size_t have = params ? p.arg_types.size() : p.results.size();
  if ((size_t)n != have) {  // worded as API.cpp:1551-1555
    rx::set_last_error(RX_ERR_ARG, "Expected " + std::to_string(n) + " shardings, got " + std::to_string(have));
    return;
  }
  for (int32_t i = 0; i < n; ++i) {
    if (params) out[i] = make_sharding(p.arg_types[i].shape.size(), p.arg_sharded_dim[i], p.num_partitions);
    else out[i] = make_sharding(p.results[i].type.shape.size(), p.results[i].sharded_dim, p.num_partitions);
  }
}
template <class V>
void copy_out(const V& v, int32_t* dst) {
  for (size_t i = 0; i < v.size(); ++i) dst[i] = v[i];
}
}  // namespace

extern "C" {

// API.cpp:1538-1583
void PjRtLoadedExecutableGetParameterShardings(RxExecutable* exec, RxOpSharding** op_shardings, int32_t num_op_shardings) { fill(exec, op_shardings, num_op_shardings, true); }
void PjRtLoadedExecutableGetOuputShardings(RxExecutable* exec, RxOpSharding** op_shardings, int32_t num_op_shardings) { fill(exec, op_shardings, num_op_shardings, false); }

// API.cpp:2459-2590
void free_op_sharding(RxOpSharding* s) { delete s; }
int32_t op_sharding_to_op_sharding_type(RxOpSharding* s) { return s->type; }
int32_t op_sharding_to_shard_group_type(RxOpSharding*) { return 0; }
int32_t op_sharding_to_shard_group_id(RxOpSharding*) { return 0; }
uint8_t op_sharding_is_shard_group(RxOpSharding*) { return 0; }
uint8_t op_sharding_replicate_on_last_tile_dim(RxOpSharding*) { return 0; }
uint8_t op_sharding_has_last_tile_dims(RxOpSharding*) { return 0; }
int32_t op_sharding_last_tile_dims_size(RxOpSharding*) { return 0; }
void op_sharding_last_tile_dims(RxOpSharding*, int32_t*) {}
uint8_t op_sharding_has_iota_reshape_dims(RxOpSharding*) { return 0; }
int32_t op_sharding_iota_reshape_dims_size(RxOpSharding*) { return 0; }
void op_sharding_iota_reshape_dims(RxOpSharding*, int32_t*) {}
uint8_t op_sharding_has_iota_transpose_perm(RxOpSharding*) { return 0; }
int32_t op_sharding_iota_transpose_perm_size(RxOpSharding*) { return 0; }
void op_sharding_iota_transpose_perm(RxOpSharding*, int32_t*) {}
uint8_t op_sharding_has_tile_assignment_dimensions(RxOpSharding* s) { return !s->tile_dims.empty(); }
int32_t op_sharding_tile_assignment_dimensions_size(RxOpSharding* s) { return (int32_t)s->tile_dims.size(); }
void op_sharding_tile_assignment_dimensions(RxOpSharding* s, int32_t* out) { copy_out(s->tile_dims, out); }
uint8_t op_sharding_has_tile_assignment_devices(RxOpSharding* s) { return !s->tile_devices.empty(); }
int32_t op_sharding_tile_assignment_devices_size(RxOpSharding* s) { return (int32_t)s->tile_devices.size(); }
void op_sharding_tile_assignment_devices(RxOpSharding* s, int32_t* out) { copy_out(s->tile_devices, out); }

// API.cpp:2064-2071.  There is no HLO behind an executable of this engine (RxExecutableDescribe returns the
// launch plan instead); Reactant's compile path calls this unconditionally (src/compiler/Compiler.jl:1360), so
// it answers "zero modules" rather than failing.
void PjRtLoadedExecutableGetHloModules(RxExecutable*, void** hlo_modules, int32_t* nmodules) {
  (void)hlo_modules;
  if (nmodules) *nmodules = 0;
}

// API.cpp:864-930
int32_t ReactantCudaDriverGetVersion(void) {
  int v = 0;
  if (cudaDriverGetVersion(&v) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return v;
}
static int32_t device_attr(cudaDeviceAttr a) {
  int v = 0;
  if (cudaDeviceGetAttribute(&v, a, 0) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return v;
}
int32_t ReactantCudaDeviceGetComputeCapalilityMajor(void) { return device_attr(cudaDevAttrComputeCapabilityMajor); }
int32_t ReactantCudaDeviceGetComputeCapalilityMinor(void) { return device_attr(cudaDevAttrComputeCapabilityMinor); }
int32_t ReactantCudaDeviceGetWarpSizeInThreads(void) { return device_attr(cudaDevAttrWarpSize); }
void ReactantCudaDeviceGetProperties(RxDeviceProperties* out, int32_t device_id) {
  rx::clear_last_error();
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, device_id);
  if (e != cudaSuccess) {
    cudaGetLastError();
    rx::set_last_error(RX_ERR_CUDA, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    return;
  }
  out->totalGlobalMem = p.totalGlobalMem;
  out->sharedMemPerBlock = p.sharedMemPerBlock;
  out->regsPerBlock = p.regsPerBlock;
  out->warpSize = p.warpSize;
  out->maxThreadsPerBlock = p.maxThreadsPerBlock;
  for (int k = 0; k < 3; ++k) {
    out->maxThreadsDim[k] = p.maxThreadsDim[k];
    out->maxGridSize[k] = p.maxGridSize[k];
  }
  out->totalConstMem = p.totalConstMem;
  out->major = p.major;
  out->minor = p.minor;
  out->multiProcessorCount = p.multiProcessorCount;
  out->canMapHostMemory = p.canMapHostMemory;
  out->l2CacheSize = p.l2CacheSize;
  out->maxThreadsPerMultiProcessor = p.maxThreadsPerMultiProcessor;
}

}  // extern "C"
