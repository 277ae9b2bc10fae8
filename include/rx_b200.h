/* rx_b200.h -- C ABI of librx_b200.so, the B200-native execution engine that
 * takes the place of Reactant.jl's PJRT runtime shim for the fused map-reduce /
 * stencil / dot_general hot path.
 *
 * The first group of entry points keeps the names, argument order and meaning
 * of the `extern "C"` functions Reactant's PJRT wrapper structs call today
 * (deps/ReactantExtra/API.cpp; the Julia callers live in src/xla/PJRT/*.jl), so
 * that src/xla/PJRT/{Client,Device,Buffer,Future,LoadedExecutable}.jl bind to
 * this library with no change in their ccall sites.  Every handle is opaque.
 * Citations are file:line in the Reactant.jl tree.
 *
 * Conventions
 *  - Shapes cross the boundary as row-major dims; a Julia column-major array of
 *    size (d1..dn) is passed with dims (dn..d1) and unchanged bytes
 *    (src/xla/PJRT/Buffer.jl:9-17).
 *  - Element types use XLA primitive-type codes (src/xla/Utils.jl:18-40):
 *    PRED 1, S8..S64 2-5, U8..U64 6-9, F16 10, F32 11, F64 12, BF16 16.
 *  - Errors: runtime failures call `ReactantThrowError(msg)` when the host has
 *    installed it (src/xla/XLA.jl:203-204; the Julia callback throws, so control
 *    may not return).  When it is NULL the message is kept per thread and
 *    `RxLastError()` returns it; the failing call then returns NULL / does
 *    nothing.  Factories additionally set `*error` to a malloc'd message.
 *  - Nothing here falls back to a CPU or library implementation: an op outside
 *    the supported set fails compilation with a message naming the op.
 */
#ifndef RX_B200_H
#define RX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct RxClient RxClient;         /* stands in for xla::PjRtClient            */
typedef struct RxDevice RxDevice;         /* stands in for xla::PjRtDevice            */
typedef struct RxBuffer RxBuffer;         /* stands in for xla::PjRtBuffer            */
typedef struct RxFuture RxFuture;         /* stands in for xla::Future<>              */
typedef struct RxExecutable RxExecutable; /* stands in for xla::PjRtLoadedExecutable  */
typedef struct RxEvent RxEvent;
typedef struct RxOpSharding RxOpSharding; /* stands in for xla::OpSharding                */

/* ---- errors ------------------------------------------------------------- */
/* API.cpp:262.  Host-installed callback; NULL by default. */
extern void (*ReactantThrowError)(const char*);
/* No counterpart in the reference: errno-style access for hosts that cannot
 * install a throwing callback (ctypes, C tests).  Returns "" when the last call
 * on this thread succeeded.  RxLastErrorCode returns one of RX_ERR_*. */
const char* RxLastError(void);
int RxLastErrorCode(void);
void RxClearError(void);
enum {
  RX_OK = 0, RX_ERR_PARSE = 1, RX_ERR_UNSUPPORTED_OP = 2, RX_ERR_UNSUPPORTED_TYPE = 3,
  RX_ERR_PLAN = 4, RX_ERR_BAD_HANDLE = 5, RX_ERR_SHAPE = 6, RX_ERR_DONATED = 7,
  RX_ERR_CUDA = 8, RX_ERR_NO_DEVICE = 9, RX_ERR_PEER_TIMEOUT = 10, RX_ERR_NCCL = 11,
  RX_ERR_ARG = 12, RX_ERR_TOO_LARGE = 13
};

/* ---- client (API.cpp:528-582, 688-732, 1254) ------------------------------ */
/* One client per process.  `allowed_devices` restricts the CUDA ordinals used
 * (NULL = all visible).  With num_nodes > 1 the process is rank `node_id` of a
 * multi-process mesh: each process addresses only its own devices and
 * RxClientInitCollectives must be called before a sharded executable runs.
 * memory_fraction caps the bytes the device pools may hold; preallocate and
 * distributed_runtime_client are accepted for signature compatibility. */
RxClient* MakeGPUClient(int node_id, int num_nodes, int64_t* allowed_devices, int64_t num_allowed_devices,
                        double memory_fraction, uint8_t preallocate, const char* platform_name,
                        const char** error, void* distributed_runtime_client);
void FreeClient(RxClient* client);
int ClientNumDevices(RxClient* client);
int ClientNumAddressableDevices(RxClient* client);
int ClientProcessIndex(RxClient* client);
RxDevice* ClientGetDevice(RxClient* client, int device_id);
RxDevice* ClientGetAddressableDevice(RxClient* client, int device_id);
void ClientGetDevices(RxClient* client, RxDevice** out);
void ClientGetAddressableDevices(RxClient* client, RxDevice** out);
const char* ClientGetPlatformName(RxClient* client); /* "cuda"; caller frees (src/xla/Utils.jl:51-55) */

/* ---- device (API.cpp:714, 734-765, 803, 1256-1266, 3296) ------------------ */
RxClient* DeviceToClient(RxDevice* device);
int64_t PjRtDeviceGetLocalDeviceId(RxDevice* device);
int64_t PjRtDeviceGetGlobalDeviceId(RxDevice* device);
int64_t PjRtDeviceGetLocalHardwareId(RxDevice* device);
const char* DeviceGetKind(RxDevice* device); /* caller frees */
uint8_t pjrt_device_is_addressable(RxDevice* device);
typedef struct {
  int64_t num_allocs, bytes_in_use, peak_bytes_in_use, largest_alloc_size, bytes_limit, bytes_reserved,
      peak_bytes_reserved, bytes_reservable_limit, largest_free_block_bytes, pool_bytes, peak_pool_bytes;
} JLAllocatorStats; /* API.cpp:734-746 */
void PjRtDeviceGetAllocatorStats(RxDevice* device, JLAllocatorStats* stats);

/* CUDA device queries (API.cpp:841-930; callers src/xla/Device.jl:43-60, src/compiler/Compiler.jl:154,336). */
typedef struct {
  size_t totalGlobalMem, sharedMemPerBlock;
  int regsPerBlock, warpSize, maxThreadsPerBlock, maxThreadsDim[3], maxGridSize[3];
  size_t totalConstMem;
  int major, minor, multiProcessorCount, canMapHostMemory, l2CacheSize, maxThreadsPerMultiProcessor;
} RxDeviceProperties; /* layout of DeviceProperties, API.cpp:841-856 */
void ReactantCudaDeviceGetProperties(RxDeviceProperties* props, int32_t device_id);
int32_t ReactantCudaDriverGetVersion(void);
int32_t ReactantCudaDeviceGetComputeCapalilityMajor(void);
int32_t ReactantCudaDeviceGetComputeCapalilityMinor(void);
int32_t ReactantCudaDeviceGetWarpSizeInThreads(void);

/* ---- buffers (API.cpp:781-801, 1075-1098, 1162-1177, 1230-1252) ----------- */
/* H2D upload.  The host memory may be reused as soon as the call returns. */
RxBuffer* ArrayFromHostBuffer(RxClient* client, void* data, uint64_t ptype, size_t ndim, const int64_t* dims, RxDevice* device);
RxBuffer* UninitPJRTBuffer(RxClient* client, RxDevice* device, uint64_t ptype, uint64_t ndim, uint64_t* dims);
/* Thread-safe; may be called from a finalizer while work that reads or writes
 * the buffer is still queued (storage is reference counted and stream ordered). */
void PjRtBufferFree(RxBuffer* buffer);
const int64_t* BufferShape(RxBuffer* buffer); /* borrowed */
int64_t BufferNDimensions(RxBuffer* buffer);
int BufferPrimitiveType(RxBuffer* buffer);
RxDevice* BufferToDevice(RxBuffer* buffer);
RxClient* BufferToClient(RxBuffer* buffer);
uint8_t BufferOnCPU(RxBuffer* buffer); /* always 0 */
/* Blocking D2H into `dst` (row-major over the buffer's dims).  A failed copy
 * reports an error and never returns garbage silently. */
void BufferToHost(RxBuffer* buffer, void* dst);
void* UnsafeBufferPointer(RxBuffer* buffer);
RxBuffer* CopyBufferToDevice(RxBuffer* buffer, RxDevice* dst_device);
/* Partial host<->device copies at a byte offset (API.cpp:1100, 1179). */
void CopyToBuffer(RxClient* client, RxBuffer* buffer, void* data, size_t offset, size_t size, RxBuffer** bufferP);
void CopyFromBuffer(RxClient* client, RxBuffer* buffer, void* data, size_t offset, size_t size, RxBuffer** bufferP);

/* ---- futures (API.cpp:1357-1373) ------------------------------------------ */
void FreeFuture(RxFuture* future);
uint8_t FutureIsReady(RxFuture* future);
void FutureAwait(RxFuture* future); /* reports a failed execution as an error */

/* ---- compile (API.cpp:1482-1536, 777, 807, 1730-1736) ---------------------- */
/* Takes the place of ClientCompileWithProto(client, MlirModule, opts, n)
 * (API.cpp:1528-1536): the module arrives as MLIR text (`string(mod)` on the
 * Julia side) instead of an in-memory MlirModule, because this library does not
 * link MLIR.  `compile_options`/`n` are accepted and ignored (XLA option proto).
 * Returns NULL and reports an error naming the op when the module contains
 * anything outside the supported subset. */
RxExecutable* ClientCompileText(RxClient* client, const char* mlir_text, size_t text_len,
                                const char* compile_options, size_t compile_options_len);
void ExecutableFree(RxExecutable* exec);
RxClient* PjRtLoadedExecutableGetClient(RxExecutable* exec);
int PjRtLoadedExecutableNumReplicas(RxExecutable* exec);
int PjRtLoadedExecutableNumPartitions(RxExecutable* exec);
/* Takes the place of PjRtLoadedExecutableGetParameterShardings /
 * GetOuputShardings + the op_sharding_* accessors (API.cpp:1538-1583,
 * 2459-2590): for parameter / result `index`, writes the tensor dim that is
 * split over the mesh axis, or -1 when the value is replicated. */
int RxExecutableNumParameters(RxExecutable* exec);
int RxExecutableNumResults(RxExecutable* exec);
int RxExecutableParameterShardedDim(RxExecutable* exec, int index);
int RxExecutableResultShardedDim(RxExecutable* exec, int index);
/* The `tf.aliasing_output` of parameter `index` (src/compiler/Compiler.jl:1103-1127):
 * the result whose storage may reuse this argument's when it is donated; -1 = none. */
int RxExecutableParameterAlias(RxExecutable* exec, int index);
/* The reference's own sharding getters (API.cpp:1538-1583; callers src/xla/PJRT/LoadedExecutable.jl:34-48,
 * asserted against the traced shardings at src/compiler/Compiler.jl:1416 and src/compiler/Codegen.jl:838,1400).
 * `num_op_shardings` must equal the number of parameters / results; each out[i] is a fresh object the caller
 * releases with free_op_sharding.  A replicated value reports type 0 (REPLICATED); a value split along one
 * tensor dimension over the N devices of the mesh reports type 3 (OTHER) with tile_assignment_dimensions equal to
 * 1 everywhere except N at that dimension and tile_assignment_devices 0..N-1 -- what XLA reports for the
 * NamedSharding of a 1-D mesh. */
void PjRtLoadedExecutableGetParameterShardings(RxExecutable* exec, RxOpSharding** op_shardings, int32_t num_op_shardings);
void PjRtLoadedExecutableGetOuputShardings(RxExecutable* exec, RxOpSharding** op_shardings, int32_t num_op_shardings);
/* The OpSharding accessor family (API.cpp:2459-2590; callers src/xla/Sharding.jl:20-120).  The iota, last-tile
 * and shard-group forms never occur for a 1-D mesh and report "absent". */
void free_op_sharding(RxOpSharding* op_sharding);
int32_t op_sharding_to_op_sharding_type(RxOpSharding* op_sharding);
int32_t op_sharding_to_shard_group_type(RxOpSharding* op_sharding);
int32_t op_sharding_to_shard_group_id(RxOpSharding* op_sharding);
uint8_t op_sharding_is_shard_group(RxOpSharding* op_sharding);
uint8_t op_sharding_replicate_on_last_tile_dim(RxOpSharding* op_sharding);
uint8_t op_sharding_has_last_tile_dims(RxOpSharding* op_sharding);
int32_t op_sharding_last_tile_dims_size(RxOpSharding* op_sharding);
void op_sharding_last_tile_dims(RxOpSharding* op_sharding, int32_t* last_tile_dims);
uint8_t op_sharding_has_iota_reshape_dims(RxOpSharding* op_sharding);
int32_t op_sharding_iota_reshape_dims_size(RxOpSharding* op_sharding);
void op_sharding_iota_reshape_dims(RxOpSharding* op_sharding, int32_t* iota_reshape_dims);
uint8_t op_sharding_has_iota_transpose_perm(RxOpSharding* op_sharding);
int32_t op_sharding_iota_transpose_perm_size(RxOpSharding* op_sharding);
void op_sharding_iota_transpose_perm(RxOpSharding* op_sharding, int32_t* iota_transpose_perm);
uint8_t op_sharding_has_tile_assignment_dimensions(RxOpSharding* op_sharding);
int32_t op_sharding_tile_assignment_dimensions_size(RxOpSharding* op_sharding);
void op_sharding_tile_assignment_dimensions(RxOpSharding* op_sharding, int32_t* tile_assignment_dimensions);
uint8_t op_sharding_has_tile_assignment_devices(RxOpSharding* op_sharding);
int32_t op_sharding_tile_assignment_devices_size(RxOpSharding* op_sharding);
void op_sharding_tile_assignment_devices(RxOpSharding* op_sharding, int32_t* tile_assignment_devices);
/* API.cpp:2064-2071; called unconditionally after every compile (src/compiler/Compiler.jl:1360,
 * src/xla/PJRT/LoadedExecutable.jl:50-60).  This engine keeps no HLO: *nmodules is set to 0 and nothing is
 * written to hlo_modules (RxExecutableDescribe is the way to look at what was built). */
void PjRtLoadedExecutableGetHloModules(RxExecutable* exec, void** hlo_modules, int32_t* nmodules);
/* JSON description of the launch plan (fusion groups, chosen kernels); the
 * analogue of dumping the compiled HLO (PjRtLoadedExecutableGetHloModules,
 * src/xla/PJRT/LoadedExecutable.jl:50-60).  Caller frees. */
const char* RxExecutableDescribe(RxExecutable* exec);
/* Parse + plan without a client or a GPU: returns the same JSON (caller frees)
 * or NULL with the error set.  Used to validate modules on machines without a
 * device. */
const char* RxPlanDescribe(const char* mlir_text, size_t text_len);
/* ClientCompileText keeps the plan of every module it has seen (keyed by the
 * module text) and hands it out again when the same module is compiled once
 * more -- what src/PersistentCompileCache.jl does for XLA executables, in
 * memory.  This returns how many compilations were served from that cache. */
int64_t RxPlanCacheHits(void);

/* ---- run-time specialisation of fused chains ---------------------------------
 * Fusion groups whose launch covers at least `min_elems` elements (default 2^20)
 * run a kernel compiled for that chain with NVRTC on first use (cached for the
 * life of the process); smaller launches, and every launch when NVRTC cannot be
 * loaded, run the same kernel skeleton over a bytecode interpreter on the GPU.
 * Both produce the same bits.  The counterpart in the reference is XLA's own
 * code generation inside ClientCompile (API.cpp:1482-1507); these three entry
 * points have no counterpart of their own.
 * RxChainSpecialiser: set the threshold; a negative value switches it off.
 * RxChainSpecialiserStats: out5 = {kernels compiled, in-memory cache hits,
 *   compile failures, 1 if NVRTC or the driver entry points are unavailable,
 *   kernels read from the on-disk cache}.  With RX_JIT_CACHE_DIR set to an
 *   existing directory compiled chains are kept there across processes (the
 *   counterpart of src/PersistentCompileCache.jl for this engine's only
 *   compiled artefact).
 * RxPlanSpecialiseCheck: plan a module and compile every chain in it for each
 *   kernel family it could run in, without a device; returns a JSON list
 *   (caller frees) or NULL with the error set to the compiler log. */
void RxChainSpecialiser(int64_t min_elems);
void RxChainSpecialiserStats(int64_t* out5);
const char* RxPlanSpecialiseCheck(const char* mlir_text, size_t text_len);

/* ---- execute (API.cpp:1585-1630, 1653-1728) --------------------------------- */
/* Single-device launch.  `is_arg_donatable[i]` != 0 allows argument i's storage
 * to be reused for the output it aliases.  Writes `num_results` fresh buffer
 * handles; `*futures` is set to 1 and `future_results[i]` receive one heap
 * future per result.  Asynchronous: returns after enqueueing. */
void XLAExecuteSharded(RxExecutable* exec, int num_args, RxBuffer** op_args, RxDevice* device,
                       uint8_t* is_arg_donatable, int num_results, RxBuffer** op_results,
                       uint8_t* futures, RxFuture** future_results);
/* Multi-device launch over the client's addressable devices: op_args is laid
 * out [device][arg], op_results [device][result]; is_arg_donatable is per arg. */
void XLAExecute(RxExecutable* exec, int op_args_len, RxBuffer** op_args, uint8_t* is_arg_donatable,
                int num_results, RxBuffer** op_results, uint8_t* futures, RxFuture** future_results);

/* ---- living beside another runtime (no counterpart in the reference) ----------
 * A Julia session that loads this engine still has Reactant's XLA CPU client, and both answer to the same
 * entry-point names.  RxOwns tells whether `handle` (client, device, buffer, future or executable) was handed
 * out by this library and has not been freed; the binding routes every call by it.  The two execute entry
 * points can be reached without passing through the binding (Reactant's generated thunks call them by symbol,
 * src/xla/PJRT/LoadedExecutable.jl:85-246): once the host has registered the other runtime's functions here, an
 * executable that is not this library's is passed on to them untouched.  That is routing between two
 * runtimes, not a fallback: a module this engine cannot run still fails at compile time. */
uint8_t RxOwns(const void* handle);
void RxSetForeignExecute(void* xla_execute_sharded, void* xla_execute);

/* ---- allocation-free entry point (no counterpart in the reference) -----------
 * out_dev[0] = sum(sin(x_dev[i]) + y_dev[i], i < n), computed on `stream`
 * (a cudaStream_t; NULL = the default stream) of the current device, for hosts
 * that cannot let this library allocate device memory: ones that have given all
 * of it to their own arena, ones that cannot take the device-wide stall of
 * cudaMalloc / cudaFree inside a latency-critical loop, ones that account for
 * every byte themselves.  It calls no cudaMalloc, cudaFree or any allocating
 * routine: x_dev, y_dev (16-byte aligned) and out_dev are the caller's device
 * pointers, and the cross-CTA scratch is a fixed 64 KiB + 256 B array inside the
 * library image (resident on every GPU that loads the library until exit).
 * Limits and rules: n <= 2^30 elements, larger n returns RX_ERR_TOO_LARGE and
 * launches nothing; the first call on each device resolves the array's address
 * and should be made outside any stream capture; every call shares the array,
 * so calls whose kernels could overlap on one GPU must be serialised by the
 * caller.  Returns RX_OK or an RX_ERR_* code (message in RxLastError()).  The
 * result is deterministic and independent of the GPU's SM count. */
int RxSinSumAddNoAlloc(const float* x_dev, const float* y_dev, int64_t n, float* out_dev, void* stream);

/* ---- collectives bootstrap (takes the place of the NCCL clique setup XLA
 * performs through its distributed KV store, API.cpp:536-547, 2896-3050) ------ */
/* Rank 0 obtains an id (128 bytes), the host distributes it to every process,
 * and every process calls RxClientInitCollectives.  For a single-process client
 * both steps are done internally on first use and these calls are optional. */
int RxCollectivesUniqueId(uint8_t* id128);
int RxClientInitCollectives(RxClient* client, const uint8_t* id128);
/* NVLink peer mailbox for the fused reduce + all-reduce kernel.  Multi-process:
 * each process exports one 64-byte handle per local device; the host gathers
 * all of them in global device order and passes the table to
 * RxClientOpenMailboxes.  Single-process clients set this up internally. */
int RxClientMailboxHandle(RxClient* client, int local_device, uint8_t* handle64);
/* Every wait for a peer inside a kernel is bounded.  This sets the bound for the client's all-reduces, in
 * milliseconds (1..60000); when it runs out the kernel returns, the rank keeps its own partial value and the
 * next FutureAwait / BufferToHost reports RX_ERR_PEER_TIMEOUT.  Defaults: 1000 ms when one process drives all
 * devices, 8000 ms when the ranks are separate processes; the environment variable RX_PEER_WAIT_MS, read when
 * the client is made, overrides both. */
int RxClientSetPeerWaitMs(RxClient* client, int64_t milliseconds);
int RxClientOpenMailboxes(RxClient* client, const uint8_t* handles, int n_global_devices);

/* ---- page-locked host memory (no counterpart in the reference, where XLA stages
 * pageable host arrays itself inside BufferFromHostBuffer, API.cpp:1093-1095) -----
 * ArrayFromHostBuffer / BufferToHost move data at the full PCIe rate only from
 * page-locked memory; a host that wants that rate keeps its arrays in blocks
 * obtained here.  RxHostAlloc returns NULL and reports an error when the memory
 * cannot be locked; RxHostFree accepts NULL. */
void* RxHostAlloc(size_t bytes);
void RxHostFree(void* ptr);

/* ---- measurement helpers (no counterpart in the reference, which times with
 * the XLA profiler, src/Profiler.jl:109-184) --------------------------------- */
RxEvent* RxEventRecord(RxDevice* device);           /* record on the device's stream */
void RxEventSynchronize(RxEvent* ev);
float RxEventElapsedMs(RxEvent* start, RxEvent* stop);
void RxEventFree(RxEvent* ev);
void RxDeviceSynchronize(RxDevice* device);
/* Gradient all-reduces run on a second stream per device and may still be in flight when an execution
 * returns (its futures and the next user of each result wait for them).  This makes the device's compute
 * stream wait for everything queued on that stream so far, so that an event recorded afterwards covers it. */
void RxDeviceJoinStreams(RxDevice* device);
uint64_t RxDeviceKernelLaunches(RxDevice* device);   /* kernels launched so far on this device */
/* When enabled, every step of every execute on this device is bracketed by
 * events; RxDeviceProfileJson returns {"<step kind>": {"launches": n, "ms": t}, ...}
 * accumulated since the last call (caller frees). */
void RxDeviceSetProfiling(RxDevice* device, int enabled);
const char* RxDeviceProfileJson(RxDevice* device);
void* RxDeviceStream(RxDevice* device);              /* the cudaStream_t all work of the device is ordered on */
/* Writes `bytes` bytes of a device buffer larger than L2 so that the next
 * kernel starts with a cold L2. */
void RxDeviceFlushL2(RxDevice* device);

#ifdef __cplusplus
}
#endif
#endif /* RX_B200_H */
