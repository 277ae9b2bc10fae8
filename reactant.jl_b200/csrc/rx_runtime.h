// Runtime objects behind the C ABI: client, devices with their stream-ordered
// memory pools, reference-counted buffer storage, futures and executables.
// They stand in for the PjRt objects Reactant's wrapper structs hold
// (src/xla/PJRT/{Client,Device,Buffer,Future,LoadedExecutable}.jl).
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "rx_ir.h"
#include "rx_kernels.h"
#include "rx_plan.h"

struct RxClient;

constexpr int kMaxRanks = 32;
// Layout of a device's mailbox allocation: 2 x kMaxRanks 64-bit all-reduce slots, then (at kHaloFlagsOffset bytes) the
// halo-exchange flags [parity][direction] as 32-bit sequence numbers, then (at kHaloWindowOffset bytes) the halo
// windows [parity][direction][kHaloMaxRows][kHaloMaxCols] of floats.  Direction 0 = rows arriving from the device
// above (smaller rank), 1 = from the device below.
constexpr int kHaloMaxRows = 2;
constexpr int kHaloMaxCols = 16384;
constexpr size_t kHaloFlagsOffset = sizeof(unsigned long long) * 2 * kMaxRanks;
constexpr size_t kHaloWindowOffset = kHaloFlagsOffset + 512;
constexpr size_t kMailboxBytes = kHaloWindowOffset + sizeof(float) * 2 * 2 * kHaloMaxRows * kHaloMaxCols;

// Peer mailboxes for the NVLink all-reduce: slot [parity][rank] of every device.
struct MailTable {
  unsigned long long* peer[kMaxRanks];
};

struct RxDevice : std::enable_shared_from_this<RxDevice> {
  RxClient* client = nullptr;
  std::atomic<bool> closed{false};  // client freed: late buffer finalizers free straight to the driver
  int ordinal = 0;    // CUDA device ordinal
  int local_id = 0;   // index among this process's devices
  int global_id = 0;  // index in the mesh
  bool addressable = true;
  cudaStream_t stream = nullptr;
  cudaStream_t comm_stream = nullptr;  // vector all-reduces run here, ordered against `stream` by events
  int sm_count = 148;
  std::string kind;   // device name and compute capability, from cudaGetDeviceProperties
  size_t total_mem = 0;
  // One execution at a time enqueues on a device: launches of different host threads must not interleave (they
  // share the reduction scratch in stream order) and the launch-side tables below are not otherwise protected.
  std::mutex exec_mu;
  // memory pool (exact-size free lists, stream ordered on `stream`)
  std::mutex mu;
  std::map<size_t, std::vector<void*>> pool;
  int64_t num_allocs = 0, bytes_in_use = 0, peak_bytes_in_use = 0, largest_alloc = 0, bytes_limit = 0, pool_bytes = 0, peak_pool_bytes = 0;
  uint32_t* scratch = nullptr;
  size_t scratch_words = 0;
  uint64_t launches = 0;
  // Storage written by the most recent launch on `stream` (and by copies queued since): a kernel launched with
  // programmatic stream serialization may read its operands early only if none of them is in this list.
  std::vector<const void*> last_writes;
  uint64_t foreign_seen = 0;  // value of rx::foreign_launches() when last_writes was last brought up to date
  bool last_gemm_tc = false, last_stencil_tma = false;  // which kernel family the last such step used
  // profiling
  bool profiling = false;
  struct Span { std::string kind; cudaEvent_t a, b; };
  std::vector<Span> spans;
  std::map<std::string, std::pair<int64_t, double>> prof;
  void* flush_buf = nullptr;
  size_t flush_bytes = 0;
  // NVLink mailbox
  unsigned long long* mailbox = nullptr;  // [2][kMaxRanks]
  int* status = nullptr;                  // device-visible status word (pinned host memory)
  MailTable mail{};
  bool mail_own[kMaxRanks] = {};          // entry maps one of this process's own mailboxes (no IPC mapping to close)
  bool mail_ready = false;
  std::map<const void*, std::vector<uint8_t>> tmaps;  // tensor-map cache keyed by base pointer

  void* alloc(size_t bytes);
  void release(void* p, size_t bytes);
  void trim();
  rx::LaunchCtx ctx() {
    rx::LaunchCtx c;
    c.stream = stream;
    c.sm_count = sm_count;
    c.device = ordinal;
    c.scratch = scratch;
    c.scratch_words = scratch_words;
    c.launches = &launches;
    return c;
  }
};

// Device memory block.  Keeps its device object alive: handles may be finalized
// (from a garbage collector, on any thread) after the client itself was freed.
struct Storage {
  RxDevice* dev;
  std::shared_ptr<RxDevice> keep;
  void* ptr;
  size_t bytes;
  // Set when the last writer of this block ran on the device's communication stream (an all-reduce that was still
  // in flight when the execution that produced it returned): whoever touches the block next on the compute stream
  // -- the next execution, a copy to the host, or the release of the memory -- waits for this event first.
  std::mutex pending_mu;
  cudaEvent_t pending = nullptr;
  Storage(RxDevice* d, void* p, size_t b) : dev(d), keep(d->shared_from_this()), ptr(p), bytes(b) {}
  void make_ready() {  // call with the owning device current
    std::lock_guard<std::mutex> g(pending_mu);
    if (!pending) return;
    if (dev->stream) cudaStreamWaitEvent(dev->stream, pending, 0);
    cudaEventDestroy(pending);
    pending = nullptr;
  }
  ~Storage() {
    if (pending) {
      int cur = 0;
      cudaGetDevice(&cur);
      cudaSetDevice(dev->ordinal);
      make_ready();  // the pool hands the block out again in compute-stream order
      cudaSetDevice(cur);
    }
    dev->release(ptr, bytes);
  }
};

struct RxBuffer {
  std::shared_ptr<Storage> st;
  rx::DT dt;
  std::vector<int64_t> dims;
  RxDevice* dev;
  std::atomic<bool> donated{false};
  size_t bytes() const {
    size_t n = rx::dt_size(dt);
    for (auto d : dims) n *= (size_t)d;
    return n;
  }
};

namespace rx {
// Kernels that this library's other entry points launch on caller-supplied streams (RxSinSumAddNoAlloc) are not
// tracked per device; each bumps this counter, and an execution that sees it moved assumes nothing about what
// the kernel in front of it wrote.
uint64_t foreign_launches();
void note_foreign_launch();
}  // namespace rx

struct EventState {
  // A failure found when this execution was awaited (a bounded device-side wait that ran out): kept here so that
  // every future of the execution reports it, not only the first one to look at the device's status word.
  std::mutex error_mu;
  int error_code = 0;
  std::string error;
  // Completion of the execution on the device's compute stream.  The event is recorded only when somebody asks
  // (FutureIsReady / FutureAwait): most futures are freed unasked, and an event record between two launches would
  // keep the second from starting under the first (programmatic dependent launch).  Recording late is safe: the
  // event then also covers whatever was queued after the execution, so "ready" is never reported too early.
  std::mutex ev_mu;
  cudaEvent_t ev = nullptr;
  RxDevice* dev = nullptr;
  std::shared_ptr<RxDevice> keep;
  cudaEvent_t event();  // records on first use; nullptr once the device's client has been freed (everything has drained)
  ~EventState();
};

struct RxFuture {
  std::shared_ptr<EventState> state;
};

struct RxEvent {
  cudaEvent_t ev = nullptr;
  RxDevice* dev = nullptr;
  std::shared_ptr<RxDevice> keep;
};

struct RxExecutable {
  RxClient* client = nullptr;
  std::shared_ptr<const rx::Plan> plan;  // shared with the process-wide plan cache
  std::mutex mu;
  std::map<int, std::map<int, std::shared_ptr<Storage>>> consts;  // [local device][slot]
};

struct RxClient {
  int node_id = 0, num_nodes = 1;
  std::vector<std::shared_ptr<RxDevice>> devices;     // addressable devices
  std::vector<std::shared_ptr<RxDevice>> remote;      // placeholders for other processes' devices
  std::mutex mu;
  // NCCL
  void* nccl_comms[kMaxRanks] = {};
  bool nccl_ready = false;
  bool peers_enabled = false;
  uint32_t epoch = 0;       // all-reduce sequence number (same on every rank)
  uint32_t halo_epoch = 0;  // halo-exchange sequence number (same on every rank)
  int allreduce_mode = 0;   // 0 auto, 1 nccl, 2 mailbox
  // How long a kernel waits for a peer's word in an all-reduce mailbox before it gives up and reports
  // RX_ERR_PEER_TIMEOUT.  Ranks that are separate processes can be far apart in host time (a cold compile cache, a
  // garbage collection, data loading), so they get several seconds; devices driven by one process are launched
  // back to back.  RX_PEER_WAIT_MS or RxClientSetPeerWaitMs override the default.
  int64_t peer_wait_ms = 1000;
  long long peer_wait_polls() const { return (long long)peer_wait_ms * 4000; }  // one poll is about 0.25 us
  int n_global() const { return (int)devices.size() * num_nodes; }
};
