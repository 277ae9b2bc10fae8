// all_reduce(sum) over the 1-D mesh.
//
// Two transports:
//  * NCCL (ncclAllReduce on each device's stream), loaded with dlopen so that
//    single-GPU use needs no NCCL at all;
//  * an NVLink "mailbox" kernel for single-word payloads (the scalar of a
//    sharded full reduce): every rank stores {epoch, value} into its slot of
//    every peer's mailbox with one 64-bit store, then polls its own mailbox --
//    bounded -- and adds the N words in rank order, so all ranks produce the
//    same bits.  The data lands in the consumer's own memory first; nothing here
//    issues TMA or multicast loads from a peer.
//
// In the reference this collective is inserted and executed by XLA's SPMD
// partitioner and NCCL thunks (deps/ReactantExtra/API.cpp:1487-1497).
#include "rx_collective.h"
#include "rx_halo.cuh"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <string>

namespace rx {

namespace {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.lib) break;
    }
    if (!api.lib) return;
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.lib, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.lib, "ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.lib, "ncclCommDestroy");
    api.AllReduce = (decltype(api.AllReduce))dlsym(api.lib, "ncclAllReduce");
    api.GroupStart = (decltype(api.GroupStart))dlsym(api.lib, "ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))dlsym(api.lib, "ncclGroupEnd");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.lib, "ncclGetErrorString");
  });
  if (!api.lib || !api.AllReduce || !api.CommInitRank) throw Error(RX_ERR_NCCL, "NCCL (libnccl.so.2) could not be loaded");
  return api;
}

void nck(ncclResult_t r, const char* what) {
  if (r != ncclSuccess) throw Error(RX_ERR_NCCL, std::string(what) + ": " + nccl().GetErrorString(r));
}
void cck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Error(RX_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

// One warp; lane r handles rank r.  The wait for a peer's word is bounded by `poll_limit` polls (the same
// per-client limit the fused form in the reduce kernel uses, RxClient::peer_wait_polls).
__global__ void k_allreduce_mailbox(float* __restrict__ val, MailTable mail, int rank, int n, unsigned epoch, int* status, long long poll_limit) {
  int lane = threadIdx.x;
  float mine = *val;
  unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(mine);
  int set = (epoch & 1) * kMaxRanks;
  if (lane < n) {
    volatile unsigned long long* dst = mail.peer[lane] + set + rank;
    *dst = word;  // single 64-bit store: value and sequence number arrive together
  }
  __threadfence_system();
  float got = 0.f;
  int failed = 0;
  if (lane < n) {
    volatile unsigned long long* src = mail.peer[rank] + set + lane;
    unsigned long long w = *src;
    long long spins = 0;
    while ((unsigned)(w >> 32) != epoch) {
      if (++spins > poll_limit) { failed = 1; break; }
      __nanosleep(kPeerPollNs);
      w = *src;
    }
    got = __uint_as_float((unsigned)w);
  }
  failed = __any_sync(0xFFFFFFFFu, failed);
  float sum = 0.f;
  for (int r = 0; r < n; ++r) sum += __shfl_sync(0xFFFFFFFFu, got, r);  // rank order: identical on every rank
  if (lane == 0) {
    if (failed) *status = 1;  // host reads this after the stream drains; value left untouched
    else *val = sum;
  }
}

// ---- halo exchange of row-sharded arrays -------------------------------------------------------------------------
// One CTA per device (rx_halo.cuh); a wait that runs out sets status 2 for the host.
__global__ void __launch_bounds__(1024) k_halo_exchange(const __grid_constant__ HaloArgs a, int* status) {
  if (!halo_exchange_cta(a) && threadIdx.x == 0) *status = 2;
}

void ensure_mailbox(RxDevice* d) {
  if (d->mailbox) return;
  cck(cudaSetDevice(d->ordinal), "cudaSetDevice");
  cck(cudaMalloc(&d->mailbox, kMailboxBytes), "cudaMalloc(mailbox)");
  cck(cudaMemset(d->mailbox, 0, kMailboxBytes), "cudaMemset(mailbox)");
}

// single-process client: enable peer access between all local devices and wire the tables
bool setup_local_mailboxes(RxClient* c) {
  if (c->num_nodes != 1) return false;
  size_t n = c->devices.size();
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < n; ++j) {
      if (i == j) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, c->devices[i]->ordinal, c->devices[j]->ordinal);
      if (!can) return false;
    }
  for (size_t i = 0; i < n; ++i) {
    ensure_mailbox(c->devices[i].get());
    cudaSetDevice(c->devices[i]->ordinal);
    for (size_t j = 0; j < n; ++j) {
      if (i == j) continue;
      cudaError_t e = cudaDeviceEnablePeerAccess(c->devices[j]->ordinal, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return false; }
      cudaGetLastError();
    }
  }
  for (size_t i = 0; i < n; ++i) {
    for (size_t j = 0; j < n; ++j) c->devices[i]->mail.peer[j] = c->devices[j]->mailbox;
    c->devices[i]->mail_ready = true;
  }
  return true;
}

}  // namespace

void nccl_unique_id(uint8_t* id128) {
  ncclUniqueId id;
  nck(nccl().GetUniqueId(&id), "ncclGetUniqueId");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  memcpy(id128, &id, 128);
}

void init_nccl(RxClient* c, const uint8_t* id128) {
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->nccl_ready) return;
  ncclUniqueId id;
  if (id128) memcpy(&id, id128, 128);
  else {
    if (c->num_nodes > 1) throw Error(RX_ERR_NCCL, "a multi-process client needs the unique id from rank 0 (RxClientInitCollectives)");
    nck(nccl().GetUniqueId(&id), "ncclGetUniqueId");
  }
  int nloc = (int)c->devices.size(), world = c->n_global();
  nck(nccl().GroupStart(), "ncclGroupStart");
  for (int k = 0; k < nloc; ++k) {
    cck(cudaSetDevice(c->devices[k]->ordinal), "cudaSetDevice");
    nck(nccl().CommInitRank((ncclComm_t*)&c->nccl_comms[k], world, id, c->devices[k]->global_id), "ncclCommInitRank");
  }
  nck(nccl().GroupEnd(), "ncclGroupEnd");
  c->nccl_ready = true;
}

void mailbox_handle(RxClient* c, int local_device, uint8_t* handle64) {
  if (local_device < 0 || local_device >= (int)c->devices.size()) throw Error(RX_ERR_ARG, "no such local device");
  RxDevice* d = c->devices[local_device].get();
  ensure_mailbox(d);
  cudaIpcMemHandle_t h;
  cck(cudaIpcGetMemHandle(&h, d->mailbox), "cudaIpcGetMemHandle");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  memcpy(handle64, &h, 64);
}

void open_mailboxes(RxClient* c, const uint8_t* handles, int n_global) {
  if (n_global != c->n_global()) throw Error(RX_ERR_ARG, "mailbox table has " + std::to_string(n_global) + " entries, mesh has " + std::to_string(c->n_global()));
  for (auto& d : c->devices) {
    ensure_mailbox(d.get());
    cck(cudaSetDevice(d->ordinal), "cudaSetDevice");
    for (int g = 0; g < n_global; ++g) {
      RxDevice* local = nullptr;
      for (auto& o : c->devices) if (o->global_id == g) local = o.get();
      if (local) {
        if (local != d.get()) {
          cudaError_t e = cudaDeviceEnablePeerAccess(local->ordinal, 0);
          if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) cck(e, "cudaDeviceEnablePeerAccess");
          cudaGetLastError();
        }
        ensure_mailbox(local);
        d->mail.peer[g] = local->mailbox;
      } else {
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)g * 64, 64);
        // a handle exported by this very process cannot be opened through IPC: map it directly
        unsigned long long* own = nullptr;
        for (auto& o : c->devices) {
          if (!o->mailbox) continue;
          cudaIpcMemHandle_t mine;
          cudaSetDevice(o->ordinal);
          if (cudaIpcGetMemHandle(&mine, o->mailbox) == cudaSuccess && !memcmp(&mine, &h, 64)) own = o->mailbox;
          cudaGetLastError();
        }
        cck(cudaSetDevice(d->ordinal), "cudaSetDevice");
        if (own) {
          d->mail.peer[g] = own;
          d->mail_own[g] = true;
        } else {
          void* p = nullptr;
          cck(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
          d->mail.peer[g] = (unsigned long long*)p;
        }
      }
    }
    d->mail_ready = true;
  }
}

void destroy_collectives(RxClient* c) {
  if (c->nccl_ready) {
    for (size_t k = 0; k < c->devices.size(); ++k)
      if (c->nccl_comms[k]) nccl().CommDestroy((ncclComm_t)c->nccl_comms[k]);
    c->nccl_ready = false;
  }
  for (auto& d : c->devices) {
    if (!d->mailbox) continue;
    cudaSetDevice(d->ordinal);
    if (c->num_nodes > 1 && d->mail_ready)
      for (int g = 0; g < c->n_global(); ++g) {
        bool local = false;
        for (auto& o : c->devices) local = local || o->global_id == g;
        if (!local && d->mail.peer[g] && !d->mail_own[g]) cudaIpcCloseMemHandle(d->mail.peer[g]);
      }
    cudaFree(d->mailbox);
    d->mailbox = nullptr;
  }
}

namespace {
bool mailboxes_ready_impl(RxClient* c) {
  std::lock_guard<std::mutex> lk(c->mu);
  bool ready = true;
  for (auto& d : c->devices) ready = ready && d->mail_ready;
  if (!ready && c->num_nodes == 1) ready = setup_local_mailboxes(c);
  return ready;
}
}  // namespace

bool halo_exchange_possible(RxClient* c, int64_t cols, int up, int down) {
  if (c->n_global() <= 1) return false;
  if (cols % 4 || cols > kHaloMaxCols || up > kHaloMaxRows || down > kHaloMaxRows || up < 0 || down < 0) return false;
  return mailboxes_ready_impl(c);
}

void halo_fill_args(RxClient* c, RxDevice* d, int64_t rows_local, int64_t cols, int up, int down, HaloArgs* out) {
  const int world = c->n_global();
  HaloArgs a{};
  a.rows_local = rows_local;
  a.cols = cols;
  a.up = up;
  a.down = down;
  a.rank = d->global_id;
  a.n = world;
  a.poll_limit = c->peer_wait_polls();
  a.mail_self = d->mail.peer[a.rank];
  a.mail_above = a.rank > 0 ? d->mail.peer[a.rank - 1] : nullptr;
  a.mail_below = a.rank + 1 < world ? d->mail.peer[a.rank + 1] : nullptr;
  *out = a;
}

unsigned halo_reserve_epochs(RxClient* c, unsigned count) {
  const unsigned first = c->halo_epoch + 1;
  c->halo_epoch += count;
  return first;
}

void run_halo_exchange(RxClient* c, size_t n_local, const std::function<RxDevice*(size_t)>& dev, const std::function<float*(size_t)>& block, int64_t rows_local,
                       int64_t cols, int up, int down) {
  const int world = c->n_global();
  if (world <= 1) return;
  if (n_local != c->devices.size()) throw Error(RX_ERR_ARG, "a halo exchange must run on every addressable device of the client");
  if (cols % 4 || cols > kHaloMaxCols || up > kHaloMaxRows || down > kHaloMaxRows || up < 0 || down < 0)
    throw Error(RX_ERR_UNSUPPORTED_OP, "row-sharded stencil: rows of " + std::to_string(cols) + " floats or a halo of " + std::to_string(std::max(up, down)) +
                                           " rows do not fit the exchange windows (rows up to " + std::to_string(kHaloMaxCols) + " floats, a multiple of 4; halo up to " +
                                           std::to_string(kHaloMaxRows) + ")");
  if (!mailboxes_ready_impl(c)) throw Error(RX_ERR_ARG, "row-sharded stencil: the devices' peer mailboxes are not open (RxClientOpenMailboxes)");
  const unsigned epoch = ++c->halo_epoch;
  for (size_t k = 0; k < n_local; ++k) {
    RxDevice* d = dev(k);
    cck(cudaSetDevice(d->ordinal), "cudaSetDevice");
    int* dstatus = nullptr;
    cck(cudaHostGetDevicePointer(&dstatus, d->status, 0), "cudaHostGetDevicePointer");
    HaloArgs a{};
    a.block = block(k);
    a.rows_local = rows_local;
    a.cols = cols;
    a.up = up;
    a.down = down;
    a.rank = d->global_id;
    a.n = world;
    a.epoch = epoch;
    a.poll_limit = c->peer_wait_polls();
    a.mail_self = d->mail.peer[a.rank];
    a.mail_above = a.rank > 0 ? d->mail.peer[a.rank - 1] : nullptr;
    a.mail_below = a.rank + 1 < world ? d->mail.peer[a.rank + 1] : nullptr;
    if ((uintptr_t)a.block % 16) throw Error(RX_ERR_PLAN, "internal: row block is not 16-byte aligned");
    bool prof = d->profiling;
    cudaEvent_t ea = nullptr, eb = nullptr;
    if (prof) { cudaEventCreate(&ea); cudaEventCreate(&eb); cudaEventRecord(ea, d->stream); }
    k_halo_exchange<<<1, 1024, 0, d->stream>>>(a, dstatus);
    if (prof) { cudaEventRecord(eb, d->stream); d->spans.push_back({"halo_exchange", ea, eb}); }
    ++d->launches;
    cck(cudaGetLastError(), "k_halo_exchange");
  }
}

bool prepare_fused_allreduce(RxClient* c, const Step& st, const std::vector<RxDevice*>& devs, std::vector<FusedAllReduce>* out) {
  int world = c->n_global();
  if (world <= 1 || c->allreduce_mode == 1 || st.count != 1 || devs.size() != c->devices.size()) return false;
  if (getenv("RX_NO_FUSED_ALLREDUCE")) return false;
  if (!mailboxes_ready_impl(c)) return false;
  unsigned epoch = ++c->epoch;
  out->clear();
  for (RxDevice* d : devs) {
    FusedAllReduce ar{};
    for (int r = 0; r < kMailRanks && r < kMaxRanks; ++r) ar.peer[r] = d->mail.peer[r];
    ar.rank = d->global_id;
    ar.n = world;
    ar.epoch = epoch;
    int* dstatus = nullptr;
    cudaSetDevice(d->ordinal);
    cudaHostGetDevicePointer(&dstatus, d->status, 0);
    ar.status = dstatus;
    ar.poll_limit = c->peer_wait_polls();
    out->push_back(ar);
  }
  return true;
}

void run_allreduce(RxClient* c, const Step& st, size_t n_local, const std::function<RxDevice*(size_t)>& dev, const std::function<void*(size_t)>& ptr,
                   bool on_comm_stream) {
  int world = c->n_global();
  if (world <= 1) return;
  if (n_local != c->devices.size()) throw Error(RX_ERR_ARG, "all_reduce must run on every addressable device of the client");
  bool want_mailbox = c->allreduce_mode != 1 && st.count == 1;
  if (want_mailbox) {
    std::lock_guard<std::mutex> lk(c->mu);
    bool ready = true;
    for (auto& d : c->devices) ready = ready && d->mail_ready;
    if (!ready && c->num_nodes == 1) ready = setup_local_mailboxes(c);
    if (!ready && c->allreduce_mode == 2) throw Error(RX_ERR_ARG, "mailbox all-reduce requested but peer mailboxes are not open");
    want_mailbox = ready;
  }
  if (want_mailbox) {
    unsigned epoch = ++c->epoch;
    for (size_t k = 0; k < n_local; ++k) {
      RxDevice* d = dev(k);
      cck(cudaSetDevice(d->ordinal), "cudaSetDevice");
      int* dstatus = nullptr;
      cck(cudaHostGetDevicePointer(&dstatus, d->status, 0), "cudaHostGetDevicePointer");
      bool prof = d->profiling;
      cudaEvent_t a = nullptr, b = nullptr;
      if (prof) { cudaEventCreate(&a); cudaEventCreate(&b); cudaEventRecord(a, d->stream); }
      k_allreduce_mailbox<<<1, 32, 0, d->stream>>>((float*)ptr(k), d->mail, d->global_id, world, epoch, dstatus, c->peer_wait_polls());
      if (prof) { cudaEventRecord(b, d->stream); d->spans.push_back({"all_reduce", a, b}); }
      ++d->launches;
      cck(cudaGetLastError(), "k_allreduce_mailbox");
    }
    return;
  }
  if (!c->nccl_ready) init_nccl(c, nullptr);
  nck(nccl().GroupStart(), "ncclGroupStart");
  for (size_t k = 0; k < n_local; ++k) {
    RxDevice* d = dev(k);
    cck(cudaSetDevice(d->ordinal), "cudaSetDevice");
    const ncclDataType_t ty = st.red_dt == DT::BF16 ? ncclBfloat16 : ncclFloat32;
    cudaStream_t s = (on_comm_stream && d->comm_stream) ? d->comm_stream : d->stream;
    nck(nccl().AllReduce(ptr(k), ptr(k), (size_t)st.count, ty, ncclSum, (ncclComm_t)c->nccl_comms[d->local_id], s), "ncclAllReduce");
    ++d->launches;
  }
  nck(nccl().GroupEnd(), "ncclGroupEnd");
}

}  // namespace rx
