// C ABI + executor.  Entry points keep the names and meaning of Reactant's
// PJRT shim (deps/ReactantExtra/API.cpp; see include/rx_b200.h for the
// line-by-line mapping).  Device memory is owned here through the CUDA runtime
// only; there is no CPU or library fallback behind any entry point.
#include "rx_runtime.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <sstream>
#include <unordered_set>

#include "../../include/rx_b200.h"
#include "rx_collective.h"
#include "rx_gemm.h"
#include "rx_jit.h"
#include "rx_stencil.h"

using namespace rx;

extern "C" {
void (*ReactantThrowError)(const char*) = nullptr;
}

namespace {

thread_local std::string g_err;
thread_local int g_code = 0;

void report(int code, const std::string& msg) {
  g_err = msg;
  g_code = code;
  if (ReactantThrowError) ReactantThrowError(msg.c_str());
}
void clear_error() {
  g_err.clear();
  g_code = 0;
}
struct CudaError : Error {
  explicit CudaError(cudaError_t e, const char* what) : Error(RX_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)) {}
};
#define CK(call)                                   \
  do {                                             \
    cudaError_t e__ = (call);                      \
    if (e__ != cudaSuccess) throw CudaError(e__, #call); \
  } while (0)

// Every handle this library has handed out and not yet been asked to free.  A host that runs this engine next to
// another runtime behind the same entry-point names (Reactant's XLA CPU client in the same Julia session) asks
// RxOwns before routing a call.
std::mutex g_own_mu;
std::unordered_set<const void*> g_owned;
template <class T>
T* own(T* p) {
  if (p) {
    std::lock_guard<std::mutex> g(g_own_mu);
    g_owned.insert(p);
  }
  return p;
}
void disown(const void* p) {
  std::lock_guard<std::mutex> g(g_own_mu);
  g_owned.erase(p);
}

char* dup_cstr(const std::string& s) {
  char* p = (char*)malloc(s.size() + 1);
  memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

size_t round_up(size_t b) { return b == 0 ? 256 : (b + 255) & ~(size_t)255; }

}  // namespace

namespace rx {
// error reporting for entry points that live in other translation units
void set_last_error(int code, const std::string& msg) { report(code, msg); }
void clear_last_error() { clear_error(); }
}  // namespace rx

// ---------------------------------------------------------------------------
// device pool
// ---------------------------------------------------------------------------
void* RxDevice::alloc(size_t bytes) {
  if (closed.load()) throw Error(RX_ERR_BAD_HANDLE, "the client that owns this device was freed");
  size_t rb = round_up(bytes);
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = pool.find(rb);
    if (it != pool.end() && !it->second.empty()) {
      void* p = it->second.back();
      it->second.pop_back();
      pool_bytes -= (int64_t)rb;
      bytes_in_use += (int64_t)rb;
      peak_bytes_in_use = std::max(peak_bytes_in_use, bytes_in_use);
      return p;
    }
  }
  if (bytes_limit > 0 && bytes_in_use + pool_bytes + (int64_t)rb > bytes_limit) trim();
  void* p = nullptr;
  CK(cudaSetDevice(ordinal));
  cudaError_t e = cudaMalloc(&p, rb);
  if (e != cudaSuccess) {
    cudaGetLastError();
    trim();
    e = cudaMalloc(&p, rb);
    if (e != cudaSuccess) {
      cudaGetLastError();
      throw Error(RX_ERR_CUDA, "out of device memory allocating " + std::to_string(rb) + " bytes on device " + std::to_string(ordinal));
    }
  }
  std::lock_guard<std::mutex> lk(mu);
  ++num_allocs;
  bytes_in_use += (int64_t)rb;
  peak_bytes_in_use = std::max(peak_bytes_in_use, bytes_in_use);
  largest_alloc = std::max<int64_t>(largest_alloc, (int64_t)rb);
  return p;
}

void RxDevice::release(void* p, size_t bytes) {
  if (!p) return;
  if (closed.load()) {  // pool and stream are gone: hand the block back to the driver
    cudaSetDevice(ordinal);
    cudaFree(p);
    cudaGetLastError();
    return;
  }
  size_t rb = round_up(bytes);
  std::lock_guard<std::mutex> lk(mu);
  pool[rb].push_back(p);
  bytes_in_use -= (int64_t)rb;
  pool_bytes += (int64_t)rb;
  peak_pool_bytes = std::max(peak_pool_bytes, pool_bytes);
}

void RxDevice::trim() {
  std::map<size_t, std::vector<void*>> old;
  {
    std::lock_guard<std::mutex> lk(mu);
    old.swap(pool);
    pool_bytes = 0;
  }
  if (old.empty()) return;
  cudaSetDevice(ordinal);
  cudaStreamSynchronize(stream);  // cached blocks may still be read by queued work
  for (auto& kv : old)
    for (void* p : kv.second) cudaFree(p);
}

cudaEvent_t EventState::event() {
  std::lock_guard<std::mutex> g(ev_mu);
  if (ev) return ev;
  if (!dev || dev->closed.load() || !dev->stream) return nullptr;
  cudaSetDevice(dev->ordinal);
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    ev = nullptr;
    return nullptr;
  }
  cudaEventRecord(ev, dev->stream);
  return ev;
}

namespace rx {
static std::atomic<uint64_t> g_foreign_launches{0};
uint64_t foreign_launches() { return g_foreign_launches.load(); }
void note_foreign_launch() { g_foreign_launches.fetch_add(1); }
}  // namespace rx

EventState::~EventState() {
  if (ev) {
    cudaSetDevice(dev->ordinal);
    cudaEventDestroy(ev);
  }
}

// ---------------------------------------------------------------------------
// executor
// ---------------------------------------------------------------------------
namespace {

struct DevRun {
  RxDevice* dev;
  std::vector<std::shared_ptr<Storage>> table;  // per slot
  // slots with an all-reduce still running on the device's communication stream, and the event that ends it
  std::map<int, cudaEvent_t> pending;
  int64_t iter = 0;  // 0-based iteration of the innermost counted loop whose body is being enqueued
};

// Before a step touches a slot whose all-reduce is still in flight on the communication stream, the compute
// stream waits for it (and only then): gradient all-reduces overlap the GEMMs that follow them.
void join_pending(DevRun& r, int slot) {
  auto it = r.pending.find(slot);
  if (it == r.pending.end()) return;
  cudaStreamWaitEvent(r.dev->stream, it->second, 0);
  cudaEventDestroy(it->second);  // destruction is deferred until the wait has been satisfied
  r.pending.erase(it);
}
void join_pending_of(DevRun& r, const Step& st) {
  if (r.pending.empty()) return;
  for (int s : st.leaf_slot) join_pending(r, s);
  for (int s : st.out_slot) join_pending(r, s);
  for (int s : {st.gemm.a_slot, st.gemm.b_slot, st.gemm.d_slot, st.src_slot, st.dst_slot})
    if (s >= 0) join_pending(r, s);
  for (int s : st.state_slots) join_pending(r, s);
  for (int s : st.yield_slots) join_pending(r, s);
  for (auto& j : st.sums) { join_pending(r, j.src_slot); join_pending(r, j.dst_slot); }
  if (st.kind == StepK::Loop) {  // a loop body may touch anything: simplest to drain
    while (!r.pending.empty()) join_pending(r, r.pending.begin()->first);
  }
}
void join_all_pending(DevRun& r) {
  while (!r.pending.empty()) join_pending(r, r.pending.begin()->first);
}

void* slot_ptr(DevRun& r, int slot) {
  if (slot < 0 || !r.table[slot]) throw Error(RX_ERR_PLAN, "internal: slot " + std::to_string(slot) + " has no storage");
  return r.table[slot]->ptr;
}

// Elements of the given type in the storage behind a slot (for the bounds-checked build).
int64_t slot_extent(DevRun& r, int slot, int elem) {
  const auto& st = r.table[slot];
  const size_t es = elem == EL_BF16 ? 2 : (elem == EL_F32 || elem == EL_I32) ? 4 : 1;
  int64_t n = st ? (int64_t)(st->bytes / es) : 0;
#if RX_BOUNDS
  // RX_BOUNDS_SELFTEST=1 understates every extent by one element, so that a correct program trips the check on the
  // last element of a buffer (the access is skipped, nothing is out of bounds): the way the reporting path is tested.
  static const bool selftest = getenv("RX_BOUNDS_SELFTEST") != nullptr;
  if (selftest && n > 0) --n;
#endif
  return n;
}

// The step's program with its operand and result descriptors pointed at this run's buffers.  `skip_leaf`: an operand
// that is not read from memory (the accumulator of a fused GEMM epilogue).
VmProgram bind(const Step& st, DevRun& r, int skip_leaf = -1) {
  VmProgram P = st.prog;
  int* rec = nullptr;
#if RX_BOUNDS
  cudaHostGetDevicePointer(&rec, r.dev->status, 0);
  rec += 4;  // words 4..7 of the status block: {what, index low, index high, extent}
#endif
  for (int k = 0; k < P.n_leaves; ++k) {
    if (k == skip_leaf) {
      P.leaf[k].ptr = nullptr;
      continue;
    }
    P.leaf[k].ptr = slot_ptr(r, st.leaf_slot[k]);
    P.leaf[k].extent = slot_extent(r, st.leaf_slot[k], P.leaf[k].elem);
    P.leaf[k].bounds = rec;
  }
  for (int k = 0; k < P.n_outs; ++k) {
    P.out[k].ptr = slot_ptr(r, st.out_slot[k]);
    P.out[k].extent = slot_extent(r, st.out_slot[k], P.out[k].elem);
    P.out[k].bounds = rec;
  }
  return P;
}

// the init value of a reduction in a wide program: a double's bits, or the 32-bit value in the low word
uint64_t wide_init_bits(const Step& st) {
  if (st.red_dt == DT::F64) {
    uint64_t u;
    memcpy(&u, &st.init_f, 8);
    return u;
  }
  if (st.red_dt == DT::PRED) return st.init_i ? 1u : 0u;
  return (uint64_t)(uint32_t)(int32_t)st.init_i;
}

uint32_t init_bits(const Step& st) {
  if (st.red_dt == DT::F32) {
    float f = (float)st.init_f;
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
  }
  if (st.red_dt == DT::PRED) return st.init_i ? 1u : 0u;
  return (uint32_t)(int32_t)st.init_i;
}

struct ProfScope {
  RxDevice* d;
  cudaEvent_t a = nullptr, b = nullptr;
  const char* kind;
  ProfScope(RxDevice* dev, const char* k) : d(dev), kind(k) {
    if (!d->profiling) return;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a, d->stream);
  }
  ~ProfScope() {
    if (!d->profiling) return;
    if (!kind) {  // the step was not taken after all
      cudaEventDestroy(a);
      cudaEventDestroy(b);
      return;
    }
    cudaEventRecord(b, d->stream);
    d->spans.push_back({kind, a, b});
  }
};

const char* kind_name(StepK k) {
  switch (k) {
    case StepK::Map: return "map";
    case StepK::ReduceFull: return "reduce_full";
    case StepK::ReduceRow: return "reduce_row";
    case StepK::ReduceCol: return "reduce_col";
    case StepK::LogSumExp: return "logsumexp";
    case StepK::Stencil: return "stencil";
    case StepK::Gemm: return "gemm";
    case StepK::Copy: return "copy";
    case StepK::Fill: return "fill";
    case StepK::Loop: return "loop";
    case StepK::AllReduce: return "all_reduce";
    case StepK::Scan: return "scan";
    case StepK::SumPartials: return "sum_partials";
    case StepK::RowsIn: return "rows_in";
    case StepK::RowsOut: return "rows_out";
    case StepK::DynSlice: return "dyn_slice";
  }
  return "?";
}

void run_steps(RxExecutable* ex, const std::vector<Step>& steps, std::vector<DevRun>& runs);
void note_writes(struct DevRun& r, const Step& st);

// End of a loop iteration: carried value j now lives where the body left its next value; the storage it
// vacated goes to the slots the body writes next time.
void rotate_loop_state(const Step& st, DevRun& r) {
  std::vector<int> involved = st.state_slots;
  for (int y : st.yield_slots)
    if (std::find(involved.begin(), involved.end(), y) == involved.end()) involved.push_back(y);
  std::map<int, std::shared_ptr<Storage>> old;
  for (int s : involved) old[s] = r.table[s];
  std::vector<std::shared_ptr<Storage>> spare;
  std::map<int, bool> taken;
  for (size_t j = 0; j < st.state_slots.size(); ++j) {
    r.table[st.state_slots[j]] = old[st.yield_slots[j]];
    taken[st.yield_slots[j]] = true;
  }
  for (int s : involved)
    if (!taken.count(s)) spare.push_back(old[s]);
  size_t q = 0;
  for (int s : involved)
    if (std::find(st.state_slots.begin(), st.state_slots.end(), s) == st.state_slots.end()) r.table[s] = spare[q++];
}

// A counted loop whose body is only stencil updates runs as one cooperative launch (rx_stencil_tma.cu).  The
// buffer bindings of the body repeat with the period of the storage rotation (2 for the Jacobi swap); they are
// found by rotating a copy of the slot table until it returns to where it started.
bool try_stencil_loop(const Step& st, DevRun& r) {
  static const bool off = getenv("RX_STENCIL_LOOP") && atoi(getenv("RX_STENCIL_LOOP")) == 0;
  if (off || st.trip < 2 || st.body.empty() || st.body.size() > 4) return false;
  for (const Step& b : st.body)
    if (b.kind != StepK::Stencil) return false;
  RxDevice* d = r.dev;
  CK(cudaSetDevice(d->ordinal));
  const auto saved = r.table;
  std::vector<const Step*> steps;
  std::vector<VmProgram> bound;
  int period = 0;
  for (int p = 1; p <= 4 && !period; ++p) {
    if (steps.size() + st.body.size() > 4) break;
    for (const Step& b : st.body) {
      steps.push_back(&b);
      bound.push_back(bind(b, r));
    }
    rotate_loop_state(st, r);
    if (r.table == saved) period = p;
  }
  r.table = saved;
  if (!period) return false;
  bool handled = false;
  {
    ProfScope ps(d, "stencil_tma_loop");
    CK(rx::run_stencil_loop(d, steps, bound, st.trip * (int64_t)st.body.size(), &handled));
    if (!handled) ps.kind = nullptr;
  }
  if (!handled) return false;
  note_writes(r, st);
  d->last_stencil_tma = true;
  for (int64_t i = 0; i < st.trip % period; ++i) rotate_loop_state(st, r);
  return true;
}

// What the launch of `st` writes, for the early-read decision of the launch behind it.
void note_writes(DevRun& r, const Step& st) {
  RxDevice* d = r.dev;
  d->last_writes.clear();
  d->foreign_seen = rx::foreign_launches();
  auto add = [&](int slot) {
    if (slot >= 0 && r.table[slot]) d->last_writes.push_back(r.table[slot]->ptr);
  };
  for (int s : st.out_slot) add(s);
  add(st.dst_slot);
  add(st.gemm.d_slot);
  for (int s : st.state_slots) add(s);
  for (int s : st.yield_slots) add(s);
  for (auto& j : st.sums) add(j.dst_slot);
}
bool operands_settled(DevRun& r, const Step& st) {
  RxDevice* d = r.dev;
  if (d->foreign_seen != rx::foreign_launches()) return false;
  for (int s : st.leaf_slot) {
    const void* p = slot_ptr(r, s);
    for (const void* w : d->last_writes)
      if (w == p) return false;
  }
  return true;
}

void run_one(RxExecutable* ex, const Step& st, DevRun& r, const FusedAllReduce* fused = nullptr) {
  RxDevice* d = r.dev;
  CK(cudaSetDevice(d->ordinal));
  LaunchCtx c = d->ctx();
  if (st.kind == StepK::ReduceFull) c.operands_settled = operands_settled(r, st);
  struct NoteAfter {
    DevRun& r;
    const Step& st;
    ~NoteAfter() { note_writes(r, st); }
  } note_after{r, st};
  static const bool by_note = getenv("RX_PROFILE_NOTES") != nullptr;  // finer spans: one per plan step description
  ProfScope ps(d, by_note ? st.note.c_str() : kind_name(st.kind));
  switch (st.kind) {
    case StepK::Map: {
      VmProgram P = bind(st, r);
      if (P.wide) {
        CK(launch_wide_map(c, P));
        if (!by_note) ps.kind = "map_f64";
        break;
      }
      CK(launch_map(c, P));
      break;
    }
    case StepK::Stencil: {
      VmProgram P = bind(st, r);
      CK(rx::run_stencil(d, st, P));
      ps.kind = d->last_stencil_tma ? "stencil_tma" : "stencil_generic";
      break;
    }
    case StepK::ReduceFull: {
      VmProgram P = bind(st, r);
      if (P.wide) {
        if (fused) throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type f64 in a sharded reduction");
        CK(launch_wide_reduce(c, P, 0, red_code(st.red, st.red_dt), st.red_dt == DT::F64, wide_init_bits(st), 1, st.red_n, 1));
        if (!by_note) ps.kind = "reduce_f64";
        break;
      }
      CK(launch_reduce_full(c, P, red_code(st.red, st.red_dt), init_bits(st), fused));
      break;
    }
    case StepK::ReduceRow: {
      VmProgram P = bind(st, r);
      if (P.wide) {
        CK(launch_wide_reduce(c, P, 1, red_code(st.red, st.red_dt), st.red_dt == DT::F64, wide_init_bits(st), st.outer, st.red_n, 1));
        if (!by_note) ps.kind = "reduce_f64";
        break;
      }
      CK(launch_reduce_row(c, P, red_code(st.red, st.red_dt), init_bits(st), st.outer, st.red_n));
      break;
    }
    case StepK::ReduceCol: {
      VmProgram P = bind(st, r);
      if (P.wide) {
        CK(launch_wide_reduce(c, P, 2, red_code(st.red, st.red_dt), st.red_dt == DT::F64, wide_init_bits(st), st.outer, st.red_n, st.inner));
        if (!by_note) ps.kind = "reduce_f64";
        break;
      }
      int ns = reduce_col_splits(st.outer, st.red_n, st.inner, d->sm_count);
      size_t words = (size_t)st.outer * ns * st.inner;
      std::shared_ptr<Storage> tmp;
      uint32_t* partials = d->scratch;
      if (words + 1 > d->scratch_words) {
        tmp = std::make_shared<Storage>(d, d->alloc(words * 4), words * 4);
        partials = (uint32_t*)tmp->ptr;
      }
      CK(launch_reduce_col(c, P, red_code(st.red, st.red_dt), init_bits(st), st.outer, st.red_n, st.inner, partials, ns));
      break;
    }
    case StepK::LogSumExp: {
      const VmLeaf& l = st.prog.leaf[0];
      const float* x = (const float*)slot_ptr(r, st.leaf_slot[0]) + l.offset;
      CK(launch_logsumexp(c, x, l.stride[0], st.outer, st.red_n, (float*)slot_ptr(r, st.out_slot[0]), (float*)slot_ptr(r, st.out_slot[1]),
                          (float*)slot_ptr(r, st.out_slot[2])));
      break;
    }
    case StepK::Scan: {
      if (st.red_dt == DT::F64) {
        CK(launch_wide_scan(c, slot_ptr(r, st.src_slot), slot_ptr(r, st.dst_slot), red_code(st.red, st.red_dt), st.outer, st.red_n, st.inner));
        break;
      }
      CK(launch_scan(c, slot_ptr(r, st.src_slot), slot_ptr(r, st.dst_slot), red_code(st.red, st.red_dt), st.outer, st.red_n, st.inner));
      break;
    }
    case StepK::Gemm: {
      const GemmDesc& g = st.gemm;
      void* dptr = r.table[g.d_slot] ? r.table[g.d_slot]->ptr : nullptr;  // absent when the product is consumed in the epilogue only
      if (g.has_epilogue) {
        VmProgram P = bind(st, r, g.acc_leaf);
        GemmEpilogueArgs ea;
        ea.prog = &P;
        for (int q = 0; q < g.n_col; ++q) ea.col_partial[q] = (float*)slot_ptr(r, g.col_slot[q]);
        for (int q = 0; q < g.n_full; ++q) ea.full_partial[q] = (float*)slot_ptr(r, g.full_slot[q]);
        CK(rx::run_gemm(d, st, slot_ptr(r, g.a_slot), slot_ptr(r, g.b_slot), dptr, &ea));
        if (!by_note) ps.kind = "gemm_tc_fused";
      } else if (g.in_dt == DT::F64) {
        CK(launch_wide_gemm(c, (const double*)slot_ptr(r, g.a_slot) + g.a_off, (const double*)slot_ptr(r, g.b_slot) + g.b_off, slot_ptr(r, g.d_slot), g.M, g.N, g.K, g.batch, g.a_sm,
                            g.a_sk, g.b_sk, g.b_sn, g.a_sb, g.b_sb, g.d_sb));
        if (!by_note) ps.kind = "gemm_f64";
      } else {
        CK(rx::run_gemm(d, st, slot_ptr(r, g.a_slot), slot_ptr(r, g.b_slot), slot_ptr(r, g.d_slot)));
        if (!by_note) ps.kind = d->last_gemm_tc ? "gemm_tc" : "gemm_simt";
      }
      break;
    }
    case StepK::SumPartials: {
      SumPartialsJob jobs[4] = {};
      int n = 0;
      for (const SumJob& j : st.sums) {
        jobs[n].src = (const float*)slot_ptr(r, j.src_slot);
        jobs[n].dst = (float*)slot_ptr(r, j.dst_slot);
        jobs[n].rows = j.rows;
        jobs[n].n = j.n;
        jobs[n].init = (float)j.init;
        ++n;
      }
      CK(launch_sum_partials(c, jobs, n));
      break;
    }
    case StepK::Copy: {
      CK(cudaMemcpyAsync(slot_ptr(r, st.dst_slot), slot_ptr(r, st.src_slot), (size_t)st.bytes, cudaMemcpyDeviceToDevice, d->stream));
      break;
    }
    case StepK::DynSlice: {
      // the start indices follow the loop counter; each is clamped so that the slice stays inside the operand
      int64_t off = 0;
      for (size_t k = 0; k < st.dyn_a.size(); ++k) {
        const int64_t start = std::max<int64_t>(0, std::min<int64_t>(st.dyn_a[k] * r.iter + st.dyn_b[k], st.dyn_hi[k]));
        off += start * st.dyn_stride[k];
      }
      CK(cudaMemcpyAsync(slot_ptr(r, st.dst_slot), (const char*)slot_ptr(r, st.src_slot) + off * st.dyn_elem_bytes, (size_t)st.bytes, cudaMemcpyDeviceToDevice, d->stream));
      break;
    }
    default:
      throw Error(RX_ERR_PLAN, std::string("internal: step kind ") + kind_name(st.kind) + " has no single-device launch");
  }
}

// A counted loop of stencil updates over arrays split into row blocks.  The body's steps describe the update of the
// global arrays; device g applies each one to the output rows it owns (reading its halos), then every device sends
// the boundary rows of the array just written to its neighbours.  Row r of a device's block is global row
// g * rows_local - halo_up + r.
// The part of stencil step `b` that device r.dev owns, in the coordinates of its row block: the step with shifted
// offsets and its bound program.  False if none of the updated rows is this device's.
bool local_stencil_step(const Plan& plan, const Step& b, DevRun& r, Step* loc, VmProgram* P) {
  const Slot& blk = plan.slots[b.out_slot[0]];
  const int64_t ld = b.st_src_ld, rows_local = blk.type.shape[0] / plan.num_partitions;
  const int64_t drow0 = b.st_dst_off / ld;
  const int64_t g = r.dev->global_id, base = g * rows_local - blk.halo_up;
  const int64_t o0 = std::max<int64_t>(drow0, g * rows_local), o1 = std::min<int64_t>(drow0 + b.st_rows, (g + 1) * rows_local);
  if (o1 <= o0) return false;
  *loc = b;
  const int64_t shift = ((o0 - drow0) - base) * ld;  // global element index -> index in this device's block
  loc->st_rows = o1 - o0;
  loc->st_dst_off = b.st_dst_off + shift;
  loc->st_src_off = b.st_src_off + shift;
  *P = bind(*loc, r);
  P->dim[0] = loc->st_rows;
  for (int k = 0; k < P->n_leaves; ++k) P->leaf[k].offset += shift;
  P->out[0].offset += shift;
  return true;
}

// The whole row-sharded loop as one cooperative launch per device, boundary rows exchanged inside the kernel between
// sweeps.  Taken only if every device can take it (they wait for one another's rows).
bool try_row_sharded_stencil_loop(RxExecutable* ex, const Step& loop, std::vector<DevRun>& runs) {
  const bool off = getenv("RX_STENCIL_LOOP") && atoi(getenv("RX_STENCIL_LOOP")) == 0;  // read per call: tests compare both forms in one process
  if (off || loop.trip < 2 || loop.body.empty() || loop.body.size() > 4) return false;
  const Plan& plan = *ex->plan;
  const Slot& blk0 = plan.slots[loop.body[0].out_slot[0]];
  for (const Step& b : loop.body) {
    const Slot& blk = plan.slots[b.out_slot[0]];
    if (b.kind != StepK::Stencil || blk.type.shape != blk0.type.shape || blk.halo_up != blk0.halo_up || blk.halo_down != blk0.halo_down) return false;
  }
  const int64_t rows_local = blk0.type.shape[0] / plan.num_partitions, cols = blk0.type.shape[1];
  if (!rx::halo_exchange_possible(ex->client, cols, blk0.halo_up, blk0.halo_down)) return false;
  if (runs.size() != ex->client->devices.size()) return false;
  struct PerDev {
    std::vector<Step> local;
    std::vector<const Step*> steps;
    std::vector<VmProgram> bound;
    rx::StencilLoopHalo halo;
    int period = 0;
  };
  std::vector<PerDev> per(runs.size());
  const int64_t total = loop.trip * (int64_t)loop.body.size();
  int passes = 0;
  for (size_t k = 0; k < runs.size(); ++k) {
    DevRun& r = runs[k];
    PerDev& pd = per[k];
    CK(cudaSetDevice(r.dev->ordinal));
    const auto saved = r.table;
    pd.local.reserve(8);
    bool ok = true;
    for (int p = 1; p <= 4 && !pd.period && ok; ++p) {
      if (pd.local.size() + loop.body.size() > 4) break;
      for (const Step& b : loop.body) {
        Step loc;
        VmProgram P;
        if (!local_stencil_step(plan, b, r, &loc, &P)) { ok = false; break; }
        pd.local.push_back(loc);
        pd.bound.push_back(P);
        pd.halo.block.push_back((float*)slot_ptr(r, b.out_slot[0]));
      }
      rotate_loop_state(loop, r);
      if (r.table == saved) pd.period = p;
    }
    r.table = saved;
    if (!ok || !pd.period) return false;
    for (const Step& s : pd.local) pd.steps.push_back(&s);
    rx::halo_fill_args(ex->client, r.dev, rows_local, cols, blk0.halo_up, blk0.halo_down, &pd.halo.args);
    {
      // does the update window continue into the rows above / below this device's?
      const Step& b0 = loop.body[0];
      const int64_t ld = b0.st_src_ld, drow0 = b0.st_dst_off / ld, g = r.dev->global_id;
      pd.halo.window_above = g * rows_local > drow0;
      pd.halo.window_below = (g + 1) * rows_local < drow0 + b0.st_rows;
    }
    bool would = false;
    int dev_passes = 0;
    CK(rx::run_stencil_loop(r.dev, pd.steps, pd.bound, total, &would, &pd.halo, true, &dev_passes));
    if (!would) return false;
    if (k == 0) passes = dev_passes;
    else if (dev_passes != passes) return false;  // the devices must run the same sequence of passes
  }
  const unsigned epoch0 = rx::halo_reserve_epochs(ex->client, (unsigned)(passes - 1));
  for (size_t k = 0; k < runs.size(); ++k) {
    DevRun& r = runs[k];
    PerDev& pd = per[k];
    CK(cudaSetDevice(r.dev->ordinal));
    pd.halo.epoch0 = epoch0;
    bool handled = false;
    {
      ProfScope ps(r.dev, "stencil_rows_loop");
      CK(rx::run_stencil_loop(r.dev, pd.steps, pd.bound, total, &handled, &pd.halo, false));
    }
    // every device passed the dry run with the same arguments; a launch that is refused now leaves the others waiting
    // until their bounded wait runs out, which the host then reports
    if (!handled) throw Error(RX_ERR_CUDA, "row-sharded stencil loop: cooperative launch refused after the dry run accepted it");
    note_writes(r, loop);
    r.dev->last_stencil_tma = true;
    for (int64_t i = 0; i < loop.trip % pd.period; ++i) rotate_loop_state(loop, r);
  }
  return true;
}

void run_row_sharded_loop(RxExecutable* ex, const Step& loop, std::vector<DevRun>& runs) {
  const Plan& plan = *ex->plan;
  const int64_t nparts = plan.num_partitions;
  if (try_row_sharded_stencil_loop(ex, loop, runs)) return;
  for (int64_t it = 0; it < loop.trip; ++it) {
    for (const Step& b : loop.body) {
      const Slot& blk = plan.slots[b.out_slot[0]];
      const int64_t rows_local = blk.type.shape[0] / nparts;
      for (auto& r : runs) {
        RxDevice* d = r.dev;
        CK(cudaSetDevice(d->ordinal));
        Step loc;
        VmProgram P;
        if (!local_stencil_step(plan, b, r, &loc, &P)) continue;  // none of the updated rows is this device's
        ProfScope ps(d, "stencil_rows");
        CK(rx::run_stencil(d, loc, P));
        note_writes(r, loc);
      }
      rx::run_halo_exchange(ex->client, runs.size(), [&](size_t k) { return runs[k].dev; }, [&](size_t k) { return (float*)slot_ptr(runs[k], b.out_slot[0]); }, rows_local,
                            blk.type.shape[1], blk.halo_up, blk.halo_down);
    }
    for (auto& r : runs) rotate_loop_state(loop, r);
  }
}

void run_steps(RxExecutable* ex, const std::vector<Step>& steps, std::vector<DevRun>& runs) {
  for (size_t si = 0; si < steps.size(); ++si) {
    const Step& st = steps[si];
    for (auto& r : runs) join_pending_of(r, st);
    // a full reduce of f32 followed by the all-reduce of its scalar: one kernel does both
    if (st.kind == StepK::ReduceFull && si + 1 < steps.size() && steps[si + 1].kind == StepK::AllReduce && st.out_slot.size() == 1 &&
        steps[si + 1].dst_slot == st.out_slot[0] && st.red == RedK::Add && st.red_dt == DT::F32 && st.prog.out[0].elem == EL_F32) {
      std::vector<RxDevice*> devs;
      for (auto& r : runs) devs.push_back(r.dev);
      std::vector<FusedAllReduce> fused;
      if (rx::prepare_fused_allreduce(ex->client, steps[si + 1], devs, &fused)) {
        for (size_t k = 0; k < runs.size(); ++k) run_one(ex, st, runs[k], &fused[k]);
        ++si;
        continue;
      }
    }
    if (st.kind == StepK::RowsIn || st.kind == StepK::RowsOut) {
      const Plan& plan = *ex->plan;
      const Slot& blk = plan.slots[st.kind == StepK::RowsIn ? st.dst_slot : st.src_slot];
      const int64_t cols = blk.type.shape[1], rows_local = blk.type.shape[0] / plan.num_partitions;
      const size_t bytes = (size_t)rows_local * cols * sizeof(float), skip = (size_t)blk.halo_up * cols * sizeof(float);
      for (auto& r : runs) {
        CK(cudaSetDevice(r.dev->ordinal));
        char* src = (char*)slot_ptr(r, st.src_slot);
        char* dst = (char*)slot_ptr(r, st.dst_slot);
        if (st.kind == StepK::RowsIn) CK(cudaMemcpyAsync(dst + skip, src, bytes, cudaMemcpyDeviceToDevice, r.dev->stream));
        else CK(cudaMemcpyAsync(dst, src + skip, bytes, cudaMemcpyDeviceToDevice, r.dev->stream));
        note_writes(r, st);
      }
      if (st.kind == StepK::RowsIn)
        rx::run_halo_exchange(ex->client, runs.size(), [&](size_t k) { return runs[k].dev; }, [&](size_t k) { return (float*)slot_ptr(runs[k], st.dst_slot); }, rows_local,
                              cols, blk.halo_up, blk.halo_down);
      continue;
    }
    if (st.kind == StepK::Loop && st.row_sharded) {
      run_row_sharded_loop(ex, st, runs);
      continue;
    }
    if (st.kind == StepK::Loop) {
      // Same plan and same shapes on every device, so they normally take the same decision; should one decline after
      // others ran the whole loop, only the ones that declined go through the step-by-step form below.
      std::vector<DevRun> rest;
      std::vector<size_t> rest_index;
      for (size_t k = 0; k < runs.size(); ++k)
        if (!try_stencil_loop(st, runs[k])) { rest.push_back(std::move(runs[k])); rest_index.push_back(k); }
      if (rest.empty()) continue;
      std::vector<int64_t> outer_iter;
      for (auto& r : rest) outer_iter.push_back(r.iter);
      for (int64_t it = 0; it < st.trip; ++it) {
        for (auto& r : rest) r.iter = it;
        run_steps(ex, st.body, rest);
        for (auto& r : rest) {
          join_all_pending(r);  // in-flight all-reduces are tracked by slot, and the rotation moves storages between slots
          rotate_loop_state(st, r);
        }
      }
      for (size_t q = 0; q < rest.size(); ++q) rest[q].iter = outer_iter[q];
      for (size_t q = 0; q < rest.size(); ++q) runs[rest_index[q]] = std::move(rest[q]);
    } else if (st.kind == StepK::AllReduce) {
      // vectors (gradients) go to the communication stream so that the steps after them keep the SMs busy;
      // single words stay on the compute stream (mailbox kernel, a few microseconds)
      static const bool overlap_off = getenv("RX_ALLREDUCE_OVERLAP") && atoi(getenv("RX_ALLREDUCE_OVERLAP")) == 0;
      const bool side = st.count > 1 && !overlap_off && ex->client->n_global() > 1;
      if (side) {
        for (auto& r : runs) {
          RxDevice* d = r.dev;
          CK(cudaSetDevice(d->ordinal));
          if (!d->comm_stream) CK(cudaStreamCreateWithFlags(&d->comm_stream, cudaStreamNonBlocking));
          cudaEvent_t ready;
          CK(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming));
          CK(cudaEventRecord(ready, d->stream));
          CK(cudaStreamWaitEvent(d->comm_stream, ready, 0));
          cudaEventDestroy(ready);
        }
      }
      rx::run_allreduce(ex->client, st, runs.size(), [&](size_t k) { return runs[k].dev; }, [&](size_t k) { return slot_ptr(runs[k], st.dst_slot); }, side);
      for (auto& r : runs) note_writes(r, st);
      if (side) {
        for (auto& r : runs) {
          CK(cudaSetDevice(r.dev->ordinal));
          cudaEvent_t done;
          CK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
          CK(cudaEventRecord(done, r.dev->comm_stream));
          r.pending[st.dst_slot] = done;
        }
      }
    } else {
      for (auto& r : runs) run_one(ex, st, r);
    }
  }
}

void check_arg(const Plan& p, int i, RxBuffer* b, RxDevice* d) {
  if (!b) throw Error(RX_ERR_BAD_HANDLE, "argument " + std::to_string(i) + " is a null buffer");
  if (b->donated.load() || !b->st) throw Error(RX_ERR_DONATED, "argument " + std::to_string(i) + " was donated to an earlier execution");
  if (b->dev != d) throw Error(RX_ERR_ARG, "argument " + std::to_string(i) + " lives on a different device than the one executing");
  const Type& t = p.arg_types[i];
  if (b->dt != t.dt || b->dims != t.shape) {
    Type got{b->dt, b->dims};
    throw Error(RX_ERR_SHAPE, "argument " + std::to_string(i) + " is " + got.str() + ", executable expects " + t.str());
  }
}

// Runs the plan on `devs` (one program instance per device), args laid out [device][arg].
void execute(RxExecutable* ex, const std::vector<RxDevice*>& devs, RxBuffer** args, int nargs_per_dev, const uint8_t* donatable,
             int num_results, RxBuffer** results, uint8_t* futures, RxFuture** future_results) {
  const Plan& p = *ex->plan;
  if (nargs_per_dev != (int)p.arg_types.size())
    throw Error(RX_ERR_ARG, "executable takes " + std::to_string(p.arg_types.size()) + " arguments per device, got " + std::to_string(nargs_per_dev));
  if (num_results != (int)p.results.size())
    throw Error(RX_ERR_ARG, "Error: results.size()=" + std::to_string(p.results.size()) + " does not match num_results=" + std::to_string(num_results));
  if (p.num_partitions > 1 && (int64_t)devs.size() * ex->client->num_nodes != p.num_partitions)
    throw Error(RX_ERR_ARG, "executable is partitioned over " + std::to_string(p.num_partitions) + " devices, launch covers " + std::to_string(devs.size() * ex->client->num_nodes));
  // Thunks may be called from any host thread (Julia tasks): serialise the enqueueing per device, taking the
  // devices in a fixed order so that two multi-device executions cannot deadlock.
  std::vector<RxDevice*> order(devs.begin(), devs.end());
  std::sort(order.begin(), order.end(), [](RxDevice* a, RxDevice* b) { return a->ordinal < b->ordinal; });
  order.erase(std::unique(order.begin(), order.end()), order.end());
  std::vector<std::unique_lock<std::mutex>> held;
  for (RxDevice* d : order) held.emplace_back(d->exec_mu);
  std::vector<DevRun> runs(devs.size());
  for (size_t k = 0; k < devs.size(); ++k) {
    RxDevice* d = devs[k];
    DevRun& r = runs[k];
    r.dev = d;
    r.table.resize(p.slots.size());
    CK(cudaSetDevice(d->ordinal));
    for (int i = 0; i < nargs_per_dev; ++i) check_arg(p, i, args[k * nargs_per_dev + i], d);
    for (size_t s = 0; s < p.slots.size(); ++s) {
      const Slot& sl = p.slots[s];
      if (sl.kind == SlotK::Arg) {
        RxBuffer* b = args[k * nargs_per_dev + sl.arg_index];
        b->st->make_ready();
        if (sl.writable && !(donatable && donatable[sl.arg_index])) {
          // the plan updates this argument in place but the caller keeps it: work on a private copy
          size_t bytes = (size_t)sl.bytes();
          auto st = std::make_shared<Storage>(d, d->alloc(bytes), bytes);
          CK(cudaMemcpyAsync(st->ptr, b->st->ptr, bytes, cudaMemcpyDeviceToDevice, d->stream));
          d->last_writes.push_back(st->ptr);  // a copy may run as a kernel: its target is not settled yet
          r.table[s] = st;
        } else {
          r.table[s] = b->st;
        }
      } else if (sl.kind == SlotK::Const) {
        std::lock_guard<std::mutex> lk(ex->mu);
        auto& cs = ex->consts[d->local_id];
        auto it = cs.find((int)s);
        if (it == cs.end()) {
          size_t bytes = (size_t)sl.bytes();
          auto st = std::make_shared<Storage>(d, d->alloc(bytes), bytes);
          CK(cudaMemcpyAsync(st->ptr, sl.init.data(), bytes, cudaMemcpyHostToDevice, d->stream));
          CK(cudaStreamSynchronize(d->stream));
          it = cs.emplace((int)s, st).first;
        }
        r.table[s] = it->second;
      } else if (sl.row_block) {
        // this device's block of rows plus the halo rows above and below it
        const int64_t rows_local = sl.type.shape[0] / p.num_partitions;
        size_t bytes = (size_t)(rows_local + sl.halo_up + sl.halo_down) * (size_t)sl.type.shape[1] * dt_size(sl.type.dt);
        r.table[s] = std::make_shared<Storage>(d, d->alloc(bytes), bytes);
      } else if (!sl.dead) {
        size_t bytes = (size_t)sl.bytes();
        r.table[s] = std::make_shared<Storage>(d, d->alloc(bytes), bytes);
      }
    }
  }
  run_steps(ex, p.steps, runs);
  // All-reduces still in flight on the communication stream: a result keeps the event (its future and its next user
  // wait for it), so the compute stream is free to start the next execution; anything else is joined now.
  std::vector<std::map<int, std::shared_ptr<EventState>>> late(devs.size());  // [device][slot] -> completion of a result's all-reduce
  for (size_t k = 0; k < devs.size(); ++k) {
    DevRun& r = runs[k];
    CK(cudaSetDevice(r.dev->ordinal));
    for (const ResultBinding& rb : p.results) {
      auto it = r.pending.find(rb.slot);
      if (it == r.pending.end() || late[k].count(rb.slot)) continue;
      auto es = std::make_shared<EventState>();
      es->dev = r.dev;
      es->keep = r.dev->shared_from_this();
      es->ev = it->second;              // recorded on the communication stream after the all-reduce
      late[k][rb.slot] = es;
      cudaEvent_t again;               // a second event for the storage itself (the future may be freed first)
      CK(cudaEventCreateWithFlags(&again, cudaEventDisableTiming));
      CK(cudaEventRecord(again, r.dev->comm_stream));
      {
        Storage& st = *r.table[rb.slot];
        std::lock_guard<std::mutex> g(st.pending_mu);
        if (st.pending) cudaEventDestroy(st.pending);
        st.pending = again;
      }
      r.pending.erase(it);
    }
    join_all_pending(r);
  }
  for (size_t k = 0; k < devs.size(); ++k) {
    RxDevice* d = devs[k];
    CK(cudaSetDevice(d->ordinal));
    auto es = std::make_shared<EventState>();
    es->dev = d;
    es->keep = d->shared_from_this();
    for (int j = 0; j < num_results; ++j) {
      const ResultBinding& rb = p.results[j];
      auto* b = own(new RxBuffer());
      b->st = runs[k].table[rb.slot];
      b->dt = rb.type.dt;
      b->dims = rb.type.shape;
      b->dev = d;
      results[k * num_results + j] = b;
      if (future_results) {
        auto* f = own(new RxFuture());
        auto lt = late[k].find(rb.slot);
        f->state = lt != late[k].end() ? lt->second : es;
        future_results[k * num_results + j] = f;
      }
    }
    // donated arguments whose storage the plan may have rewritten are dead for the caller
    for (int i = 0; i < nargs_per_dev; ++i)
      if (donatable && donatable[i] && p.arg_alias[i] >= 0) {
        RxBuffer* b = args[k * nargs_per_dev + i];
        b->donated.store(true);
        b->st.reset();
      }
  }
  if (futures) *futures = future_results ? 1 : 0;
}

std::shared_ptr<RxDevice> make_device(RxClient* c, int ordinal, int local_id, double fraction) {
  auto d = std::make_shared<RxDevice>();
  d->client = c;
  d->ordinal = ordinal;
  d->local_id = local_id;
  CK(cudaSetDevice(ordinal));
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, ordinal));
  d->sm_count = prop.multiProcessorCount;
  d->kind = std::string(prop.name) + " (sm_" + std::to_string(prop.major) + std::to_string(prop.minor) + ")";
  d->total_mem = prop.totalGlobalMem;
  d->bytes_limit = (int64_t)((double)prop.totalGlobalMem * (fraction > 0 && fraction <= 1 ? fraction : 0.9));
  CK(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  d->scratch_words = (size_t)1 << 20;
  CK(cudaMalloc(&d->scratch, d->scratch_words * 4));
  CK(cudaMemset(d->scratch, 0, d->scratch_words * 4));  // the last word is the finished-CTA ticket of the reductions
  CK(cudaHostAlloc(&d->status, 64, cudaHostAllocMapped));
  memset(d->status, 0, 64);
  return d;
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
#define API_BEGIN clear_error(); try {
#define API_END(ret)                                  \
  }                                                   \
  catch (const Error& e) { report(e.code, e.what()); } \
  catch (const std::exception& e) { report(RX_ERR_PLAN, e.what()); } \
  return ret;
#define API_END_VOID                                  \
  }                                                   \
  catch (const Error& e) { report(e.code, e.what()); } \
  catch (const std::exception& e) { report(RX_ERR_PLAN, e.what()); }

extern "C" {

const char* RxLastError(void) { return g_err.c_str(); }
int RxLastErrorCode(void) { return g_code; }
void RxClearError(void) { clear_error(); }

RxClient* MakeGPUClient(int node_id, int num_nodes, int64_t* allowed_devices, int64_t num_allowed_devices, double memory_fraction,
                        uint8_t preallocate, const char* platform_name, const char** error, void* distributed_runtime_client) {
  (void)preallocate; (void)platform_name; (void)distributed_runtime_client;
  clear_error();
  try {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
      cudaGetLastError();
      throw Error(RX_ERR_NO_DEVICE, std::string("no CUDA device available: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
    }
    auto c = std::make_unique<RxClient>();
    c->node_id = node_id;
    c->num_nodes = num_nodes < 1 ? 1 : num_nodes;
    std::vector<int> ords;
    if (allowed_devices && num_allowed_devices > 0) {
      for (int64_t i = 0; i < num_allowed_devices; ++i) {
        if (allowed_devices[i] < 0 || allowed_devices[i] >= count) throw Error(RX_ERR_ARG, "allowed device " + std::to_string(allowed_devices[i]) + " does not exist");
        ords.push_back((int)allowed_devices[i]);
      }
    } else {
      for (int i = 0; i < count; ++i) ords.push_back(i);
    }
    if (ords.size() * (size_t)c->num_nodes > (size_t)kMaxRanks) throw Error(RX_ERR_ARG, "more than " + std::to_string(kMaxRanks) + " devices in the mesh");
    for (size_t i = 0; i < ords.size(); ++i) {
      std::shared_ptr<RxDevice> d = make_device(c.get(), ords[i], (int)i, memory_fraction);
      d->global_id = node_id * (int)ords.size() + (int)i;
      c->devices.push_back(d);
    }
    for (int n = 0; n < c->num_nodes; ++n) {
      if (n == node_id) continue;
      for (size_t i = 0; i < ords.size(); ++i) {
        auto d = std::make_shared<RxDevice>();
        d->client = c.get();
        d->addressable = false;
        d->local_id = (int)i;
        d->global_id = n * (int)ords.size() + (int)i;
        c->remote.push_back(d);
      }
    }
    c->peer_wait_ms = c->num_nodes > 1 ? 8000 : 1000;
    if (const char* w = getenv("RX_PEER_WAIT_MS"))
      if (atoll(w) > 0) c->peer_wait_ms = std::min<int64_t>(atoll(w), 60000);
    const char* mode = getenv("RX_ALLREDUCE");
    if (mode && !strcmp(mode, "nccl")) c->allreduce_mode = 1;
    if (mode && !strcmp(mode, "mailbox")) c->allreduce_mode = 2;
    for (auto& d : c->devices) own(d.get());
    for (auto& d : c->remote) own(d.get());
    return own(c.release());
  } catch (const Error& e) {
    g_err = e.what();
    g_code = e.code;
    if (error) *error = dup_cstr(e.what());
    return nullptr;
  }
}

void FreeClient(RxClient* client) {
  if (!client) return;
  clear_error();
  disown(client);
  for (auto& d : client->devices) disown(d.get());
  for (auto& d : client->remote) disown(d.get());
  rx::destroy_collectives(client);
  for (auto& d : client->devices) {
    cudaSetDevice(d->ordinal);
    cudaStreamSynchronize(d->stream);
    if (d->comm_stream) cudaStreamSynchronize(d->comm_stream);
    d->trim();
    if (d->scratch) cudaFree(d->scratch);
    if (d->flush_buf) cudaFree(d->flush_buf);
    if (d->status) cudaFreeHost(d->status);
    for (auto& s : d->spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
    d->spans.clear();
    d->closed.store(true);
    cudaStreamDestroy(d->stream);
    if (d->comm_stream) cudaStreamDestroy(d->comm_stream);  // joined into `stream` at the end of every execution
    d->comm_stream = nullptr;
    d->stream = nullptr;
    d->scratch = nullptr;
    d->flush_buf = nullptr;
    d->client = nullptr;
  }
  delete client;
}

int ClientNumDevices(RxClient* c) { return c ? c->n_global() : 0; }
int ClientNumAddressableDevices(RxClient* c) { return c ? (int)c->devices.size() : 0; }
int ClientProcessIndex(RxClient* c) { return c ? c->node_id : 0; }

RxDevice* ClientGetDevice(RxClient* c, int id) {
  API_BEGIN
  if (!c) throw Error(RX_ERR_BAD_HANDLE, "null client");
  for (auto& d : c->devices) if (d->global_id == id) return d.get();
  for (auto& d : c->remote) if (d->global_id == id) return d.get();
  throw Error(RX_ERR_ARG, "no device with global id " + std::to_string(id));
  API_END(nullptr)
}
RxDevice* ClientGetAddressableDevice(RxClient* c, int id) {
  API_BEGIN
  if (!c) throw Error(RX_ERR_BAD_HANDLE, "null client");
  if (id < 0 || id >= (int)c->devices.size()) throw Error(RX_ERR_ARG, "no addressable device " + std::to_string(id));
  return c->devices[id].get();
  API_END(nullptr)
}
void ClientGetDevices(RxClient* c, RxDevice** out) {
  for (int i = 0; i < c->n_global(); ++i) out[i] = ClientGetDevice(c, i);
}
void ClientGetAddressableDevices(RxClient* c, RxDevice** out) {
  for (size_t i = 0; i < c->devices.size(); ++i) out[i] = c->devices[i].get();
}
const char* ClientGetPlatformName(RxClient*) { return dup_cstr("cuda"); }

RxClient* DeviceToClient(RxDevice* d) { return d ? d->client : nullptr; }
int64_t PjRtDeviceGetLocalDeviceId(RxDevice* d) { return d->local_id; }
int64_t PjRtDeviceGetGlobalDeviceId(RxDevice* d) { return d->global_id; }
int64_t PjRtDeviceGetLocalHardwareId(RxDevice* d) { return d->ordinal; }
const char* DeviceGetKind(RxDevice* d) { return dup_cstr(d && !d->kind.empty() ? d->kind : std::string("unknown (not addressable from this process)")); }
uint8_t pjrt_device_is_addressable(RxDevice* d) { return d && d->addressable; }
void PjRtDeviceGetAllocatorStats(RxDevice* d, JLAllocatorStats* s) {
  std::lock_guard<std::mutex> lk(d->mu);
  int64_t none = INT64_MIN;
  s->num_allocs = d->num_allocs;
  s->bytes_in_use = d->bytes_in_use;
  s->peak_bytes_in_use = d->peak_bytes_in_use;
  s->largest_alloc_size = d->largest_alloc;
  s->bytes_limit = d->bytes_limit;
  s->bytes_reserved = d->bytes_in_use + d->pool_bytes;
  s->peak_bytes_reserved = d->peak_bytes_in_use + d->peak_pool_bytes;
  s->bytes_reservable_limit = none;
  s->largest_free_block_bytes = d->pool.empty() ? 0 : (int64_t)d->pool.rbegin()->first;
  s->pool_bytes = d->pool_bytes;
  s->peak_pool_bytes = d->peak_pool_bytes;
}

// Device-side waits are bounded; one that ran out leaves a code in the host-mapped status words.
static void check_device_status(RxDevice* d) {
  if (d->status[0]) {
    int s = d->status[0];
    d->status[0] = 0;
    throw Error(RX_ERR_PEER_TIMEOUT, std::string("a peer did not arrive at ") + (s == 2 ? "a halo exchange" : "an all-reduce") + " within the wait limit (status " + std::to_string(s) + ")");
  }
  if (d->status[4]) {
    const int what = d->status[4];
    const long long at = ((long long)d->status[6] << 32) | (unsigned)d->status[5];
    const int extent = d->status[7];
    d->status[4] = d->status[5] = d->status[6] = d->status[7] = 0;
    throw Error(RX_ERR_CUDA, std::string("bounds check: ") + (what >= 200 ? "a result" : "an operand") + " (register " + std::to_string(what % 100) + ") was accessed at element " +
                                 std::to_string(at) + " of a buffer of " + std::to_string(extent) + " elements; the access was skipped");
  }
  for (int w = 1; w <= 2; ++w)
    if (d->status[w]) {
      int s = d->status[w];
      d->status[w] = 0;
      throw Error(RX_ERR_CUDA, std::string(w == 1 ? "stencil" : "gemm") + " kernel: an on-chip copy did not complete within the wait limit (status " + std::to_string(s) + "); results are invalid");
    }
}

static RxBuffer* new_buffer(RxDevice* d, uint64_t ptype, size_t ndim, const int64_t* dims) {
  if (!d || !d->addressable) throw Error(RX_ERR_BAD_HANDLE, "device is null or not addressable from this process");
  DT dt = (DT)ptype;
  if (dt_size(dt) == 0) throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported primitive type code " + std::to_string(ptype));
  auto b = std::make_unique<RxBuffer>();
  b->dt = dt;
  b->dev = d;
  for (size_t i = 0; i < ndim; ++i) {
    if (dims[i] < 0) throw Error(RX_ERR_SHAPE, "negative dimension");
    b->dims.push_back(dims[i]);
  }
  size_t bytes = b->bytes();
  b->st = std::make_shared<Storage>(d, d->alloc(bytes), bytes);
  return own(b.release());
}

RxBuffer* ArrayFromHostBuffer(RxClient* client, void* data, uint64_t ptype, size_t ndim, const int64_t* dims, RxDevice* device) {
  (void)client;
  API_BEGIN
  std::unique_ptr<RxBuffer> b(new_buffer(device, ptype, ndim, dims));
  size_t bytes = b->bytes();
  if (bytes) {
    if (!data) throw Error(RX_ERR_ARG, "null host pointer");
    CK(cudaSetDevice(device->ordinal));
    CK(cudaMemcpyAsync(b->st->ptr, data, bytes, cudaMemcpyHostToDevice, device->stream));
    CK(cudaStreamSynchronize(device->stream));  // host memory is reusable on return
  }
  return b.release();
  API_END(nullptr)
}

RxBuffer* UninitPJRTBuffer(RxClient* client, RxDevice* device, uint64_t ptype, uint64_t ndim, uint64_t* dims) {
  (void)client;
  API_BEGIN
  return new_buffer(device, ptype, (size_t)ndim, (const int64_t*)dims);
  API_END(nullptr)
}

void PjRtBufferFree(RxBuffer* b) {
  disown(b);
  delete b;
}
const int64_t* BufferShape(RxBuffer* b) { return b->dims.data(); }
int64_t BufferNDimensions(RxBuffer* b) { return (int64_t)b->dims.size(); }
int BufferPrimitiveType(RxBuffer* b) { return (int)b->dt; }
RxDevice* BufferToDevice(RxBuffer* b) { return b->dev; }
RxClient* BufferToClient(RxBuffer* b) { return b->dev->client; }
uint8_t BufferOnCPU(RxBuffer*) { return 0; }

static void live(RxBuffer* b) {
  if (!b) throw Error(RX_ERR_BAD_HANDLE, "null buffer");
  if (b->donated.load() || !b->st) throw Error(RX_ERR_DONATED, "buffer was donated to an execution and can no longer be read");
}

void BufferToHost(RxBuffer* b, void* dst) {
  API_BEGIN
  live(b);
  size_t bytes = b->bytes();
  if (bytes) {
    CK(cudaSetDevice(b->dev->ordinal));
    b->st->make_ready();
    CK(cudaMemcpyAsync(dst, b->st->ptr, bytes, cudaMemcpyDeviceToHost, b->dev->stream));
    CK(cudaStreamSynchronize(b->dev->stream));
    check_device_status(b->dev);
  }
  API_END_VOID
}

void* UnsafeBufferPointer(RxBuffer* b) {
  API_BEGIN
  live(b);
  if (b->st->pending) {  // the caller will use the pointer outside this library's streams
    CK(cudaSetDevice(b->dev->ordinal));
    b->st->make_ready();
    CK(cudaStreamSynchronize(b->dev->stream));
    check_device_status(b->dev);
  }
  return b->st->ptr;
  API_END(nullptr)
}

RxBuffer* CopyBufferToDevice(RxBuffer* b, RxDevice* dst) {
  API_BEGIN
  live(b);
  std::unique_ptr<RxBuffer> o(new_buffer(dst, (uint64_t)b->dt, b->dims.size(), b->dims.data()));
  size_t bytes = b->bytes();
  if (bytes) {
    // order after the producer, then copy on the destination's stream
    CK(cudaSetDevice(b->dev->ordinal));
    b->st->make_ready();
    cudaEvent_t ev;
    CK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    CK(cudaEventRecord(ev, b->dev->stream));
    CK(cudaSetDevice(dst->ordinal));
    CK(cudaStreamWaitEvent(dst->stream, ev, 0));
    CK(cudaMemcpyPeerAsync(o->st->ptr, dst->ordinal, b->st->ptr, b->dev->ordinal, bytes, dst->stream));
    CK(cudaStreamSynchronize(dst->stream));
    cudaEventDestroy(ev);
    check_device_status(b->dev);
  }
  return o.release();
  API_END(nullptr)
}

void CopyToBuffer(RxClient*, RxBuffer* b, void* data, size_t offset, size_t size, RxBuffer** bufferP) {
  API_BEGIN
  live(b);
  if (offset + size > b->bytes()) throw Error(RX_ERR_ARG, "copy range exceeds the buffer");
  CK(cudaSetDevice(b->dev->ordinal));
  b->st->make_ready();
  CK(cudaMemcpyAsync((char*)b->st->ptr + offset, data, size, cudaMemcpyHostToDevice, b->dev->stream));
  CK(cudaStreamSynchronize(b->dev->stream));
  if (bufferP) *bufferP = b;
  API_END_VOID
}
void CopyFromBuffer(RxClient*, RxBuffer* b, void* data, size_t offset, size_t size, RxBuffer** bufferP) {
  API_BEGIN
  live(b);
  if (offset + size > b->bytes()) throw Error(RX_ERR_ARG, "copy range exceeds the buffer");
  CK(cudaSetDevice(b->dev->ordinal));
  b->st->make_ready();
  CK(cudaMemcpyAsync(data, (char*)b->st->ptr + offset, size, cudaMemcpyDeviceToHost, b->dev->stream));
  CK(cudaStreamSynchronize(b->dev->stream));
  check_device_status(b->dev);
  if (bufferP) *bufferP = b;
  API_END_VOID
}

void FreeFuture(RxFuture* f) {
  disown(f);
  delete f;
}
uint8_t FutureIsReady(RxFuture* f) {
  if (!f || !f->state) return 1;
  cudaEvent_t ev = f->state->event();
  if (!ev) return 1;
  cudaSetDevice(f->state->dev->ordinal);
  return cudaEventQuery(ev) == cudaSuccess;
}
void FutureAwait(RxFuture* f) {
  API_BEGIN
  if (!f || !f->state) return;
  RxDevice* d = f->state->dev;
  CK(cudaSetDevice(d->ordinal));
  if (cudaEvent_t ev = f->state->event()) CK(cudaEventSynchronize(ev));
  std::lock_guard<std::mutex> g(f->state->error_mu);
  if (f->state->error_code) throw Error(f->state->error_code, f->state->error);
  try {
    check_device_status(d);
  } catch (const Error& e) {
    f->state->error_code = e.code;
    f->state->error = e.what();
    throw;
  }
  API_END_VOID
}

static std::atomic<int64_t> g_plan_cache_hits{0};
int64_t RxPlanCacheHits() { return g_plan_cache_hits.load(); }

RxExecutable* ClientCompileText(RxClient* client, const char* text, size_t len, const char* opts, size_t nopts) {
  (void)opts; (void)nopts;
  API_BEGIN
  if (!client) throw Error(RX_ERR_BAD_HANDLE, "null client");
  std::string s(text, len);
  auto ex = std::make_unique<RxExecutable>();
  ex->client = client;
  // Plan cache keyed by the module text (the in-memory analogue of Reactant's persistent compile cache,
  // src/PersistentCompileCache.jl): compiling the same module again, on any client, reuses the plan.  A plan
  // holds no device state (buffers are bound at launch), so sharing it is safe.
  static std::mutex cache_mu;
  static std::map<std::string, std::shared_ptr<const Plan>> cache;
  static int64_t hits = 0;
  // (the fusion switches are read when the plan is built: a module planned under other settings is another plan)
  std::string key = s;
  for (const char* v : {"RX_GEMM_EPILOGUE", "RX_GEMM_SIMT", "RX_GEMM_1CTA", "RX_NO_MAP_MERGE"}) {
    const char* e = getenv(v);
    key += std::string("\n") + v + "=" + (e ? e : "");
  }
  {
    std::lock_guard<std::mutex> g(cache_mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      ex->plan = it->second;
      ++hits;
      g_plan_cache_hits.store(hits);
    }
  }
  if (!ex->plan) {
    auto mod = parse_module(s);
    std::shared_ptr<const Plan> plan(build_plan(*mod).release());
    std::lock_guard<std::mutex> g(cache_mu);
    if (cache.size() >= 256) cache.clear();
    cache[key] = plan;
    ex->plan = plan;
  }
  if (const char* dir = getenv("RX_DUMP_PLAN")) {
    static int counter = 0;
    std::string path = std::string(dir) + "/plan_" + std::to_string(counter++) + ".json";
    if (FILE* f = fopen(path.c_str(), "w")) {
      std::string d = ex->plan->describe();
      fwrite(d.data(), 1, d.size(), f);
      fclose(f);
    }
  }
  return own(ex.release());
  API_END(nullptr)
}

const char* RxPlanDescribe(const char* text, size_t len) {
  API_BEGIN
  std::string s(text, len);
  auto mod = parse_module(s);
  auto plan = build_plan(*mod);
  return dup_cstr(plan->describe());
  API_END(nullptr)
}

static void specialise_check_steps(const std::vector<Step>& steps, std::string& out, bool& first) {
  for (const Step& st : steps) {
    if (st.kind == StepK::Loop) {
      specialise_check_steps(st.body, out, first);
      continue;
    }
    if (st.kind == StepK::Gemm && st.gemm.has_epilogue) {
      const std::string extra = gemm_epilogue_members(st.gemm);
      for (bool wide : {true, false}) {
        std::string log;
        int64_t bytes = jit_compile_only(st.prog, -1, gemm_epilogue_family(wide), &log, extra.c_str());
        if (bytes < 0) throw Error(RX_ERR_CUDA, std::string("epilogue of step '") + st.note + "' does not compile: " + log);
        out += first ? "" : ",";
        first = false;
        out += "{\"step\":\"" + st.note + "\",\"kernel\":\"" + gemm_epilogue_family(wide) + "\",\"cubin_bytes\":" + std::to_string(bytes) + "}";
      }
      continue;
    }
    if (st.prog.wide) continue;  // f64 programs run on the interpreter kernels only
    std::vector<const char*> families;
    int code = -1;
    if (st.kind == StepK::Map) families = {"k_map_linear<rx::SpecChain>", "k_map_rows<rx::SpecChain, 2>", "k_map_runs<rx::SpecChain, 4>", "k_map_runs<rx::SpecChain, 8>", "k_map_generic<rx::SpecChain, true>"};
    else if (st.kind == StepK::ReduceFull) families = {"k_reduce_full_linear<rx::SpecChain>", "k_reduce_full_rows<rx::SpecChain>", "k_reduce_full_generic<rx::SpecChain>"};
    else if (st.kind == StepK::ReduceRow) families = {"k_reduce_row<rx::SpecChain, 256>", "k_reduce_row<rx::SpecChain, 32>"};
    else if (st.kind == StepK::ReduceCol) families = {"k_reduce_col_vec<rx::SpecChain>", "k_reduce_col<rx::SpecChain>"};
    else continue;
    if (st.kind != StepK::Map) code = red_code(st.red, st.red_dt);
    for (const char* fam : families) {
      std::string log;
      int64_t bytes = jit_compile_only(st.prog, code, fam, &log);
      if (bytes < 0) throw Error(RX_ERR_CUDA, std::string("chain of step '") + st.note + "' does not compile as " + fam + ": " + log);
      out += first ? "" : ",";
      first = false;
      out += "{\"step\":\"" + st.note + "\",\"kernel\":\"" + fam + "\",\"cubin_bytes\":" + std::to_string(bytes) + "}";
    }
  }
}

const char* RxPlanSpecialiseCheck(const char* text, size_t len) {
  API_BEGIN
  std::string s(text, len);
  auto mod = parse_module(s);
  auto plan = build_plan(*mod);
  std::string out = "[";
  bool first = true;
  specialise_check_steps(plan->steps, out, first);
  out += "]";
  return dup_cstr(out);
  API_END(nullptr)
}

void RxChainSpecialiser(int64_t min_elems) { rx::jit_set_min_elems(min_elems); }
void RxChainSpecialiserStats(int64_t* out5) {
  if (out5) rx::jit_stats(out5);
}

void ExecutableFree(RxExecutable* e) {
  disown(e);
  delete e;
}
RxClient* PjRtLoadedExecutableGetClient(RxExecutable* e) { return e->client; }
int PjRtLoadedExecutableNumReplicas(RxExecutable*) { return 1; }
int PjRtLoadedExecutableNumPartitions(RxExecutable* e) { return (int)e->plan->num_partitions; }
int RxExecutableNumParameters(RxExecutable* e) { return (int)e->plan->arg_types.size(); }
int RxExecutableNumResults(RxExecutable* e) { return (int)e->plan->results.size(); }
int RxExecutableParameterShardedDim(RxExecutable* e, int i) { return e->plan->arg_sharded_dim.at(i); }
int RxExecutableResultShardedDim(RxExecutable* e, int i) { return e->plan->results.at(i).sharded_dim; }
int RxExecutableParameterAlias(RxExecutable* e, int i) { return e->plan->arg_alias.at(i); }
const char* RxExecutableDescribe(RxExecutable* e) { return dup_cstr(e->plan->describe()); }

uint8_t RxOwns(const void* handle) {
  std::lock_guard<std::mutex> g(g_own_mu);
  return g_owned.count(handle) ? 1 : 0;
}

typedef void (*ExecShardedFn)(void*, int, void**, void*, uint8_t*, int, void**, uint8_t*, void**);
typedef void (*ExecFn)(void*, int, void**, uint8_t*, int, void**, uint8_t*, void**);
static ExecShardedFn g_other_execute_sharded = nullptr;
static ExecFn g_other_execute = nullptr;
void RxSetForeignExecute(void* execute_sharded, void* execute) {
  g_other_execute_sharded = (ExecShardedFn)execute_sharded;
  g_other_execute = (ExecFn)execute;
}

void XLAExecuteSharded(RxExecutable* exec, int num_args, RxBuffer** op_args, RxDevice* device, uint8_t* is_arg_donatable, int num_results,
                       RxBuffer** op_results, uint8_t* futures, RxFuture** future_results) {
  if (g_other_execute_sharded && exec && !RxOwns(exec)) {  // another runtime's executable: not ours to run
    g_other_execute_sharded(exec, num_args, (void**)op_args, device, is_arg_donatable, num_results, (void**)op_results, futures, (void**)future_results);
    return;
  }
  API_BEGIN
  if (!exec || !device) throw Error(RX_ERR_BAD_HANDLE, "null executable or device");
  execute(exec, {device}, op_args, num_args, is_arg_donatable, num_results, op_results, futures, future_results);
  API_END_VOID
}

void XLAExecute(RxExecutable* exec, int op_args_len, RxBuffer** op_args, uint8_t* is_arg_donatable, int num_results, RxBuffer** op_results,
                uint8_t* futures, RxFuture** future_results) {
  if (g_other_execute && exec && !RxOwns(exec)) {
    g_other_execute(exec, op_args_len, (void**)op_args, is_arg_donatable, num_results, (void**)op_results, futures, (void**)future_results);
    return;
  }
  API_BEGIN
  if (!exec) throw Error(RX_ERR_BAD_HANDLE, "null executable");
  std::vector<RxDevice*> devs;
  for (auto& d : exec->client->devices) devs.push_back(d.get());
  if (exec->plan->num_partitions == 1) devs.resize(1);
  int nd = (int)devs.size();
  if (op_args_len % nd) throw Error(RX_ERR_ARG, "argument count " + std::to_string(op_args_len) + " is not a multiple of the device count " + std::to_string(nd));
  execute(exec, devs, op_args, op_args_len / nd, is_arg_donatable, num_results, op_results, futures, future_results);
  API_END_VOID
}

int RxClientSetPeerWaitMs(RxClient* c, int64_t ms) {
  API_BEGIN
  if (!c) throw Error(RX_ERR_BAD_HANDLE, "null client");
  if (ms < 1 || ms > 60000) throw Error(RX_ERR_ARG, "the peer wait must be between 1 and 60000 ms");
  c->peer_wait_ms = ms;
  return 0;
  API_END(g_code)
}
int RxCollectivesUniqueId(uint8_t* id128) {
  API_BEGIN
  rx::nccl_unique_id(id128);
  return 0;
  API_END(g_code)
}
int RxClientInitCollectives(RxClient* c, const uint8_t* id128) {
  API_BEGIN
  rx::init_nccl(c, id128);
  return 0;
  API_END(g_code)
}
int RxClientMailboxHandle(RxClient* c, int local_device, uint8_t* handle64) {
  API_BEGIN
  rx::mailbox_handle(c, local_device, handle64);
  return 0;
  API_END(g_code)
}
int RxClientOpenMailboxes(RxClient* c, const uint8_t* handles, int n) {
  API_BEGIN
  rx::open_mailboxes(c, handles, n);
  return 0;
  API_END(g_code)
}

RxEvent* RxEventRecord(RxDevice* d) {
  API_BEGIN
  auto* e = new RxEvent();
  e->dev = d;
  e->keep = d->shared_from_this();
  CK(cudaSetDevice(d->ordinal));
  CK(cudaEventCreate(&e->ev));
  CK(cudaEventRecord(e->ev, d->stream));
  return e;
  API_END(nullptr)
}
void RxEventSynchronize(RxEvent* e) {
  API_BEGIN
  CK(cudaSetDevice(e->dev->ordinal));
  CK(cudaEventSynchronize(e->ev));
  API_END_VOID
}
float RxEventElapsedMs(RxEvent* a, RxEvent* b) {
  API_BEGIN
  float ms = 0;
  CK(cudaSetDevice(a->dev->ordinal));
  CK(cudaEventElapsedTime(&ms, a->ev, b->ev));
  return ms;
  API_END(-1.f)
}
void RxEventFree(RxEvent* e) {
  if (!e) return;
  cudaSetDevice(e->dev->ordinal);
  cudaEventDestroy(e->ev);
  delete e;
}
void RxDeviceSynchronize(RxDevice* d) {
  API_BEGIN
  CK(cudaSetDevice(d->ordinal));
  CK(cudaStreamSynchronize(d->stream));
  if (d->comm_stream) CK(cudaStreamSynchronize(d->comm_stream));
  check_device_status(d);
  API_END_VOID
}
void RxDeviceJoinStreams(RxDevice* d) {
  API_BEGIN
  if (d->comm_stream) {
    CK(cudaSetDevice(d->ordinal));
    cudaEvent_t ev;
    CK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    CK(cudaEventRecord(ev, d->comm_stream));
    CK(cudaStreamWaitEvent(d->stream, ev, 0));
    cudaEventDestroy(ev);
  }
  API_END_VOID
}
void* RxHostAlloc(size_t bytes) {
  API_BEGIN
  void* p = nullptr;
  cudaError_t e = cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocPortable);
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw Error(RX_ERR_CUDA, std::string("cannot allocate ") + std::to_string(bytes) + " bytes of page-locked host memory: " + cudaGetErrorString(e));
  }
  return p;
  API_END(nullptr)
}
void RxHostFree(void* p) {
  if (p) cudaFreeHost(p);
  cudaGetLastError();
}
uint64_t RxDeviceKernelLaunches(RxDevice* d) { return d->launches; }
void RxDeviceSetProfiling(RxDevice* d, int on) { d->profiling = on != 0; }
const char* RxDeviceProfileJson(RxDevice* d) {
  API_BEGIN
  CK(cudaSetDevice(d->ordinal));
  CK(cudaStreamSynchronize(d->stream));
  for (auto& s : d->spans) {
    float ms = 0;
    cudaEventElapsedTime(&ms, s.a, s.b);
    auto& p = d->prof[s.kind];
    p.first += 1;
    p.second += ms;
    cudaEventDestroy(s.a);
    cudaEventDestroy(s.b);
  }
  d->spans.clear();
  std::ostringstream os;
  os << "{";
  bool first = true;
  for (auto& kv : d->prof) {
    os << (first ? "" : ",") << "\"" << kv.first << "\":{\"launches\":" << kv.second.first << ",\"ms\":" << kv.second.second << "}";
    first = false;
  }
  os << "}";
  d->prof.clear();
  return dup_cstr(os.str());
  API_END(nullptr)
}
void* RxDeviceStream(RxDevice* d) { return (void*)d->stream; }
void RxDeviceFlushL2(RxDevice* d) {
  API_BEGIN
  CK(cudaSetDevice(d->ordinal));
  if (!d->flush_buf) {
    d->flush_bytes = (size_t)256 << 20;
    CK(cudaMalloc(&d->flush_buf, d->flush_bytes));
  }
  CK(cudaMemsetAsync(d->flush_buf, 0, d->flush_bytes, d->stream));
  API_END_VOID
}

}  // extern "C"
