// All-reduce of sharded reductions over the mesh axis: NCCL, or the NVLink
// mailbox kernel for single-word payloads.  In the reference both the
// partitioning and the NCCL call are made by XLA
// (deps/ReactantExtra/API.cpp:1487-1497); nothing in the Julia tree emits a
// collective.
#pragma once
#include <functional>
#include <vector>

#include "rx_runtime.h"

namespace rx {

void nccl_unique_id(uint8_t* id128);
void init_nccl(RxClient* c, const uint8_t* id128);
void mailbox_handle(RxClient* c, int local_device, uint8_t* handle64);
void open_mailboxes(RxClient* c, const uint8_t* handles, int n_global);
void destroy_collectives(RxClient* c);

// Sum `st.count` f32 values at ptr(k) on dev(k) for every local device k with the
// matching values of all other ranks of the mesh; every rank ends with the same bits.
// on_comm_stream: enqueue on each device's communication stream instead of its compute stream (the caller
// orders the two with events); only the NCCL path honours it.
void run_allreduce(RxClient* c, const Step& st, size_t n_local, const std::function<RxDevice*(size_t)>& dev,
                   const std::function<void*(size_t)>& ptr, bool on_comm_stream = false);

// Halo exchange of a row-sharded array (one launch per device): device g sends the first `down` rows it owns to the
// lower halo of device g - 1 and the last `up` rows it owns to the upper halo of device g + 1, then waits -- bounded by
// the client's peer wait -- for the rows its own neighbours send and copies them into its halos.  `block(k)` is local
// device k's allocation: (rows_local + up + down) rows of `cols` floats, owned rows starting at row `up`.  The rows
// travel as plain peer stores into a window next to the receiver's all-reduce mailbox (the receiver's own memory, so the
// stencil kernel's tensor maps never cover peer memory), two windows alternating by sequence number.
void run_halo_exchange(RxClient* c, size_t n_local, const std::function<RxDevice*(size_t)>& dev, const std::function<float*(size_t)>& block, int64_t rows_local,
                       int64_t cols, int up, int down);

// For kernels that do the exchange themselves (the whole-loop stencil kernel): whether rows of `cols` floats with these
// halo heights fit the exchange windows and the peer mailboxes are open; the device-independent part of the arguments
// for local device d; and a run of `count` consecutive sequence numbers (the first is returned).
bool halo_exchange_possible(RxClient* c, int64_t cols, int up, int down);
struct HaloArgs;
void halo_fill_args(RxClient* c, RxDevice* d, int64_t rows_local, int64_t cols, int up, int down, HaloArgs* out);
unsigned halo_reserve_epochs(RxClient* c, unsigned count);

// If a single-word all-reduce can go through the mailboxes, advance the epoch and fill
// one FusedAllReduce per local device (to be handed to the producing reduce kernel).
bool prepare_fused_allreduce(RxClient* c, const Step& ar_step, const std::vector<RxDevice*>& devs, std::vector<FusedAllReduce>* out);

}  // namespace rx
