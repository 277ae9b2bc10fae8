// Exchange of the boundary rows of a row-sharded 2-D f32 array between neighbouring devices of a 1-D mesh (what the
// SPMD partitioner emits as collective-permutes for shifted slices, test/core/sharding/optimize_comm.jl:48-56), as
// device code for ONE CTA: used by the stand-alone exchange kernel and, between sweeps, by the whole-loop stencil
// kernel.  A device's block is [up halo][owned rows][down halo], `cols` floats per row.  Rows travel as plain peer
// stores into a window beside the RECEIVER's mailbox (so no tensor map and no load ever covers another GPU's
// memory), followed by a sequence number; the receiver polls its own memory with a bounded wait and copies the
// window into its halos.  Two windows alternate by sequence parity: a sender can only be two exchanges ahead of a
// receiver after having received rows which that receiver sent after it emptied the window in question.
#pragma once
#include "rx_runtime.h"

namespace rx {

struct HaloArgs {
  float* block;            // this device's rows: [up halo][owned][down halo], `cols` floats each
  long long rows_local, cols;
  int up, down;            // halo heights
  int rank, n;
  unsigned epoch;          // sequence number of this exchange
  long long poll_limit;
  unsigned long long* mail_self;
  unsigned long long* mail_above;  // mailbox of rank - 1 (unused for rank 0)
  unsigned long long* mail_below;  // mailbox of rank + 1 (unused for the last rank)
};

__device__ __forceinline__ float* halo_window(unsigned long long* mailbox, int parity, int dir) {
  return (float*)((char*)mailbox + kHaloWindowOffset) + ((size_t)(parity * 2 + dir) * kHaloMaxRows) * kHaloMaxCols;
}
__device__ __forceinline__ volatile unsigned* halo_flag(unsigned long long* mailbox, int parity, int dir) {
  return (volatile unsigned*)((char*)mailbox + kHaloFlagsOffset) + parity * 2 + dir;
}

// `rows` rows of `c4` float4 from `src` (row pitch `sp` float4) to `dst` (row pitch `dp`), by all threads of the CTA.
// A thread issues all its loads of a row (up to 8) before the first store: the copy then costs a few memory round
// trips instead of one per element, which is what the exchange CTA of a long-running kernel has to hide behind a pass.
// VOLATILE: read with ld.volatile (rows a peer has just written), else past L1 (rows other CTAs have just written).
template <bool VOLATILE>
__device__ __noinline__ void halo_copy_rows(float4* dst, int dp, const float4* src, int sp, int rows, int c4) {
  constexpr int U = 8;
  const int step = (int)blockDim.x;
#pragma unroll 1
  for (int r = 0; r < rows; ++r) {
    const float4* s = src + (long long)r * sp + threadIdx.x;
    float4* d = dst + (long long)r * dp + threadIdx.x;
#pragma unroll 1
    for (int i0 = (int)threadIdx.x; i0 < c4; i0 += U * step, s += U * step, d += U * step) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * step < c4) v[u] = VOLATILE ? __ldcv(s + u * step) : __ldcg(s + u * step);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * step < c4) d[u * step] = v[u];
    }
  }
}

// Every thread of the CTA calls this (the rows to send are read past L1: inside a long-running kernel the CTA may
// hold lines of an earlier version of the same rows); rows are whole multiples of 4 floats (checked by the launcher), so everything
// moves as float4.  False (for all threads) if a neighbour's rows did not arrive within the bounded wait: the halos
// then keep their old rows and the caller reports the failure.
__device__ __forceinline__ bool halo_exchange_cta(const HaloArgs& a) {
  __shared__ int halo_failed;
  const int parity = a.epoch & 1;
  const int c4 = (int)(a.cols >> 2);  // at most kHaloMaxCols / 4
  if (threadIdx.x == 0) halo_failed = 0;
  // send: my first `down` owned rows to the device above (they are its lower halo), my last `up` owned rows to the device below
  if (a.rank > 0 && a.down > 0) {
    const float4* src = (const float4*)(a.block + (long long)a.up * a.cols);
    float4* dst = (float4*)halo_window(a.mail_above, parity, 1);
    halo_copy_rows<false>(dst, kHaloMaxCols / 4, src, c4, a.down, c4);
  }
  if (a.rank + 1 < a.n && a.up > 0) {
    const float4* src = (const float4*)(a.block + a.rows_local * a.cols);  // block row (up + rows_local - up)
    float4* dst = (float4*)halo_window(a.mail_below, parity, 0);
    halo_copy_rows<false>(dst, kHaloMaxCols / 4, src, c4, a.up, c4);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (a.rank > 0) *halo_flag(a.mail_above, parity, 1) = a.epoch;
    if (a.rank + 1 < a.n) *halo_flag(a.mail_below, parity, 0) = a.epoch;
    __threadfence_system();
    // receive: bounded wait for the neighbours' sequence numbers
    for (int dir = 0; dir < 2; ++dir) {
      if (dir == 0 ? a.rank == 0 : a.rank + 1 >= a.n) continue;
      volatile unsigned* f = halo_flag(a.mail_self, parity, dir);
      long long spins = 0;
      while (*f != a.epoch) {
        if (++spins > a.poll_limit) { halo_failed = 1; break; }
        __nanosleep(kPeerPollNs);
      }
    }
  }
  __syncthreads();
  if (halo_failed) return false;
  __threadfence_system();
  if (a.rank > 0 && a.up > 0) {
    const float4* src = (const float4*)halo_window(a.mail_self, parity, 0);
    float4* dst = (float4*)a.block;
    halo_copy_rows<true>(dst, c4, src, kHaloMaxCols / 4, a.up, c4);
  }
  if (a.rank + 1 < a.n && a.down > 0) {
    const float4* src = (const float4*)halo_window(a.mail_self, parity, 1);
    float4* dst = (float4*)(a.block + (a.up + a.rows_local) * a.cols);
    halo_copy_rows<true>(dst, c4, src, kHaloMaxCols / 4, a.down, c4);
  }
  return true;
}

}  // namespace rx
