// 2-D stencil step with TMA-staged tiles.
//
// out[r][c] = chain(src[r + dy_k][c + dx_k], k = 0..taps)   for a window of a
// row-major f32 array -- the fused form of the slice / add / multiply /
// dynamic_update_slice sequence Reactant traces for
//     B[2:end-1, 2:end-1] = 0.2f0 .* (A[2:end-1, 2:end-1] .+ A[1:end-2, 2:end-1] .+ ...)
// (src/Indexing.jl:552-627 getindex -> stablehlo.slice, :350-446 setindex! ->
// dynamic_update_slice; benchmark/polybench/stencil.jl:263-289).
//
// Each CTA works through 32 x 252 (or 248) output tiles: every n-th one in the single-launch
// kernel, the next free one of a per-pass queue in the whole-loop kernel.  One elected thread
// issues a cp.async.bulk.tensor.2d (TMA) load of the tile plus its halo into a
// two-stage shared-memory ring, signalled through mbarriers; the other threads
// compute the previous tile meanwhile.  Halo rows/columns are re-read from L2,
// not HBM (neighbouring tiles are in flight at the same time), so DRAM traffic
// stays at one read and one write per element.  The adds are evaluated in the
// traced order and nothing is contracted into an FMA, so results are bit-exact
// with the CPU evaluation.  TMA loads start on 16-byte boundaries (x is rounded
// down to a multiple of 4 floats and the box is widened); no multicast is used.
#include "rx_device.cuh"
#include "rx_stencil.h"
#include "rx_halo.cuh"
#include "rx_tma.h"

namespace rx {

namespace {

constexpr int HALO_H = 8;
constexpr int BOX_W = 256;                  // TMA boxes are at most 256 elements wide; a tile is BOX_W - halo columns
constexpr int STAGES = 2;                   // a deeper ring measured slower (more tiles in flight hurt DRAM locality)
constexpr int kMaxTaps = 8;
constexpr long long kWaitLimit = 2000000;  // bounded mbarrier polling


struct StencilParams {
  float* dst;
  int64_t rows, cols, dst_ld, dst_off;
  int x_base, y_base, x_shift;  // tensor coordinates of window column/row 0; columns skipped inside the box
  int box_h;
  int tw;       // output columns per tile
  int cross;    // taps are (centre, left, right, up, down) of a radius-1 cross, in that order
  int n_taps;
  int dy[kMaxTaps], dx[kMaxTaps];
  int tiles_x, tiles_y;
  int* status;
  long long dst_extent;  // bounds-checked builds: elements in the destination buffer, and where a miss is recorded
  int* bounds;
};

// Row-sharded arrays: the tile rows that hold rows the neighbouring devices wait for (up to two at either end of the
// window) come first in a sweep's order: the first tile row, and the last one -- or the last two, when the last holds
// a single row.  edge_tail() is how many tile rows at the end, edge_tiles() how many tiles in all.
__device__ __forceinline__ int edge_tail(long long rows, int tiles_y, int th) {
  if (tiles_y < 2) return 0;
  return (rows - (long long)(tiles_y - 1) * th >= 2 || tiles_y < 3) ? 1 : 2;
}
__device__ __forceinline__ int edge_tiles(long long rows, int tiles_x, int tiles_y, int th) { return (1 + edge_tail(rows, tiles_y, th)) * tiles_x; }

// Shared-memory accesses by 32-bit shared address: the tile pointers reach the sweep functions as generic pointers,
// and generic loads are slower than ld.shared and wait on the long scoreboard.  Volatile, so that they stay behind
// the mbarrier wait and the CTA barriers they follow in program order.
__device__ __forceinline__ float lds(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v)); }

// the five values of a radius-1 cross, added in the order the traced program adds them
//   ORDER 0: centre, left, right, up, down      (the swap spelling, and the pad / concatenate spellings)
//   ORDER 1: centre, up, down, right, left      (benchmark/polybench/stencil.jl:263-289 after the layout fold)
template <int ORDER>
__device__ __forceinline__ float cross_sum(float c, float l, float r, float u, float d) {
  if (ORDER == 0) return __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(c, l), r), u), d);
  return __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(c, u), d), r), l);
}

// B consecutive rows of one column of a radius-1 cross over a tile in shared memory.  `qa` is the shared address of
// the first row's centre; `up` and `c` hold the two values above the row after it and are carried on.  All 3 B loads
// are issued before the arithmetic, so that B independent chains of adds are in flight.
constexpr int kRowBatch = 8;
template <int B, int ORDER, class Store>
__device__ __forceinline__ void cross_rows(uint32_t qa, float& up, float& c, float k, Store&& store) {
  constexpr uint32_t R = BOX_W * sizeof(float);
  float v[B + 2], l[B], r[B];
  v[0] = up;
  v[1] = c;
#pragma unroll
  for (int j = 0; j < B; ++j) {
    l[j] = lds(qa + j * R - 4);
    r[j] = lds(qa + j * R + 4);
    v[j + 2] = lds(qa + (j + 1) * R);
  }
#pragma unroll
  for (int j = 0; j < B; ++j) store(j, __fmul_rn(k, cross_sum<ORDER>(v[j + 1], l[j], r[j], v[j], v[j + 2])));
  up = v[B];
  c = v[B + 1];
}

// rows [0, n) of a column: batches of kRowBatch, then pairs, then one
template <int ORDER, class Store, class Advance>
__device__ __forceinline__ void cross_column(uint32_t qa, int n, float k, Store&& store, Advance&& advance) {
  constexpr uint32_t R = BOX_W * sizeof(float);
  float up = lds(qa - R), c = lds(qa);
  int r = 0;
  for (; r + kRowBatch <= n; r += kRowBatch) {
    cross_rows<kRowBatch, ORDER>(qa, up, c, k, store);
    qa += kRowBatch * R;
    advance(kRowBatch);
  }
  for (; r + 2 <= n; r += 2) {
    cross_rows<2, ORDER>(qa, up, c, k, store);
    qa += 2 * R;
    advance(2);
  }
  if (r < n) cross_rows<1, ORDER>(qa, up, c, k, store);
}

// One sweep of this CTA's tiles.  `it` counts the tiles this CTA has processed since the kernel started: it
// selects the ring stage and the mbarrier parity, so that several sweeps can share one ring.  On entry every
// stage is drained.  Returns false if a load did not arrive within the wait limit.
// `reverse` walks the tile list from its far end: consecutive sweeps of one launch alternate direction, so that a
// sweep starts on the part of the arrays the previous sweep touched last, which is still in L2.
// `cta` of `ncta` CTAs share the tile list.  With `edge_rows` the tiles of the first and last tile row come first
// (they hold the rows a row-sharded array's neighbours are waiting for), each counted in *edge_counter once its
// rows are written, and only the remaining tiles alternate direction.
// With `queue` (a counter in device memory, zero when the sweep starts) the CTAs take the positions of the sweep's
// order one by one as they become free instead of every ncta-th one: CTAs do not run at the same speed (by 20 %
// between the first and the last to finish a pass of 30 tiles each), and what the slowest one needs is what the
// grid barrier after the sweep waits for.  A position is claimed one step before its load is issued, so the
// atomic's latency is off the issuing thread's path.  Every CTA's first position is its own number, the queue hands
// out the ones from ncta on: the tiles at the front of the order (the edge tiles of a row-sharded array, which the
// exchange waits for) are then all worked on at once instead of two or three in a row by the CTAs that start first.
template <bool FAST5, int TH>
__device__ __forceinline__ bool stencil_sweep(const CUtensorMap* tmap, const StencilParams& p, const VmProgram* P, float fast_c, float* const* tile, uint64_t* bars,
                                              int& it, bool reverse = false, int cta = blockIdx.x, int ncta = gridDim.x, bool edge_rows = false,
                                              unsigned* edge_counter = nullptr, unsigned* queue = nullptr) {
  __shared__ int claimed[STAGES];  // position in the sweep's order of the tile in (or on its way into) each stage; >= ntiles: none
  const uint32_t bytes = (uint32_t)(BOX_W * p.box_h * sizeof(float));
  const int ntiles = p.tiles_x * p.tiles_y;
  const int n_edge = edge_rows ? edge_tiles(p.rows, p.tiles_x, p.tiles_y, TH) : 0;
  // position in this sweep's order -> tile
  auto tile_of = [&](int t) {
    if (t < n_edge) return t < p.tiles_x ? t : ntiles - n_edge + t;  // the first tile row, then the last ones
    if (!edge_rows) return reverse ? ntiles - 1 - t : t;
    const int u = t - n_edge, n_int = ntiles - n_edge;
    return p.tiles_x + (reverse ? n_int - 1 - u : u);
  };
  auto issue = [&](int t, int s) {
    t = tile_of(t);
    int ty = t / p.tiles_x, tx = t - ty * p.tiles_x;
    mbar_expect_tx(&bars[s], bytes);
    tma_load_2d(tile[s], tmap, p.x_base + tx * p.tw, p.y_base + ty * TH, &bars[s]);
  };
  // thread 0: claims made; the position claimed but not yet issued (its value is first looked at one step later, so
  // the warp does not wait for the atomic)
  unsigned n_claims = 0, pending = 0;
  auto claim = [&]() -> unsigned {
    const unsigned k = n_claims++;
    if (!queue) return (unsigned)cta + k * (unsigned)ncta;
    return k == 0 ? (unsigned)cta : (unsigned)ncta + atomicAdd(queue, 1u);  // the first ncta positions go one to each CTA
  };
  if (threadIdx.x == 0) {
    for (int q = 0; q < STAGES - 1; ++q) {
      const int t = (int)min(claim(), (unsigned)ntiles);
      claimed[(it + q) % STAGES] = t;
      if (t < ntiles) issue(t, (it + q) % STAGES);
    }
    pending = claim();
  }
  __syncthreads();
  for (;; ++it) {
    int s = it % STAGES;
    uint32_t parity = (it / STAGES) & 1;
    const int t = claimed[s];
    if (t >= ntiles) break;
    if (threadIdx.x == 0) {  // the other stage was drained before the last barrier, and its position read before that
      const int sn = (it + STAGES - 1) % STAGES, tn = (int)min(pending, (unsigned)ntiles);
      claimed[sn] = tn;
      if (tn < ntiles) issue(tn, sn);
      pending = claim();
    }
    if (!mbar_wait(&bars[s], parity, kWaitLimit)) return false;
    const int tt = tile_of(t);
    int ty = tt / p.tiles_x, tx = tt - ty * p.tiles_x;
    int64_t c = (int64_t)tx * p.tw + threadIdx.x;
    int64_t r0 = (int64_t)ty * TH;
    const float* sm = tile[s] + p.x_shift + threadIdx.x;
    if ((int)threadIdx.x < p.tw && c < p.cols) {
      float* out = p.dst + p.dst_off + r0 * p.dst_ld + c;
      int rmax = (int)min((int64_t)TH, p.rows - r0);
#if RX_BOUNDS
      // this thread writes one element per row of the tile: first and last must lie inside the destination
      if (rmax > 0 && !(rx_in_bounds(p.bounds, p.dst_extent, p.dst_off + r0 * p.dst_ld + c, 1, 299) &&
                        rx_in_bounds(p.bounds, p.dst_extent, p.dst_off + (r0 + rmax - 1) * p.dst_ld + c, 1, 299)))
        rmax = 0;
#endif
      if (FAST5) {
        const float k = fast_c;
        if (p.cross) {
          // taps are centre, left, right, up, down in that evaluation order: slide a three-row window
          // down the column so that each output costs three shared-memory reads instead of five
          const uint32_t qa = smem_u32(sm + p.dx[0] + p.dy[0] * BOX_W);  // the centre tap of the first row
          const int64_t ld = p.dst_ld;
          cross_column<0>(qa, rmax, k, [&](int j, float v) { out[j * ld] = v; }, [&](int n) { out += n * ld; });
        } else {
          const int o0 = p.dy[0] * BOX_W + p.dx[0], o1 = p.dy[1] * BOX_W + p.dx[1], o2 = p.dy[2] * BOX_W + p.dx[2], o3 = p.dy[3] * BOX_W + p.dx[3],
                    o4 = p.dy[4] * BOX_W + p.dx[4];
#pragma unroll 4
          for (int r = 0; r < rmax; ++r) {
            const float* q = sm + r * BOX_W;
            float v = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(q[o0], q[o1]), q[o2]), q[o3]), q[o4]);
            out[(int64_t)r * p.dst_ld] = __fmul_rn(k, v);
          }
        }
      } else {
        int64_t idx0[kMaxRank] = {0, 0, 0, 0};
        for (int r = 0; r < rmax; ++r) {
          const float* q = sm + r * BOX_W;
          __align__(16) uint32_t R[kVmMaxRegs][1];
          for (int k = 0; k < P->n_leaves; ++k) R[P->leaf[k].reg][0] = f2u(q[p.dy[k] * BOX_W + p.dx[k]]);
          vm_exec<1>(*P, R, idx0);
          out[(int64_t)r * p.dst_ld] = u2f(R[P->out[0].reg][0]);
        }
      }
    }
    __syncthreads();  // every thread is done with stage s before it is refilled
    if (t < n_edge && threadIdx.x == 0) {
      __threadfence();  // the tile's rows, written by all threads before the barrier, precede the count
      atomicAdd(edge_counter, 1u);
    }
  }
  return true;
}

// a load may still be in flight into this CTA's shared memory after a failed wait: give it a bounded chance to land
__device__ __forceinline__ void stencil_drain(uint64_t* bars) {
  __syncthreads();
  if (threadIdx.x == 0)
    for (int s = 0; s < STAGES; ++s) mbar_wait(&bars[s], 0, kWaitLimit) || mbar_wait(&bars[s], 1, kWaitLimit);
}

template <bool FAST5, int TH>
__global__ void __launch_bounds__(256) k_stencil_tma(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ StencilParams p,
                                                     const __grid_constant__ VmProgram P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[STAGES];
  float* tile[STAGES];
  const int stage_floats = BOX_W * p.box_h;
  uintptr_t base = ((uintptr_t)smem_raw + 127) & ~(uintptr_t)127;  // 128-byte aligned stages
#pragma unroll
  for (int s = 0; s < STAGES; ++s) tile[s] = (float*)base + (size_t)s * stage_floats;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  int it = 0;
  if (!stencil_sweep<FAST5, TH>(&tmap, p, &P, P.fast_c, tile, bars, it)) {
    if (threadIdx.x == 0) *p.status = 2;
    stencil_drain(bars);
  }
}

// ---- two sweeps per pass over memory (temporal blocking) ----------------------------------------------------
// A Jacobi-style loop alternates between two arrays: sweep s reads X[s % 2] and writes the update window of
// X[(s + 1) % 2]; outside the window each array keeps its own values for ever.  Two consecutive sweeps can therefore
// be done on one tile while it is on chip: load the tile of state s with a halo of two (one bulk copy), compute
// state s + 1 on the tile plus a halo of one into shared memory -- taking the points outside the window from the
// other array, whose values there never change -- then state s + 2 on the tile itself, and store only that.  Every
// point is computed by the same operations in the same order as in two separate sweeps, so the result is the same
// bits; the arrays cross HBM once per two sweeps instead of twice (plus 7 % redundant work on the halos).
// State s + 2 belongs in the array state s sits in, which other CTAs are still reading: the fused passes ping-pong
// between that array and a scratch array with the same border, and the last two (three, for an odd count) sweeps of
// the loop run one at a time, so that both carried arrays end with exactly the contents the unfused loop leaves.
struct FuseParams {
  int n_fused;              // fused double sweeps before the remaining single sweeps (0: none)
  float* buf[2];            // [0]: the array the first sweep reads; [1]: scratch array of the same shape and border
  const float* other;       // the other carried array
  long long ld, rows_total;
  long long r0, r1, c0, c1; // update window [r0, r1) x [c0, c1), the same for both directions
  long long m0, m1;         // rows on which the intermediate state is computed: [r0, r1), or one more row on a side where a
                            // row-sharded device's rows border a neighbour's (those rows are the neighbour's to write, but
                            // their intermediate values are needed here)
  int order;                // in which order the five values of the cross are added (cross_sum)
  int xs;                   // columns skipped at the left of a box so that the copy starts on a 16-byte boundary
  int tw2, tiles_x2, tiles_y2;
  float k;
  int* status;
  long long extent;         // bounds-checked builds
  int* bounds;
};
struct alignas(64) FuseMaps { CUtensorMap m[3]; };  // buf[0] and buf[1] with (TH + 4)-row boxes; buf[1] with the single-sweep box

template <int TH, int ORDER>
__device__ __forceinline__ bool stencil_sweep2(const CUtensorMap* tmap, const FuseParams& f, float* dst, float* const* tile, float* mid, uint64_t* bars, int& it,
                                               bool reverse, int cta, int ncta, bool edge_rows = false, unsigned* edge_counter = nullptr, unsigned* queue = nullptr) {
  __shared__ int claimed[STAGES];
  constexpr int BH = TH + 4;
  const uint32_t bytes = (uint32_t)(BOX_W * BH * sizeof(float));
  const int ntiles = f.tiles_x2 * f.tiles_y2;
  const float k = f.k;
  const int n_edge = edge_rows ? edge_tiles(f.r1 - f.r0, f.tiles_x2, f.tiles_y2, TH) : 0;
  // position in this pass's order -> tile (first and last tile rows first when the rows are traded with neighbours)
  auto tile_of = [&](int t) {
    if (t < n_edge) return t < f.tiles_x2 ? t : ntiles - n_edge + t;
    if (!edge_rows) return reverse ? ntiles - 1 - t : t;
    const int u = t - n_edge, n_int = ntiles - n_edge;
    return f.tiles_x2 + (reverse ? n_int - 1 - u : u);
  };
  auto issue = [&](int t, int s) {
    t = tile_of(t);
    const int ty = t / f.tiles_x2, tx = t - ty * f.tiles_x2;
    mbar_expect_tx(&bars[s], bytes);
    // the box starts two points up and to the left of the tile (minus the alignment columns); negative coordinates
    // read the fill value, which is never used: those positions come from the other array
    tma_load_2d(tile[s], tmap, (int)(f.c0 + (long long)tx * f.tw2 - 2 - f.xs), (int)(f.r0 + (long long)ty * TH - 2), &bars[s]);
  };
  // Only the first of the two steps on a tile reads the ring stage, so the stage is refilled as soon as that step is
  // over: the whole ring is in flight at the start, and the load of the CTA's next tile but one overlaps the second
  // step on this tile and everything on the next.  Positions come from `queue` as in stencil_sweep.
  unsigned n_claims = 0, pending = 0;
  auto claim = [&]() -> unsigned {
    const unsigned k = n_claims++;
    if (!queue) return (unsigned)cta + k * (unsigned)ncta;
    return k == 0 ? (unsigned)cta : (unsigned)ncta + atomicAdd(queue, 1u);  // the first ncta positions go one to each CTA
  };
  if (threadIdx.x == 0) {
    for (int q = 0; q < STAGES; ++q) {
      const int t = (int)min(claim(), (unsigned)ntiles);
      claimed[(it + q) % STAGES] = t;
      if (t < ntiles) issue(t, (it + q) % STAGES);
    }
    pending = claim();
  }
  __syncthreads();
  for (;; ++it) {
    const int s = it % STAGES;
    const uint32_t parity = (it / STAGES) & 1;
    const int t = claimed[s];
    if (t >= ntiles) break;
    if (!mbar_wait(&bars[s], parity, kWaitLimit)) return false;
    const int tt = tile_of(t);
    const int ty = tt / f.tiles_x2, tx = tt - ty * f.tiles_x2;
    const long long Y0 = f.r0 + (long long)ty * TH, X0 = f.c0 + (long long)tx * f.tw2;  // first point of the tile
    const float* sm = tile[s];
    // state s + 1 on the tile and a halo of one: thread x' owns a column of the intermediate tile, rows
    // [lo, hi) of it lie inside the update window (computed, with a three-row window sliding down the column), the
    // rest is the other array's own
    {
      const int xp = threadIdx.x;
      const long long X = X0 - 1 + xp;
      if (xp < f.tw2 + 2) {
        const bool col_in = X >= f.c0 && X < f.c1, col_ok = X >= 0 && X < f.ld;
        const int lo = col_in ? (int)max(0ll, f.m0 - (Y0 - 1)) : TH + 2;
        const int hi = col_in ? (int)min((long long)(TH + 2), f.m1 - (Y0 - 1)) : TH + 2;
        const float* other = f.other + (Y0 - 1) * f.ld + X;
        if (!col_in) {
          // a column left or right of the window: all of it is the other array's.  The loads are issued together --
          // one after the other they cost the whole CTA, which waits at the barrier below, 34 memory round trips
          float v[TH + 2];
#pragma unroll
          for (int yp = 0; yp < TH + 2; ++yp) {
            const long long Y = Y0 - 1 + yp;
            v[yp] = (col_ok && Y >= 0 && Y < f.rows_total) ? __ldg(other + (long long)yp * f.ld) : 0.f;
          }
#pragma unroll
          for (int yp = 0; yp < TH + 2; ++yp) mid[yp * BOX_W + xp] = v[yp];
        }
        for (int yp = 0; yp < min(lo, TH + 2) && col_in; ++yp) {
          const long long Y = Y0 - 1 + yp;
          mid[yp * BOX_W + xp] = (col_ok && Y >= 0 && Y < f.rows_total) ? __ldg(other + (long long)yp * f.ld) : 0.f;
        }
        if (lo < hi) {
          constexpr uint32_t R = BOX_W * sizeof(float);  // one row
          const uint32_t qa = smem_u32(sm) + (uint32_t)(((lo + 1) * BOX_W + (f.xs + xp + 1)) * sizeof(float));  // the point itself in the source box
          uint32_t ma = smem_u32(mid) + (uint32_t)((lo * BOX_W + xp) * sizeof(float));
          cross_column<ORDER>(qa, hi - lo, k, [&](int j, float v) { sts(ma + j * R, v); }, [&](int n) { ma += n * R; });
        }
        for (int yp = max(hi, 0); yp < TH + 2 && col_in; ++yp) {
          const long long Y = Y0 - 1 + yp;
          mid[yp * BOX_W + xp] = (col_ok && Y >= 0 && Y < f.rows_total) ? __ldg(other + (long long)yp * f.ld) : 0.f;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // every thread is done with stage s, and has read its position
      const int tn = (int)min(pending, (unsigned)ntiles);
      claimed[s] = tn;
      if (tn < ntiles) issue(tn, s);
      pending = claim();
    }
    // state s + 2 on the tile
    {
      const int cx = threadIdx.x;
      const long long X = X0 + cx;
      if (cx < f.tw2 && X < f.c1) {
        int rmax = (int)min((long long)TH, f.r1 - Y0);
#if RX_BOUNDS
        if (rmax > 0 && !(rx_in_bounds(f.bounds, f.extent, Y0 * f.ld + X, 1, 299) && rx_in_bounds(f.bounds, f.extent, (Y0 + rmax - 1) * f.ld + X, 1, 299))) rmax = 0;
#endif
        float* out = dst + Y0 * f.ld + X;
        const long long ld = f.ld;
        const uint32_t qa = smem_u32(mid) + (uint32_t)((BOX_W + (cx + 1)) * sizeof(float));
        cross_column<ORDER>(qa, rmax, k, [&](int j, float v) { out[j * ld] = v; }, [&](int n) { out += n * ld; });
      }
    }
    __syncthreads();  // stage s and the intermediate tile are free again
    if (t < n_edge && threadIdx.x == 0) {
      __threadfence();  // the tile's rows, written by all threads before the barrier, precede the count
      atomicAdd(edge_counter, 1u);
    }
  }
  return true;
}

// ---- whole counted loop in one launch ------------------------------------------------------------------
// A `stablehlo.while` whose body is nothing but 5-point stencil updates (Jacobi: A -> B, B -> A, ...) runs as ONE
// cooperative launch: every CTA keeps its tile list and its shared-memory ring, sweeps follow each other
// separated by a grid-wide barrier instead of a kernel boundary (about 6 us per sweep on B200).  `phase` i uses
// tensor map and destination i mod n_phases.  The barrier is a monotonic counter in device memory: arrive with a
// release (after making this CTA's stores visible to the async proxy that serves the next sweep's TMA loads),
// poll with acquire loads and a limit; a CTA that gives up reports through the status word and returns.  The
// launch is cooperative, so all CTAs are resident and the barrier cannot wait for a CTA that never started.
constexpr int kMaxPhases = 4;
struct alignas(64) PhaseMaps { CUtensorMap m[kMaxPhases]; };
struct LoopParams {
  StencilParams ph[kMaxPhases];
  float k[kMaxPhases];
  int n_phases;
  int total;          // sweeps to run = loop trip count x stencil steps per iteration
  int alternate;      // odd sweeps walk the tiles backwards
  unsigned* counter;  // zero at launch
  unsigned* queue;    // two words, zero at launch: the tile queues of even and odd passes (see stencil_sweep)
  FuseParams fuse;    // double sweeps that come first (n_fused = 0: none); `total` then counts the single sweeps after them
  // Row-sharded arrays (the device owns a block of rows of each array and keeps copies of its neighbours' boundary
  // rows): between two sweeps CTA 0 exchanges the boundary rows of the array just written with the neighbouring
  // devices, and the other CTAs are released into the next sweep only when the received rows are in place.
  int halo;           // 1: CTA 0 exchanges after every sweep but the last, the other CTAs share the tiles
  unsigned* edge;     // zero at launch: finished first- and last-row tiles, over all sweeps
  int* peer_status;   // the device's status word for waits on peers
  HaloArgs hx;        // .block and .epoch are filled per sweep: block = halo_block[phase], epoch = halo_epoch0 + sweep
  float* halo_block[kMaxPhases];
  unsigned halo_epoch0;
  unsigned* release;  // zero at launch; sweep + 1 once the exchange after `sweep` is done, 0xFFFFFFFF if it failed
};

template <int TH>
__global__ void __launch_bounds__(256, 2) k_stencil_loop(const __grid_constant__ PhaseMaps maps, const __grid_constant__ LoopParams lp, const __grid_constant__ FuseMaps fm) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[STAGES];
  float* tile[STAGES];
  // all phases share the ring geometry; with double sweeps the stages hold their taller boxes and a third region
  // the intermediate tile
  const int stage_floats = BOX_W * (lp.fuse.n_fused > 0 ? TH + 4 : lp.ph[0].box_h);
  uintptr_t base = ((uintptr_t)smem_raw + 127) & ~(uintptr_t)127;
#pragma unroll
  for (int s = 0; s < STAGES; ++s) tile[s] = (float*)base + (size_t)s * stage_floats;
  float* mid = (float*)base + (size_t)STAGES * stage_floats;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  if (lp.halo && blockIdx.x == 0) {
    // The exchange CTA.  As soon as the tiles holding the first and last owned rows of a pass (a double sweep or a
    // single one) are written -- the workers take them first -- it trades those rows with the neighbouring devices
    // while the workers are busy with the rest of the pass, and publishes `release = pass + 1`, which the workers
    // need before the next pass.
    const int n_pass = lp.fuse.n_fused + lp.total;
    unsigned edge_target = 0;
    for (int pass = 0; pass + 1 < n_pass; ++pass) {
      const bool dbl = pass < lp.fuse.n_fused;
      const int ph = dbl ? 0 : (pass - lp.fuse.n_fused) % lp.n_phases;
      // the array this pass writes, and how many of its tiles hold rows the neighbours wait for
      float* block = dbl ? lp.fuse.buf[(pass + 1) & 1] : lp.halo_block[ph];
      edge_target += dbl ? (unsigned)edge_tiles(lp.fuse.r1 - lp.fuse.r0, lp.fuse.tiles_x2, lp.fuse.tiles_y2, TH)
                         : (unsigned)edge_tiles(lp.ph[ph].rows, lp.ph[ph].tiles_x, lp.ph[ph].tiles_y, TH);
      int ok = 1;
      if (threadIdx.x == 0) {
        long long spins = 0;
        for (;;) {
          unsigned v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(lp.edge) : "memory");
          if (v >= edge_target) break;
          if (++spins > kWaitLimit) { ok = 0; break; }
          if (spins > 64) __nanosleep(100);
        }
      }
      ok = __syncthreads_and(ok);
      bool got = false;
      if (ok) {
        HaloArgs hx = lp.hx;
        hx.block = block;
        hx.epoch = lp.halo_epoch0 + (unsigned)pass;
        got = halo_exchange_cta(hx);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");  // the received rows are read by the next pass's bulk loads
        if (!ok) *lp.ph[0].status = 3;
        else if (!got) *lp.peer_status = 2;  // what the stand-alone exchange kernel reports
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(lp.release), "r"(got ? (unsigned)(pass + 1) : 0xFFFFFFFFu) : "memory");
      }
      if (!got) return;
    }
    return;
  }

  const int cta = lp.halo ? (int)blockIdx.x - 1 : (int)blockIdx.x;
  const int ncta = lp.halo ? (int)gridDim.x - 1 : (int)gridDim.x;
  int it = 0;
  int epoch = 0;  // grid barriers passed
  // grid-wide barrier between sweeps (over the worker CTAs); with an exchange, its rows must be in place too
  auto sweep_barrier = [&]() -> bool {
    __syncthreads();
    int ok = 1;
    if (threadIdx.x == 0) {
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");
      atomicAdd(lp.counter, 1u);
      const unsigned target = (unsigned)(epoch + 1) * (unsigned)ncta;
      long long spins = 0;
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(lp.counter) : "memory");
        if (v >= target) break;
        if (++spins > kWaitLimit) { ok = 0; break; }
      }
      if (ok && lp.halo) {
        spins = 0;
        for (;;) {
          unsigned v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(lp.release) : "memory");
          if (v == 0xFFFFFFFFu) { ok = -1; break; }  // the exchange CTA gave up and has reported why
          if (v >= (unsigned)(epoch + 1)) break;
          if (++spins > kWaitLimit + lp.hx.poll_limit) { ok = 0; break; }
          if (spins > 64) __nanosleep(100);
        }
      }
      asm volatile("fence.proxy.async;" ::: "memory");
      if (ok == 0) *lp.ph[0].status = 3;
    }
    ok = __syncthreads_and(ok == 1);
    ++epoch;
    return ok != 0;  // false: nothing of this CTA is in flight (the sweep before drained its ring)
  };
  // double sweeps first: state 2q -> state 2q + 2, ping-ponging between the first array and the scratch array
  // The queue of pass p is word p & 1; the worker CTA 0 clears the other word, which every CTA stopped using before
  // the barrier that ended pass p - 1 and which is next used after the barrier that ends pass p.
  auto pass_queue = [&](int pass) -> unsigned* {
    if (!lp.queue) return nullptr;  // every ncta-th position
    if (cta == 0 && threadIdx.x == 0) lp.queue[(pass + 1) & 1] = 0;
    return lp.queue + (pass & 1);
  };
  for (int q = 0; q < lp.fuse.n_fused; ++q) {
    unsigned* queue = pass_queue(q);
    const bool done =
        lp.fuse.order == 0
            ? stencil_sweep2<TH, 0>(&fm.m[q & 1], lp.fuse, lp.fuse.buf[(q + 1) & 1], tile, mid, bars, it, lp.alternate && (q & 1), cta, ncta, lp.halo != 0, lp.edge, queue)
            : stencil_sweep2<TH, 1>(&fm.m[q & 1], lp.fuse, lp.fuse.buf[(q + 1) & 1], tile, mid, bars, it, lp.alternate && (q & 1), cta, ncta, lp.halo != 0, lp.edge, queue);
    if (!done) {
      if (threadIdx.x == 0) *lp.ph[0].status = 2;
      stencil_drain(bars);
      return;
    }
    if (!sweep_barrier()) return;
  }
  for (int sweep = 0; sweep < lp.total; ++sweep) {
    const int ph = sweep % lp.n_phases;
    // after an odd number of double sweeps the current state sits in the scratch array: the first single sweep reads it there
    const CUtensorMap* src_map = (sweep == 0 && (lp.fuse.n_fused & 1)) ? &fm.m[2] : &maps.m[ph];
    if (!stencil_sweep<true, TH>(src_map, lp.ph[ph], nullptr, lp.k[ph], tile, bars, it, lp.alternate && ((sweep + lp.fuse.n_fused) & 1), cta, ncta, lp.halo != 0, lp.edge,
                                 pass_queue(lp.fuse.n_fused + sweep))) {
      if (threadIdx.x == 0) *lp.ph[0].status = 2;
      stencil_drain(bars);
      return;
    }
    if (sweep + 1 == lp.total) break;
    if (!sweep_barrier()) return;
  }
}

}  // namespace

namespace {

struct Prepared {
  CUtensorMap tmap;
  StencilParams sp;
  size_t smem = 0;
  bool fast = false;
  bool empty = false;
};

// Tensor map over a dense [rows][ld] f32 array with boxes of BOX_W x box_h.
bool make_array_map(const float* base, int64_t ld, int64_t rows, int box_h, CUtensorMap* out) {
  EncodeTiledFn enc = tma_encode_fn();
  if (!enc) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)ld, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)BOX_W, (cuuint32_t)box_h};
  cuuint32_t estr[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tile geometry, tensor map and parameters of one stencil step; false = this path declines the step.
bool prepare_stencil(RxDevice* d, const Step& st, const VmProgram& P, Prepared* out) {
  EncodeTiledFn enc = tma_encode_fn();
  if (!enc) return false;
  if ((int)st.st_dy.size() > kMaxTaps || st.st_dy.size() != (size_t)P.n_leaves) return false;
  int max_dy = 0, max_dx = 0;
  for (size_t k = 0; k < st.st_dy.size(); ++k) {
    max_dy = std::max(max_dy, st.st_dy[k]);
    max_dx = std::max(max_dx, st.st_dx[k]);
  }
  const float* src = (const float*)P.leaf[0].ptr;
  int64_t ld = st.st_src_ld;
  int64_t slot_elems = 0;
  // the source slot is a dense [rows_total][ld] array
  {
    int64_t last = st.st_src_off + (st.st_rows - 1 + max_dy) * ld + (st.st_cols - 1 + max_dx);
    slot_elems = ((last / ld) + 1) * ld;
  }
  int64_t rows_total = slot_elems / ld;
  int64_t col0 = st.st_src_off % ld, row0 = st.st_src_off / ld;
  int x_shift = (int)(col0 % 4);
  int halo_w = (max_dx + x_shift + 3) & ~3;  // box start and tile width stay multiples of 4 floats (16 B)
  if (halo_w > 16 || max_dy > HALO_H) return false;
  int tw = BOX_W - halo_w;
  if (((uintptr_t)src % 16) || (ld % 4) || ld > (int64_t)INT32_MAX || rows_total > (int64_t)INT32_MAX) return false;
  if (st.st_rows <= 0 || st.st_cols <= 0) {
    out->empty = true;
    return true;
  }

  const int TH = 32;  // 16 x 3 CTAs/SM and 64 x 1 CTA/SM measured within 2% of 32 x 2
  int box_h = TH + max_dy;
  // tensor map cache: (base pointer, ld, rows, box height)
  struct Key { const void* p; int64_t ld, rows; int bh; };
  Key key{src, ld, rows_total, box_h};
  std::vector<uint8_t>* blob = nullptr;
  for (auto& kv : d->tmaps)
    if (kv.first == src && kv.second.size() == sizeof(CUtensorMap) + sizeof(Key) && !memcmp(kv.second.data() + sizeof(CUtensorMap), &key, sizeof(Key))) blob = &kv.second;
  if (!blob) {
    CUtensorMap m;
    cuuint64_t gdim[2] = {(cuuint64_t)ld, (cuuint64_t)rows_total};
    cuuint64_t gstride[1] = {(cuuint64_t)ld * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)BOX_W, (cuuint32_t)box_h};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)src, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;  // decline: the generic kernel handles it
    std::vector<uint8_t> v(sizeof(CUtensorMap) + sizeof(Key));
    memcpy(v.data(), &m, sizeof(CUtensorMap));
    memcpy(v.data() + sizeof(CUtensorMap), &key, sizeof(Key));
    if (d->tmaps.size() > 64) d->tmaps.clear();
    d->tmaps[src] = std::move(v);
    blob = &d->tmaps[src];
  }
  memcpy(&out->tmap, blob->data(), sizeof(CUtensorMap));

  StencilParams& sp = out->sp;
  sp = StencilParams{};
  sp.dst = (float*)P.out[0].ptr;
  sp.rows = st.st_rows;
  sp.cols = st.st_cols;
  sp.dst_ld = st.st_dst_ld;
  sp.dst_off = st.st_dst_off;
  sp.x_base = (int)(col0 - x_shift);
  sp.y_base = (int)row0;
  sp.x_shift = x_shift;
  sp.box_h = box_h;
  sp.tw = tw;
  sp.n_taps = (int)st.st_dy.size();
  for (int k = 0; k < sp.n_taps; ++k) { sp.dy[k] = st.st_dy[k]; sp.dx[k] = st.st_dx[k]; }
  if (sp.n_taps == 5) {
    const int cy = sp.dy[0], cx = sp.dx[0];
    sp.cross = cy >= 1 && cx >= 1 && sp.dy[1] == cy && sp.dx[1] == cx - 1 && sp.dy[2] == cy && sp.dx[2] == cx + 1 && sp.dy[3] == cy - 1 && sp.dx[3] == cx &&
               sp.dy[4] == cy + 1 && sp.dx[4] == cx;
  }
  sp.tiles_x = (int)((st.st_cols + tw - 1) / tw);
  sp.tiles_y = (int)((st.st_rows + TH - 1) / TH);
  int* dstatus = nullptr;
  cudaHostGetDevicePointer(&dstatus, d->status, 0);
  sp.status = dstatus + 1;
  sp.dst_extent = P.out[0].extent;
  sp.bounds = P.out[0].bounds;
  out->smem = (size_t)STAGES * BOX_W * box_h * sizeof(float) + 128;  // 2 x 34 KiB for a radius-1 stencil; two CTAs per SM measured fastest
  out->fast = P.fast_id == FAST_STENCIL5_MUL && sp.n_taps == 5;
  return true;
}

}  // namespace

cudaError_t run_stencil_tma(RxDevice* d, const Step& st, const VmProgram& P, bool* handled) {
  *handled = false;
  Prepared pr;
  if (!prepare_stencil(d, st, P, &pr)) return cudaSuccess;
  if (pr.empty) {
    *handled = true;
    return cudaSuccess;
  }
  const StencilParams& sp = pr.sp;
  const size_t smem = pr.smem;
  const bool fast = pr.fast;
  auto kern = fast ? k_stencil_tma<true, 32> : k_stencil_tma<false, 32>;
  static size_t attr_set[64][2] = {};  // function attributes are per device
  size_t& have = attr_set[d->ordinal & 63][fast];
  if (have < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    have = smem;
  }
  int ntiles = sp.tiles_x * sp.tiles_y;
  int per_sm = (int)std::max<size_t>(1, std::min<size_t>((size_t)2, (size_t)(220 * 1024) / smem));
  int grid = std::min(ntiles, d->sm_count * per_sm);
  kern<<<grid, 256, smem, d->stream>>>(pr.tmap, sp, P);
  ++d->launches;
  *handled = true;
  return cudaGetLastError();
}

// `total` sweeps cycling through the given stencil steps (already bound to their buffers) in one cooperative
// launch.  Declines (handled = false) unless every step is the 5-point fast chain on the same tile geometry.
cudaError_t run_stencil_loop(RxDevice* d, const std::vector<const Step*>& steps, const std::vector<VmProgram>& bound, int64_t total, bool* handled,
                             const StencilLoopHalo* halo, bool dry_run, int* passes) {
  *handled = false;
  if (passes) *passes = (int)total;
  const int n = (int)steps.size();
  if (n < 1 || n > kMaxPhases || total < 2 || total > INT32_MAX) return cudaSuccess;
  PhaseMaps maps{};
  LoopParams lp{};
  size_t smem = 0;
  for (int i = 0; i < n; ++i) {
    Prepared pr;
    if (!prepare_stencil(d, *steps[i], bound[i], &pr) || pr.empty || !pr.fast) return cudaSuccess;
    if (i && (pr.smem != smem || pr.sp.box_h != lp.ph[0].box_h)) return cudaSuccess;
    smem = pr.smem;
    maps.m[i] = pr.tmap;
    lp.ph[i] = pr.sp;
    lp.k[i] = bound[i].fast_c;
  }
  lp.n_phases = n;
  lp.total = (int)total;
  lp.alternate = getenv("RX_STENCIL_ONE_WAY") ? 0 : 1;
  unsigned* const words = (unsigned*)(d->scratch + d->scratch_words - 6);  // the five words before the reductions' ticket
  const char* qenv = getenv("RX_STENCIL_QUEUE");  // 0: every CTA takes every ncta-th tile instead (read per call)
  lp.queue = (qenv && atoi(qenv) == 0) ? nullptr : words;
  lp.edge = words + 2;
  lp.release = lp.edge + 1;
  lp.counter = lp.edge + 2;
  if (halo) {
    if ((int)halo->block.size() != n) return cudaSuccess;
    lp.halo = 1;
    lp.peer_status = lp.ph[0].status - 1;  // word 0 of the device's status block; the stencil's own is word 1
    lp.hx = halo->args;
    for (int i = 0; i < n; ++i) lp.halo_block[i] = halo->block[i];
    lp.halo_epoch0 = halo->epoch0;
  }
  // ---- two sweeps per pass over memory, when the loop simply alternates between two arrays -----------------------
  FuseMaps fmaps{};
  float* scratch_array = nullptr;
  size_t scratch_bytes = 0;
  const bool fuse_off = getenv("RX_STENCIL_FUSE2") && atoi(getenv("RX_STENCIL_FUSE2")) == 0;  // read per call
  // (a row-sharded loop needs two halo rows for it: the planner gives stencil loops of radius 1 that much)
  if ((!halo || (halo->args.up == 2 && halo->args.down == 2)) && !fuse_off && n == 2 && total >= 4) {
    const Step &s0 = *steps[0], &s1 = *steps[1];
    const VmProgram &p0 = bound[0], &p1 = bound[1];
    const float* x0 = (const float*)p0.leaf[0].ptr;
    const float* x1 = (const float*)p1.leaf[0].ptr;
    const int64_t ld = s0.st_src_ld;
    bool same = x0 != x1 && p0.out[0].ptr == (void*)x1 && p1.out[0].ptr == (void*)x0 && s0.st_dst_ld == ld && s1.st_src_ld == ld && s1.st_dst_ld == ld &&
                s0.st_src_off == s1.st_src_off && s0.st_dst_off == s1.st_dst_off && s0.st_rows == s1.st_rows && s0.st_cols == s1.st_cols && s0.st_dy == s1.st_dy &&
                s0.st_dx == s1.st_dx && p0.fast_c == p1.fast_c && s0.st_dy.size() == 5 && p0.leaf[0].extent == p1.leaf[0].extent && p0.leaf[0].extent % ld == 0;
    const int64_t rows_total = same ? p0.leaf[0].extent / ld : 0;
    const int64_t r0 = s0.st_dst_off / ld, c0 = s0.st_dst_off % ld, row0 = s0.st_src_off / ld, col0 = s0.st_src_off % ld;
    FuseParams f{};
    if (same) {
      // tap offsets relative to the updated point, in evaluation order: (dy, dx)
      int oy[5], ox[5];
      for (int k = 0; k < 5; ++k) {
        oy[k] = (int)(row0 + s0.st_dy[k] - r0);
        ox[k] = (int)(col0 + s0.st_dx[k] - c0);
      }
      auto is = [&](int k, int y, int x) { return oy[k] == y && ox[k] == x; };
      if (is(0, 0, 0) && is(1, 0, -1) && is(2, 0, 1) && is(3, -1, 0) && is(4, 1, 0)) f.order = 0;
      else if (is(0, 0, 0) && is(1, -1, 0) && is(2, 1, 0) && is(3, 0, 1) && is(4, 0, -1)) f.order = 1;
      else same = false;
    }
    // the window must leave room for the taps inside the array, and box starts must fall on 16-byte boundaries
    same = same && r0 >= 1 && c0 >= 1 && r0 + s0.st_rows + 1 <= rows_total && c0 + s0.st_cols + 1 <= ld && rows_total >= 4;
    if (same) {
      const int tail = 2 + (int)(total & 1);
      f.n_fused = (int)((total - tail) / 2);
      f.xs = (int)(((c0 - 2) % 4 + 4) % 4);
      f.tw2 = (BOX_W - 4 - f.xs) & ~3;
      f.tiles_x2 = (int)((s0.st_cols + f.tw2 - 1) / f.tw2);
      f.tiles_y2 = (int)((s0.st_rows + 32 - 1) / 32);
      f.ld = ld;
      f.rows_total = rows_total;
      f.r0 = r0;
      f.r1 = r0 + s0.st_rows;
      f.m0 = f.r0 - ((halo && halo->window_above) ? 1 : 0);
      f.m1 = f.r1 + ((halo && halo->window_below) ? 1 : 0);
      f.c0 = c0;
      f.c1 = c0 + s0.st_cols;
      f.k = p0.fast_c;
      f.status = lp.ph[0].status;
      f.other = x1;
      f.extent = p0.leaf[0].extent;
      f.bounds = p0.out[0].bounds;
      scratch_bytes = (size_t)p0.leaf[0].extent * sizeof(float);
      if (f.n_fused >= 1 && !dry_run) {
        scratch_array = (float*)d->alloc(scratch_bytes);
        f.buf[0] = const_cast<float*>(x0);
        f.buf[1] = scratch_array;
        if (!make_array_map(x0, ld, rows_total, 32 + 4, &fmaps.m[0]) || !make_array_map(scratch_array, ld, rows_total, 32 + 4, &fmaps.m[1]) ||
            !make_array_map(scratch_array, ld, rows_total, lp.ph[0].box_h, &fmaps.m[2])) {
          d->release(scratch_array, scratch_bytes);
          scratch_array = nullptr;
          if (halo) return cudaErrorUnknown;  // the other devices of the mesh have decided for double sweeps: do not run a different loop here
          f.n_fused = 0;
        }
      }
      if (f.n_fused >= 1) {
        lp.fuse = f;
        lp.total = tail;
        if (passes) *passes = f.n_fused + tail;
        smem = (size_t)STAGES * BOX_W * (32 + 4) * sizeof(float) + (size_t)BOX_W * (32 + 2) * sizeof(float) + 128;
      }
    }
  }
  struct ScratchGuard {  // the pool hands the block out again in stream order, so it can go back right after the launch
    RxDevice* d;
    float*& p;
    size_t bytes;
    ~ScratchGuard() { if (p) d->release(p, bytes); }
  } scratch_guard{d, scratch_array, scratch_bytes};
  auto kern = k_stencil_loop<32>;
  static size_t attr_set[64] = {};
  static int resident[64] = {};
  size_t& have = attr_set[d->ordinal & 63];
  int& occ = resident[d->ordinal & 63];
  if (have < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    have = smem;
    occ = 0;
  }
  if (!occ) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, 256, smem) != cudaSuccess || occ < 1) {
      cudaGetLastError();
      occ = 0;
      return cudaSuccess;
    }
  }
  int ntiles = 0;
  for (int i = 0; i < n; ++i) ntiles = std::max(ntiles, lp.ph[i].tiles_x * lp.ph[i].tiles_y);
  if (lp.fuse.n_fused > 0) ntiles = std::max(ntiles, lp.fuse.tiles_x2 * lp.fuse.tiles_y2);
  int grid = std::min(ntiles, d->sm_count * std::min(occ, 2));
  if (halo) {
    // one more CTA, which only exchanges; every sweep must count the same number of edge tiles
    for (int i = 1; i < n; ++i)
      if (lp.ph[i].tiles_x != lp.ph[0].tiles_x || lp.ph[i].tiles_y != lp.ph[0].tiles_y) return cudaSuccess;
    grid = std::min(ntiles, d->sm_count * std::min(occ, 2) - 1) + 1;
    if (grid < 2) return cudaSuccess;
  }
  if (dry_run) {
    *handled = true;
    return cudaSuccess;
  }
  cudaError_t e = cudaMemsetAsync(words, 0, 5 * sizeof(unsigned), d->stream);
  if (e != cudaSuccess) return e;
  if (lp.fuse.n_fused > 0) {
    // the scratch array needs the first array's values outside the update window (they are never written): the rows
    // above and below it, and the columns left and right of it
    const FuseParams& f = lp.fuse;
    const size_t pitch = (size_t)f.ld * sizeof(float);
    const float* x0 = f.buf[0];
    float* z = f.buf[1];
    // (of a row block too: its halo rows are written by the exchange after the first pass, before anything reads them
    // there, and arrive with their border columns)
    if (f.r0 > 0) e = cudaMemcpyAsync(z, x0, (size_t)f.r0 * pitch, cudaMemcpyDeviceToDevice, d->stream);
    if (e == cudaSuccess && f.r1 < f.rows_total)
      e = cudaMemcpyAsync(z + f.r1 * f.ld, x0 + f.r1 * f.ld, (size_t)(f.rows_total - f.r1) * pitch, cudaMemcpyDeviceToDevice, d->stream);
    if (e == cudaSuccess && f.c0 > 0)
      e = cudaMemcpy2DAsync(z + f.r0 * f.ld, pitch, x0 + f.r0 * f.ld, pitch, (size_t)f.c0 * sizeof(float), (size_t)(f.r1 - f.r0), cudaMemcpyDeviceToDevice, d->stream);
    if (e == cudaSuccess && f.c1 < f.ld)
      e = cudaMemcpy2DAsync(z + f.r0 * f.ld + f.c1, pitch, x0 + f.r0 * f.ld + f.c1, pitch, (size_t)(f.ld - f.c1) * sizeof(float), (size_t)(f.r1 - f.r0), cudaMemcpyDeviceToDevice,
                            d->stream);
    if (e != cudaSuccess) return e;
  }
  void* args[] = {(void*)&maps, (void*)&lp, (void*)&fmaps};
  e = cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(256), args, smem, d->stream);
  if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorNotSupported) {
    cudaGetLastError();
    return cudaSuccess;  // the caller launches sweep by sweep
  }
  ++d->launches;
  *handled = true;
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace rx
