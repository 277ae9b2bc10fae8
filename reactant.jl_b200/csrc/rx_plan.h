// Execution plan: what `XLA.compile` turns a module into in this engine.
// A plan is a list of kernel launches ("steps") over a table of buffer slots;
// it replaces the loaded executable XLA would build at
// deps/ReactantExtra/API.cpp:1482-1507 (ClientCompileInternal).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "rx_ir.h"
#include "rx_vm.h"

namespace rx {

enum class SlotK { Arg, Temp, Const };

struct Slot {
  SlotK kind = SlotK::Temp;
  Type type;                  // per-device (local) type
  int arg_index = -1;         // Arg
  bool writable = false;      // Arg: carries tf.aliasing_output (may be updated in place when donated)
  std::vector<uint8_t> init;  // Const: payload uploaded once per device
  // Temp of a row-sharded stencil loop: the type is the GLOBAL [rows][cols] array; each device allocates its own block
  // of rows / num_partitions rows plus `halo_up` rows above and `halo_down` rows below (copies of its neighbours'
  // boundary rows), and row r of the allocation is global row device * rows / num_partitions - halo_up + r.
  bool row_block = false;
  int halo_up = 0, halo_down = 0;
  bool dead = false;          // Temp that nothing writes or reads after fusion (a GEMM result consumed in its epilogue): not allocated
  int64_t bytes() const { return type.numel() * (int64_t)dt_size(type.dt); }
};

enum class StepK { Map, ReduceFull, ReduceRow, ReduceCol, LogSumExp, Stencil, Gemm, Copy, Fill, Loop, AllReduce, Scan, SumPartials, RowsIn, RowsOut, DynSlice };

struct GemmDesc {
  // D[m][n] = sum_k A(m,k) * B(k,n); strides in elements of the operand slots.
  int a_slot = -1, b_slot = -1, d_slot = -1;
  int64_t M = 0, N = 0, K = 0, batch = 1;
  int64_t a_sm = 0, a_sk = 0, b_sk = 0, b_sn = 0;  // element strides
  int64_t a_sb = 0, b_sb = 0, d_sb = 0;            // batch strides
  int64_t a_off = 0, b_off = 0;                    // element offsets of the operands inside their slots
  DT in_dt = DT::BF16, out_dt = DT::BF16;
  // Optional fused epilogue: the step's prog is evaluated per (m, n) over the root space [M][N]; leaf `acc_leaf` is the
  // accumulator (rounded to out_dt first, as if D had been stored and read back); prog.out are dense [M][N] results
  // (D itself is one of them only if something else still reads it); `col_reg` / `full_reg` are registers whose
  // column sums / full sums go to per-row-block / per-tile partials in the given slots, added up in index order by
  // the SumPartials step that follows.
  bool has_epilogue = false;
  int acc_leaf = -1, n_leaves = 0;
  int n_col = 0, n_full = 0;
  int col_reg[2] = {0, 0}, full_reg[2] = {0, 0};
  int col_slot[2] = {-1, -1}, full_slot[2] = {-1, -1};
};

// One job of a SumPartials step: dst[n] = init + sum over r (in order) of src[r][n]
struct SumJob {
  int src_slot = -1, dst_slot = -1;
  int64_t rows = 0, n = 0;
  double init = 0;
};

struct Step {
  StepK kind = StepK::Map;
  std::string note;               // human-readable summary (plan dumps, tests)
  VmProgram prog{};               // leaf/out pointers are bound at launch time
  std::vector<int> leaf_slot;     // slot of prog.leaf[i]
  std::vector<int> out_slot;      // slot of prog.out[i]
  // reductions: collapsed space is [outer][red][inner]; prog.dim holds those three
  RedK red = RedK::Add;
  DT red_dt = DT::F32;
  double init_f = 0;              // value combined with the reduction (the reduce op's init operand)
  int64_t init_i = 0;
  int64_t outer = 1, red_n = 1, inner = 1;
  // LogSumExp: out_slot = {max, sumexp, lse}
  // Stencil: prog leaves are shifted views of one slot; tile geometry derived at launch
  int64_t st_rows = 0, st_cols = 0, st_src_ld = 0, st_dst_ld = 0, st_src_off = 0, st_dst_off = 0;
  int st_radius = 0;
  std::vector<int> st_dy, st_dx;  // per leaf
  GemmDesc gemm;
  // Copy / Fill
  int src_slot = -1, dst_slot = -1;
  int64_t bytes = 0;
  double fill_f = 0;
  int64_t fill_i = 0;
  // Loop
  // row_sharded: the carried arrays are split into row blocks over the mesh (slots flagged row_block); the body's
  // stencil steps describe the update of the GLOBAL arrays, every device applies them to the rows it owns and sends
  // its boundary rows to its neighbours' halos after each one.
  // RowsIn / RowsOut: copy a device's block between an ordinary (local) slot src_slot / dst_slot and the owned rows
  // of a row_block slot (RowsIn also fetches the halos from the neighbours).
  bool row_sharded = false;
  int64_t trip = 0;
  std::vector<Step> body;
  std::vector<int> state_slots;   // slot holding loop-carried value j on entry to an iteration
  std::vector<int> yield_slots;   // slot holding its next value at the end of the body
  // Scan: inclusive prefix (red) of src_slot along the middle dim of [outer][red_n][inner] into dst_slot, combined with init
  // AllReduce (sum over the mesh axis, in place on dst_slot)
  int64_t count = 0;
  // SumPartials
  std::vector<SumJob> sums;
  // DynSlice: `bytes` contiguous bytes of src_slot copied to dst_slot, starting at element
  //   sum_d clamp(dyn_a[d] * it + dyn_b[d], 0, dyn_hi[d]) * dyn_stride[d]
  // where `it` is the current iteration (0-based) of the innermost enclosing loop: a stablehlo.dynamic_slice whose
  // start indices are affine in the loop counter (fict[t] in benchmark/polybench/stencil.jl:49).
  std::vector<int64_t> dyn_a, dyn_b, dyn_hi, dyn_stride;
  int64_t dyn_elem_bytes = 4;
};

struct ResultBinding {
  int slot = -1;
  Type type;          // per-device type handed back to the caller
  int sharded_dim = -1;
};

struct Plan {
  std::vector<Slot> slots;
  std::vector<Step> steps;
  std::vector<ResultBinding> results;
  std::vector<Type> arg_types;        // per-device
  std::vector<Type> arg_global_types;
  std::vector<int> arg_sharded_dim;   // -1 = replicated
  std::vector<int> arg_alias;         // tf.aliasing_output or -1
  int64_t num_partitions = 1;
  int64_t scratch_floats = 0;         // two-pass reduction scratch the plan needs
  std::string describe() const;       // JSON summary of the plan
};

std::unique_ptr<Plan> build_plan(const Module& m);

}  // namespace rx
