// In-memory form of the StableHLO subset the engine executes, and the parser
// entry point.  The module text is what Reactant hands to its runtime at
// XLA.compile (src/xla/PJRT/LoadedExecutable.jl:62-83): the optimised module
// in MLIR pretty form, `func.func @main` with reversed-dim tensor types
// (src/TracedUtils.jl:511-527).  Any op outside the subset is a hard error.
#pragma once
#include <stdint.h>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/rx_b200.h"  // RX_ERR_* codes

namespace rx {

// XLA primitive type codes (src/xla/Utils.jl:18-40).
enum class DT : int {
  INVALID = 0, PRED = 1, S8 = 2, S16 = 3, S32 = 4, S64 = 5, U8 = 6, U16 = 7, U32 = 8, U64 = 9,
  F16 = 10, F32 = 11, F64 = 12, C64 = 15, BF16 = 16, C128 = 18
};

size_t dt_size(DT t);
const char* dt_name(DT t);
inline bool dt_is_float(DT t) { return t == DT::F16 || t == DT::F32 || t == DT::F64 || t == DT::BF16; }
inline bool dt_is_int(DT t) { return (int)t >= 2 && (int)t <= 9; }

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

struct Type {
  DT dt = DT::INVALID;
  std::vector<int64_t> shape;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
  bool operator==(const Type& o) const { return dt == o.dt && shape == o.shape; }
  std::string str() const;
};

enum class OpK {
  Constant, Iota, Unary, Binary, Convert, Compare, Select, Clamp,
  BroadcastInDim, Transpose, Reshape, Slice, DynamicSlice, DynamicUpdateSlice, Pad, Concatenate,
  DotGeneral, Reduce, ReduceWindow, While, AllReduce, Return
};

enum class RedK { Add, Max, Min, Mul, Or, And };

struct Op;
struct Region {
  std::vector<int> args;    // value ids bound on entry
  std::vector<Op> ops;
  std::vector<int> yields;  // operands of the terminator
};

struct Op {
  OpK kind;
  std::string name;           // full op name, for messages
  int ew = 0;                 // VmOp for Unary/Binary; VmCmp for Compare
  std::vector<int> in, out;   // value ids
  std::vector<int64_t> dims;  // broadcast dims / permutation / reduce dims / concat dim / iota dim
  std::vector<int64_t> start, limit, stride;  // slice; pad: low/high/interior; reduce_window: padding low/high, window strides (dims = window)
  std::vector<int64_t> dilation;              // reduce_window: window dilations
  // constant payload
  bool splat = true;
  double fval = 0;            // splat value as double (floats)
  int64_t ival = 0;           // splat value (ints / pred)
  std::vector<uint8_t> dense; // non-splat payload, already in the element type
  // dot_general
  std::vector<int64_t> lbatch, rbatch, lcontract, rcontract;
  RedK red = RedK::Add;
  std::vector<Region> regions;  // while: {cond, body}
  int line = 0;
};

struct Value {
  Type type;
  std::string name;
};

struct ArgAttr {
  int aliasing_output = -1;       // tf.aliasing_output
  std::string sharding_mesh;      // sdy.sharding mesh symbol ("" = none)
  std::vector<std::vector<std::string>> dim_axes;  // per tensor dim: mesh axes
};

struct Func {
  std::string name;
  Region body;                   // args = function arguments, yields = returned values
  std::vector<ArgAttr> arg_attrs;
  std::vector<ArgAttr> res_attrs;
  std::vector<Type> result_types;
};

struct Module {
  std::string name;
  std::vector<Value> values;
  std::map<std::string, Func> funcs;
  std::map<std::string, std::vector<std::pair<std::string, int64_t>>> meshes;
  int64_t num_partitions = 1, num_replicas = 1;
  int new_value(const Type& t, const std::string& n) {
    values.push_back({t, n});
    return (int)values.size() - 1;
  }
};

std::unique_ptr<Module> parse_module(const std::string& text);

}  // namespace rx
