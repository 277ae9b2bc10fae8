// Planner: walks the optimised StableHLO module and groups its ops into the
// fusion templates the kernels implement:
//   * elementwise chain -> full reduce            (sum(sin.(x) .+ y))
//   * elementwise chain -> reduce over one axis   (row / column reductions)
//   * max -> exp-sum -> log over the same axis     (logsumexp, one HBM read)
//   * shifted-slice sums written into an interior (stencil updates, in place)
//   * dot_general                                 (bf16 GEMM, fp32 accumulate; operand transposes folded into strides)
//   * reduce over a mesh-sharded axis             (local reduce + all-reduce)
// Layout shims (the reversed-dims transposes Reactant inserts at function entry
// and exit, src/TracedUtils.jl:608-626, 846-883), reshapes, slices and
// broadcasts are folded into index maps and never materialised.
//
// In the reference this role is played by XLA's compiler behind
// ClientCompileWithProto (deps/ReactantExtra/API.cpp:1528-1536); SPMD
// partitioning of sharded reductions, which XLA performs there
// (API.cpp:1487-1497), is done here by rule.
#include "rx_plan.h"
#include "rx_jit.h"

#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <cmath>
#include <functional>
#include <map>
#include <set>
#include <sstream>

namespace rx {

namespace {

struct DimMap {
  int src;        // parent dim feeding this dim, or -1
  int64_t mult;
  int64_t off;
  bool operator<(const DimMap& o) const { return std::tie(src, mult, off) < std::tie(o.src, o.mult, o.off); }
  bool operator==(const DimMap& o) const { return src == o.src && mult == o.mult && off == o.off; }
};
using RMap = std::vector<DimMap>;

struct Expr;
using ExprP = std::shared_ptr<Expr>;
struct Expr {
  enum K { Leaf, Const, Op, Iota, View, Sym } k = Const;
  DT dt = DT::F32;
  std::vector<int64_t> shape;
  // Leaf
  int slot = -1;
  std::vector<int64_t> lstride;
  int64_t loffset = 0;
  // Const
  double f = 0;
  int64_t i = 0;
  // Op
  int vmop = 0, cmp = 0;
  std::vector<ExprP> kids;
  int iota_dim = 0;
  RMap map;  // View: one entry per kid dim
  int cost = 0;
  bool heavy = false;
  // Sym: the counter of an enclosing counted loop, value = sym_a * it + sym_b in 0-based iteration `it` of the loop at
  // nesting depth sym_depth (0: not a counter, nothing is known about the value)
  int sym_depth = 0;
  int64_t sym_a = 0, sym_b = 0;
};

std::vector<int64_t> canon_strides(const std::vector<int64_t>& shape) {
  std::vector<int64_t> s(shape.size());
  int64_t acc = 1;
  for (int d = (int)shape.size() - 1; d >= 0; --d) {
    s[d] = acc;
    acc *= shape[d];
  }
  return s;
}

int64_t prod(const std::vector<int64_t>& v) {
  int64_t n = 1;
  for (auto d : v) n *= d;
  return n;
}

VmElem elem_of(DT dt) {
  switch (dt) {
    case DT::F32: return EL_F32;
    case DT::BF16: return EL_BF16;
    case DT::S32: case DT::U32: return EL_I32;
    case DT::PRED: return EL_PRED;
    case DT::F64: return EL_F64;
    default: throw Error(RX_ERR_UNSUPPORTED_TYPE, std::string("unsupported element type ") + dt_name(dt) + " in a fused computation");
  }
}

bool is_transcendental(int op) {
  return op == VM_SIN || op == VM_COS || op == VM_EXP || op == VM_LOG || op == VM_TANH || op == VM_POW ||
         op == VM_LOG1P || op == VM_EXPM1 || op == VM_LOGISTIC || op == VM_DIV || op == VM_SQRT || op == VM_RSQRT || op == VM_TAN || op == VM_CBRT ||
         op == VM_ATAN2 || op == VM_REM;
}

// -------------------------------------------------------------------------
// Lowering of an expression DAG over a root iteration space into a VmProgram
// -------------------------------------------------------------------------
struct LeafRef {
  int slot;
  DT dt;
  int64_t offset;
  std::vector<int64_t> stride;  // per root dim
  bool operator==(const LeafRef& o) const { return slot == o.slot && dt == o.dt && offset == o.offset && stride == o.stride; }
};

struct VNode {
  int op;
  int a = -1, b = -1, c = -1;
  uint32_t imm = 0;
  int cmp = 0;
  int leaf = -1;
};

struct Lowering {
  std::vector<int64_t> root;
  std::vector<VNode> nodes;
  std::vector<LeafRef> leaves;
  std::map<std::pair<const Expr*, RMap>, int> memo;
  bool has_iota = false;
  // f64 anywhere in the group makes the program "wide" (64-bit registers, rx_wide.cu): its floating-point constants
  // live in a table (VNode.imm = index, VNode.cmp = 64); f32 constants are marked (cmp = 32) so that assemble() can
  // move them there too once it knows the program is wide
  bool wide = false;
  std::vector<uint64_t> wconsts;
  int wconst(double v) {
    uint64_t bits;
    memcpy(&bits, &v, 8);
    for (size_t k = 0; k < wconsts.size(); ++k)
      if (wconsts[k] == bits) return (int)k;
    wconsts.push_back(bits);
    return (int)wconsts.size() - 1;
  }

  explicit Lowering(const std::vector<int64_t>& root_shape) : root(root_shape) {}

  static RMap identity(size_t rank) {
    RMap m(rank);
    for (size_t d = 0; d < rank; ++d) m[d] = {(int)d, 1, 0};
    return m;
  }
  static RMap compose(const RMap& view, const RMap& parent) {
    RMap out(view.size());
    for (size_t d = 0; d < view.size(); ++d) {
      const DimMap& v = view[d];
      if (v.src < 0) { out[d] = {-1, 0, v.off}; continue; }
      const DimMap& p = parent[v.src];
      if (p.src < 0) out[d] = {-1, 0, v.mult * p.off + v.off};
      else out[d] = {p.src, v.mult * p.mult, v.mult * p.off + v.off};
    }
    return out;
  }
  int add(const VNode& n) {
    nodes.push_back(n);
    return (int)nodes.size() - 1;
  }
  int konst_bits(uint32_t bits) {
    VNode n{VM_CONST};
    n.imm = bits;
    return add(n);
  }
  int konst(DT dt, double f, int64_t i) {
    uint32_t bits;
    if (dt == DT::F64) {
      wide = true;
      VNode n{VM_CONST};
      n.imm = (uint32_t)wconst(f);
      n.cmp = 64;
      return add(n);
    }
    if (dt == DT::F32 || dt == DT::BF16) {
      float v32 = (float)f;
      memcpy(&bits, &v32, 4);
      if (dt == DT::BF16) bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16;
      VNode n{VM_CONST};
      n.imm = bits;
      n.cmp = 32;
      return add(n);
    }
    bits = (uint32_t)(int32_t)i;
    return konst_bits(bits);
  }

  int lower(const ExprP& e, const RMap& rmap) {
    auto key = std::make_pair((const Expr*)e.get(), rmap);
    auto it = memo.find(key);
    if (it != memo.end()) return it->second;
    int r = -1;
    switch (e->k) {
      case Expr::Leaf: {
        if (e->dt == DT::F64) wide = true;
        LeafRef lr{e->slot, e->dt, e->loffset, std::vector<int64_t>(root.size(), 0)};
        for (size_t d = 0; d < e->lstride.size(); ++d) {
          lr.offset += e->lstride[d] * rmap[d].off;
          if (rmap[d].src >= 0) lr.stride[rmap[d].src] += e->lstride[d] * rmap[d].mult;
        }
        int idx = -1;
        for (size_t k = 0; k < leaves.size(); ++k)
          if (leaves[k] == lr) idx = (int)k;
        if (idx < 0) {
          leaves.push_back(lr);
          idx = (int)leaves.size() - 1;
          VNode n{-1};
          n.leaf = idx;
          r = add(n);
        } else {
          for (size_t k = 0; k < nodes.size(); ++k)
            if (nodes[k].leaf == idx) r = (int)k;
        }
        break;
      }
      case Expr::Const:
        r = konst(e->dt, e->f, e->i);
        break;
      case Expr::View:
        r = lower(e->kids[0], compose(e->map, rmap));
        break;
      case Expr::Iota: {
        const DimMap& dm = rmap[e->iota_dim];
        if (dm.src < 0) {
          r = konst(DT::S32, 0, dm.off);
        } else {
          has_iota = true;
          VNode n{VM_IOTA};
          n.a = dm.src;  // root dim (remapped after dim sorting)
          r = add(n);
          if (dm.mult != 1) { VNode mul{VM_IMUL}; mul.a = r; mul.b = konst(DT::S32, 0, dm.mult); r = add(mul); }
          if (dm.off != 0) { VNode ad{VM_IADD}; ad.a = r; ad.b = konst(DT::S32, 0, dm.off); r = add(ad); }
        }
        if (dt_is_float(e->dt)) { VNode cv{VM_I2F}; cv.a = r; r = add(cv); }
        break;
      }
      case Expr::Op: {
        if (e->dt == DT::F64) wide = true;
        if (e->vmop == VM_MOV && e->kids.size() == 1) {  // widening converts and identities cost nothing
          r = lower(e->kids[0], rmap);
          break;
        }
        VNode n{e->vmop};
        n.cmp = e->cmp;
        if (e->kids.size() > 0) n.a = lower(e->kids[0], rmap);
        if (e->kids.size() > 1) n.b = lower(e->kids[1], rmap);
        if (e->kids.size() > 2) n.c = lower(e->kids[2], rmap);
        r = add(n);
        break;
      }
      case Expr::Sym:
        throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op: a loop-variant scalar feeds a tensor computation");
    }
    memo[key] = r;
    return r;
  }
};

// Sorted / collapsed iteration space shared by all leaves and outputs of a step.
struct Space {
  std::vector<int64_t> dim;
  std::vector<int> cls;                       // 0 kept, 1 reduced
  std::vector<std::vector<int64_t>> lstride;  // [leaf][dim]
  std::vector<std::vector<int64_t>> ostride;  // [out][dim]
  std::vector<int> origin;                    // original root dim of each dim (first of a merged run)
};

void normalise_space(Space& sp, int dominant_leaf, bool by_output, bool allow_collapse) {
  size_t nd = sp.dim.size();
  // drop unit dims
  std::vector<size_t> keep;
  for (size_t d = 0; d < nd; ++d)
    if (sp.dim[d] != 1) keep.push_back(d);
  auto take = [&](std::vector<int64_t>& v) {
    std::vector<int64_t> o;
    for (auto d : keep) o.push_back(v[d]);
    v = o;
  };
  {
    std::vector<int> c, org;
    for (auto d : keep) { c.push_back(sp.cls[d]); org.push_back(sp.origin[d]); }
    sp.cls = c;
    sp.origin = org;
  }
  take(sp.dim);
  for (auto& l : sp.lstride) take(l);
  for (auto& o : sp.ostride) take(o);
  nd = sp.dim.size();
  // order dims so that the dominant access is contiguous in the innermost dim
  std::vector<size_t> order(nd);
  for (size_t d = 0; d < nd; ++d) order[d] = d;
  const std::vector<int64_t>* ref = nullptr;
  if (by_output && !sp.ostride.empty()) ref = &sp.ostride[0];
  else if (dominant_leaf >= 0) ref = &sp.lstride[dominant_leaf];
  if (ref) {
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
      int64_t sa = std::llabs((*ref)[a]), sb = std::llabs((*ref)[b]);
      if (sa == 0) sa = INT64_MAX;  // broadcast dims outermost
      if (sb == 0) sb = INT64_MAX;
      return sa > sb;
    });
  }
  auto perm = [&](std::vector<int64_t>& v) {
    std::vector<int64_t> o(nd);
    for (size_t d = 0; d < nd; ++d) o[d] = v[order[d]];
    v = o;
  };
  {
    std::vector<int> c(nd), org(nd);
    for (size_t d = 0; d < nd; ++d) { c[d] = sp.cls[order[d]]; org[d] = sp.origin[order[d]]; }
    sp.cls = c;
    sp.origin = org;
  }
  perm(sp.dim);
  for (auto& l : sp.lstride) perm(l);
  for (auto& o : sp.ostride) perm(o);
  if (!allow_collapse) return;
  // merge adjacent dims that every access walks contiguously
  for (size_t d = 0; d + 1 < sp.dim.size();) {
    bool ok = sp.cls[d] == sp.cls[d + 1];
    auto compat = [&](const std::vector<int64_t>& s) { return s[d] == s[d + 1] * sp.dim[d + 1]; };
    for (auto& l : sp.lstride) ok = ok && compat(l);
    for (auto& o : sp.ostride) ok = ok && compat(o);
    if (!ok) { ++d; continue; }
    sp.dim[d] *= sp.dim[d + 1];
    auto fold = [&](std::vector<int64_t>& s) { s[d] = s[d + 1]; s.erase(s.begin() + d + 1); };
    for (auto& l : sp.lstride) fold(l);
    for (auto& o : sp.ostride) fold(o);
    sp.dim.erase(sp.dim.begin() + d + 1);
    sp.cls.erase(sp.cls.begin() + d + 1);
    sp.origin.erase(sp.origin.begin() + d + 1);
  }
}

// -------------------------------------------------------------------------
struct Planner {
  const Module& m;
  Plan& plan;
  std::vector<ExprP> env;
  std::vector<int> uses;
  std::vector<int> shard;  // per value: sharded dim or -1
  int64_t nparts = 1;
  std::vector<Step>* cur = nullptr;
  struct LseInfo { int m_slot, lse_slot; };
  std::map<int, LseInfo> lse_of_sum;  // sumexp slot -> companions
  std::set<int> state_slots_live;     // loop-carried slots (writable in place)

  std::vector<int> remaining;  // per value: uses by ops that have not been planned yet (function and loop results never run out)

  Planner(const Module& mod, Plan& p) : m(mod), plan(p), env(mod.values.size()), uses(mod.values.size(), 0), shard(mod.values.size(), -1) {}

  // ---- helpers -----------------------------------------------------------
  void count_uses(const Region& r) {
    for (auto& op : r.ops) {
      for (int v : op.in) uses[v]++;
      for (auto& sub : op.regions) count_uses(sub);
    }
    for (int v : r.yields) uses[v]++;
  }
  Type local_type(int v) const {
    Type t = m.values[v].type;
    if (shard[v] >= 0) t.shape[shard[v]] /= nparts;
    return t;
  }
  int new_slot(const Type& t, SlotK k = SlotK::Temp) {
    Slot s;
    s.kind = k;
    s.type = t;
    plan.slots.push_back(s);
    return (int)plan.slots.size() - 1;
  }
  ExprP leaf(int slot, const Type& t) {
    auto e = std::make_shared<Expr>();
    e->k = Expr::Leaf;
    e->dt = t.dt;
    e->shape = t.shape;
    e->slot = slot;
    e->lstride = canon_strides(t.shape);
    return e;
  }
  ExprP konst(const Type& t, double f, int64_t i) {
    auto e = std::make_shared<Expr>();
    e->k = Expr::Const;
    e->dt = t.dt;
    e->shape = t.shape;
    e->f = f;
    e->i = i;
    return e;
  }
  ExprP mkop(int vmop, const Type& t, std::vector<ExprP> kids, int cmp = 0) {
    auto e = std::make_shared<Expr>();
    e->k = Expr::Op;
    e->dt = t.dt;
    e->shape = t.shape;
    e->vmop = vmop;
    e->cmp = cmp;
    e->cost = 1;
    e->heavy = is_transcendental(vmop);
    for (auto& k : kids) {
      e->cost += k->cost;
      e->heavy = e->heavy || k->heavy;
    }
    e->kids = std::move(kids);
    return e;
  }
  ExprP view(const ExprP& kid, const Type& t, RMap map) {
    auto e = std::make_shared<Expr>();
    e->k = Expr::View;
    e->dt = t.dt;
    e->shape = t.shape;
    e->kids = {kid};
    e->map = std::move(map);
    e->cost = kid->cost;
    e->heavy = kid->heavy;
    return e;
  }
  // A contiguous leaf (any offset): reinterpretable under reshape.
  static bool contiguous_leaf(const ExprP& e) { return e->k == Expr::Leaf && e->lstride == canon_strides(e->shape); }
  bool whole_slot(const ExprP& e) const {
    return contiguous_leaf(e) && e->loffset == 0 && prod(e->shape) == plan.slots[e->slot].type.numel() && e->dt == plan.slots[e->slot].type.dt;
  }
  static bool is_splat(const ExprP& e) {
    if (e->k == Expr::Const) return true;
    if (e->k == Expr::View) return is_splat(e->kids[0]);
    if (e->k == Expr::Leaf) return prod(e->shape) == 1;
    return false;
  }
  // Does the value of `e` not depend on its index along dim `dim`?  (Such a replicated value can be
  // combined with a tensor sharded along that dim: every device evaluates it on its own index range.)
  static bool invariant_along(const ExprP& e, int dim) {
    switch (e->k) {
      case Expr::Const: return true;
      case Expr::Leaf: return dim < (int)e->shape.size() && e->shape[dim] == 1;
      case Expr::Iota: return e->iota_dim != dim;
      case Expr::Sym: return false;
      case Expr::Op:
        for (auto& k : e->kids)
          if (!invariant_along(k, dim)) return false;
        return true;
      case Expr::View:
        for (size_t d = 0; d < e->map.size(); ++d)
          if (e->map[d].src == dim && !invariant_along(e->kids[0], (int)d)) return false;
        return true;
    }
    return false;
  }

  // host evaluation of scalar integer expressions (loop bounds, update offsets)
  // Integer scalar bookkeeping that is affine in a loop counter: value = a * it + b (depth: which loop; 0 = constant).
  static bool affine_int(const ExprP& e, int64_t* a, int64_t* b, int* depth) {
    switch (e->k) {
      case Expr::Const: *a = 0; *b = dt_is_float(e->dt) ? (int64_t)e->f : e->i; *depth = 0; return true;
      case Expr::Sym:
        if (e->sym_depth <= 0) return false;
        *a = e->sym_a; *b = e->sym_b; *depth = e->sym_depth;
        return true;
      case Expr::View: return affine_int(e->kids[0], a, b, depth);
      case Expr::Op: {
        int64_t a0 = 0, b0 = 0, a1 = 0, b1 = 0;
        int d0 = 0, d1 = 0;
        if (e->kids.size() >= 1 && !affine_int(e->kids[0], &a0, &b0, &d0)) return false;
        if (e->kids.size() >= 2 && !affine_int(e->kids[1], &a1, &b1, &d1)) return false;
        if (d0 && d1 && d0 != d1) return false;  // counters of two different loops
        *depth = d0 ? d0 : d1;
        switch (e->vmop) {
          case VM_IADD: *a = a0 + a1; *b = b0 + b1; return true;
          case VM_ISUB: *a = a0 - a1; *b = b0 - b1; return true;
          case VM_IMUL:
            if (a0 && a1) return false;
            *a = a0 * b1 + a1 * b0; *b = b0 * b1;
            return true;
          case VM_MOV: *a = a0; *b = b0; return true;
          default: return false;
        }
      }
      default: return false;
    }
  }
  static bool const_int(const ExprP& e, int64_t* out) {
    switch (e->k) {
      case Expr::Const: *out = dt_is_float(e->dt) ? (int64_t)e->f : e->i; return true;
      case Expr::View: return const_int(e->kids[0], out);
      case Expr::Op: {
        int64_t a = 0, b = 0;
        if (e->kids.size() >= 1 && !const_int(e->kids[0], &a)) return false;
        if (e->kids.size() >= 2 && !const_int(e->kids[1], &b)) return false;
        switch (e->vmop) {
          case VM_IADD: *out = a + b; return true;
          case VM_ISUB: *out = a - b; return true;
          case VM_IMUL: *out = a * b; return true;
          case VM_MOV: *out = a; return true;
          default: return false;
        }
      }
      default: return false;
    }
  }
  bool slot_writable(int slot) const {
    const Slot& s = plan.slots[slot];
    if (s.kind == SlotK::Temp) return true;
    if (s.kind == SlotK::Arg) return s.writable;
    return false;
  }
  static void collect_leaves(const ExprP& e, std::vector<const Expr*>& out, std::set<const Expr*>& seen) {
    if (!seen.insert(e.get()).second) return;
    if (e->k == Expr::Leaf) out.push_back(e.get());
    for (auto& k : e->kids) collect_leaves(k, out, seen);
  }

  // ---- program assembly ---------------------------------------------------
  struct OutSpec {
    int slot;
    DT dt;
    int64_t offset;
    std::vector<int64_t> stride;  // per root dim
    int vnode;
  };

  // Strength-reduce the node list: constants become immediates of their consumer, and a
  // multiply whose only consumer is an add merges into one multiply-add instruction (still
  // two roundings, so results are unchanged).  Returns which nodes are no longer needed.
  // Set by a caller of assemble() that needs more than the outputs kept in registers to the end of the program
  // (the values a GEMM epilogue sums): value nodes in, their registers out.  asm_fixed_space keeps the root space
  // exactly as given (no reordering or merging of dims).
  std::vector<int> asm_pinned, asm_pinned_regs;
  bool asm_fixed_space = false;

  std::vector<bool> peephole(Lowering& L, const std::vector<OutSpec>& outs, int result_vnode) {
    size_t nn = L.nodes.size();
    std::vector<int> nuses(nn, 0);
    std::vector<bool> pinned(nn, false), dead(nn, false);
    for (auto& o : outs) pinned[o.vnode] = true;
    for (int v : asm_pinned) pinned[v] = true;
    if (result_vnode >= 0) pinned[result_vnode] = true;
    auto count = [&]() {
      std::fill(nuses.begin(), nuses.end(), 0);
      for (size_t k = 0; k < nn; ++k) {
        const VNode& n = L.nodes[k];
        if (dead[k] || n.leaf >= 0 || n.op == VM_IOTA) continue;
        for (int u : {n.a, n.b, n.c})
          if (u >= 0) nuses[u]++;
      }
    };
    auto is_const = [&](int v) { return v >= 0 && L.nodes[v].leaf < 0 && L.nodes[v].op == VM_CONST; };
    for (size_t k = 0; k < nn; ++k) {
      VNode& n = L.nodes[k];
      if (n.leaf >= 0) continue;
      int imm_op = -1, rimm_op = -1;
      switch (n.op) {
        case VM_ADD: imm_op = rimm_op = VM_ADDI; break;
        case VM_MUL: imm_op = rimm_op = VM_MULI; break;
        case VM_MAX: imm_op = rimm_op = VM_MAXI; break;
        case VM_MIN: imm_op = rimm_op = VM_MINI; break;
        case VM_SUB: imm_op = VM_SUBI; rimm_op = VM_RSUBI; break;
        case VM_DIV: imm_op = VM_DIVI; rimm_op = VM_RDIVI; break;
        default: break;
      }
      if (imm_op < 0 || L.wide) continue;  // a wide program's constants are table entries, not immediates
      if (is_const(n.b)) { n.imm = L.nodes[n.b].imm; n.op = imm_op; n.b = -1; }
      else if (is_const(n.a)) { n.imm = L.nodes[n.a].imm; n.op = rimm_op; n.a = n.b; n.b = -1; }
    }
    count();
    for (size_t k = 0; k < nn; ++k) {
      VNode& n = L.nodes[k];
      if (n.leaf >= 0 || n.op != VM_ADD) continue;
      for (int sw = 0; sw < 2; ++sw) {
        int m = sw ? n.b : n.a, other = sw ? n.a : n.b;
        if (m >= 0 && L.nodes[m].leaf < 0 && L.nodes[m].op == VM_MUL && nuses[m] == 1 && !pinned[m]) {
          n.op = VM_MULADD;
          n.a = L.nodes[m].a;
          n.b = L.nodes[m].b;
          n.c = other;
          dead[m] = true;
          break;
        }
      }
    }
    count();
    for (size_t k = 0; k < nn; ++k)
      if (L.nodes[k].leaf < 0 && nuses[k] == 0 && !pinned[k]) dead[k] = true;
    return dead;
  }

  // Turn lowered nodes into prog (register allocation, dim sorting/collapsing).
  void assemble(Step& st, Lowering& L, std::vector<OutSpec> outs, int result_vnode, const std::vector<int>& cls, bool by_output) {
    if (L.leaves.size() > (size_t)kVmMaxLeaves) throw Error(RX_ERR_PLAN, "fusion group reads more than " + std::to_string(kVmMaxLeaves) + " operands");
    if (outs.size() > (size_t)kVmMaxOuts) throw Error(RX_ERR_PLAN, "fusion group writes too many results");
    Space sp;
    sp.dim = L.root;
    sp.cls = cls;
    sp.origin.resize(L.root.size());
    for (size_t d = 0; d < L.root.size(); ++d) sp.origin[d] = (int)d;
    int dominant = -1;
    int64_t best = -1;
    for (size_t k = 0; k < L.leaves.size(); ++k) {
      sp.lstride.push_back(L.leaves[k].stride);
      int64_t span = 1;
      for (size_t d = 0; d < L.root.size(); ++d)
        if (L.leaves[k].stride[d] != 0) span *= L.root[d];
      if (span > best) { best = span; dominant = (int)k; }
    }
    for (auto& o : outs) sp.ostride.push_back(o.stride);
    if (!asm_fixed_space) normalise_space(sp, dominant, by_output, !L.has_iota);
    if (sp.dim.size() > (size_t)kMaxRank) throw Error(RX_ERR_PLAN, "fusion group iteration space has rank > " + std::to_string(kMaxRank));
    VmProgram& P = st.prog;
    memset(&P, 0, sizeof P);
    P.rank = (int)sp.dim.size();
    for (int d = 0; d < kMaxRank; ++d) P.dim[d] = d < P.rank ? sp.dim[d] : 1;
    std::vector<int64_t> cstr = canon_strides(sp.dim);
    const std::vector<VNode> original_nodes = L.nodes;  // chain recognition below looks at the unreduced form
    const std::vector<bool> dead = peephole(L, outs, result_vnode);
    // register allocation (linear scan over the node list, which is in topological order)
    size_t nn = L.nodes.size();
    std::vector<int> last(nn, -1);
    for (size_t k = 0; k < nn; ++k) {
      const VNode& n = L.nodes[k];
      if (n.op == VM_IOTA || dead[k]) continue;
      for (int u : {n.a, n.b, n.c})
        if (u >= 0) last[u] = (int)k;
    }
    for (auto& o : outs) last[o.vnode] = (int)nn + 1;
    for (int v : asm_pinned) last[v] = (int)nn + 1;
    if (result_vnode >= 0) last[result_vnode] = (int)nn + 1;
    std::vector<int> reg(nn, -1);
    std::vector<int> free_regs;
    for (int r = kVmMaxRegs - 1; r >= 0; --r) free_regs.push_back(r);
    auto alloc = [&]() {
      if (free_regs.empty()) throw Error(RX_ERR_PLAN, "fusion group needs more than " + std::to_string(kVmMaxRegs) + " live values");
      int r = free_regs.back();
      free_regs.pop_back();
      return r;
    };
    // leaves first: they are loaded before the program runs
    for (size_t k = 0; k < nn; ++k)
      if (L.nodes[k].leaf >= 0) reg[k] = alloc();
    st.leaf_slot.clear();
    P.n_leaves = (int)L.leaves.size();
    P.all_linear = L.has_iota ? 0 : 1;
    for (size_t k = 0; k < L.leaves.size(); ++k) {
      VmLeaf& vl = P.leaf[k];
      vl.ptr = nullptr;
      vl.offset = L.leaves[k].offset;
      vl.elem = elem_of(L.leaves[k].dt);
      bool lin = true, scalar = true;
      for (int d = 0; d < P.rank; ++d) {
        vl.stride[d] = sp.lstride[k][d];
        lin = lin && vl.stride[d] == cstr[d];
        scalar = scalar && vl.stride[d] == 0;
      }
      vl.linear = scalar ? 2 : (lin ? 1 : 0);
      if (!vl.linear) P.all_linear = 0;
      for (size_t q = 0; q < nn; ++q)
        if (L.nodes[q].leaf == (int)k) vl.reg = (uint8_t)reg[q];
      st.leaf_slot.push_back(L.leaves[k].slot);
    }
    // uses of each value, to decide which results must reach the register file
    std::vector<int> nuses(nn, 0);
    for (size_t k = 0; k < nn; ++k) {
      const VNode& n = L.nodes[k];
      if (n.leaf >= 0 || n.op == VM_IOTA || dead[k]) continue;
      for (int u : {n.a, n.b, n.c})
        if (u >= 0) nuses[u]++;
    }
    std::vector<bool> is_output(nn, false);
    for (auto& o : outs) is_output[o.vnode] = true;
    for (int v : asm_pinned) is_output[v] = true;
    if (result_vnode >= 0) is_output[result_vnode] = true;
    // ---- emission for the accumulator machine: acc = f(acc, R[b], R[c] | imm) --------------------
    int prev = -1;  // node whose value is in the accumulator
    int ni = 0;
    std::vector<int> instr_of(nn, -1);
    auto mark_store = [&](int vnode) {
      if (vnode >= 0 && L.nodes[vnode].leaf < 0 && instr_of[vnode] >= 0) P.ins[instr_of[vnode]].flags |= VMF_STORE;
    };
    auto push = [&](int op) -> VmInstr& {
      if (ni >= kVmMaxInstr) throw Error(RX_ERR_PLAN, "fusion group longer than " + std::to_string(kVmMaxInstr) + " ops");
      VmInstr& in = P.ins[ni++];
      in = VmInstr{};
      in.op = (uint8_t)op;
      return in;
    };
    auto rg = [&](int vnode) {  // operand read from the register file
      mark_store(vnode);
      return (uint8_t)reg[vnode];
    };
    auto load_acc = [&](int vnode) {
      if (vnode == prev) return;
      uint8_t r = rg(vnode);
      VmInstr& in = push(VM_LD);
      in.b = r;
    };
    auto commutative = [](int op) {
      return op == VM_ADD || op == VM_MUL || op == VM_MAX || op == VM_MIN || op == VM_IADD || op == VM_IMUL || op == VM_IMAX || op == VM_IMIN ||
             op == VM_AND || op == VM_OR || op == VM_XOR;
    };
    auto is_binary = [](int op) {
      return (op >= VM_ADD && op <= VM_POW) || (op >= VM_IADD && op <= VM_IMIN) || op == VM_AND || op == VM_OR || op == VM_XOR || op == VM_FCMP || op == VM_ICMP ||
             op == VM_ATAN2 || op == VM_REM;
    };
    for (size_t k = 0; k < nn; ++k) {
      const VNode& n = L.nodes[k];
      if (n.leaf < 0 && !dead[k]) {
        // release operands whose last use is this node before allocating dst, so dst may reuse them
        if (n.op != VM_IOTA)
          for (int u : {n.a, n.b, n.c})
            if (u >= 0 && last[u] == (int)k && reg[u] >= 0) {
              bool dup = false;
              for (int f : free_regs) dup = dup || f == reg[u];
              if (!dup) free_regs.push_back(reg[u]);
            }
        reg[k] = alloc();
        int op = n.op;
        if (op == VM_IOTA) {
          int nd = -1;
          for (int d = 0; d < P.rank; ++d)
            if (sp.origin[d] == n.a) nd = d;
          VmInstr& in = push(nd < 0 ? VM_CONST : VM_IOTA);  // unit dim: index is 0
          in.a = (uint8_t)(nd < 0 ? 0 : nd);
        } else if (op == VM_CONST) {
          VmInstr& in = push(VM_CONST);
          in.imm = n.imm;
          if (L.wide && n.cmp == 32) {  // an f32 constant inside a wide program: same value, as a double
            float f32v;
            memcpy(&f32v, &n.imm, 4);
            in.imm = (uint32_t)L.wconst((double)f32v);
            in.c = 1;
          } else if (n.cmp == 64) {
            in.c = 1;
          }
        } else if (op == VM_SELECT) {
          load_acc(n.a);
          uint8_t rb = rg(n.b), rc = rg(n.c);
          VmInstr& in = push(VM_SELECT);
          in.b = rb;
          in.c = rc;
        } else if (op == VM_MULADD) {
          int a = n.a, b = n.b, c = n.c;
          if (b == prev && a != prev) std::swap(a, b);
          if (a != prev && c == prev) {
            uint8_t rb = rg(a), rc = rg(b);
            VmInstr& in = push(VM_MULADD_C);
            in.b = rb;
            in.c = rc;
          } else {
            load_acc(a);
            uint8_t rb = rg(b), rc = rg(c);
            VmInstr& in = push(VM_MULADD);
            in.b = rb;
            in.c = rc;
          }
        } else if (is_binary(op)) {
          int a = n.a, b = n.b, cmp = n.cmp;
          if (op == VM_MUL && a == b) {
            load_acc(a);
            push(VM_SQR);
          } else {
            if (b == prev && a != prev) {
              // the accumulator holds the right operand: swap, reversing the op where it matters
              if (commutative(op)) std::swap(a, b);
              else if (op == VM_SUB) { op = VM_RSUB; std::swap(a, b); }
              else if (op == VM_DIV) { op = VM_RDIV; std::swap(a, b); }
              else if (op == VM_FCMP || op == VM_ICMP) {
                cmp = cmp == CMP_LT ? CMP_GT : cmp == CMP_GT ? CMP_LT : cmp == CMP_LE ? CMP_GE : cmp == CMP_GE ? CMP_LE : cmp;
                std::swap(a, b);
              }
            }
            load_acc(a);
            uint8_t rb = rg(b);
            VmInstr& in = push(op);
            in.b = rb;
            if (op == VM_FCMP || op == VM_ICMP) in.c = (uint8_t)cmp;
          }
        } else {
          // unary forms (including immediates)
          load_acc(n.a);
          VmInstr& in = push(op);  // VM_MOV: the accumulator already holds the value
          in.imm = n.imm;
        }
        P.ins[ni - 1].dst = (uint8_t)reg[k];
        instr_of[k] = ni - 1;
        if (is_output[k]) P.ins[ni - 1].flags |= VMF_STORE;
        prev = (int)k;
      }
      if (last[k] < 0 && reg[k] >= 0 && L.nodes[k].leaf < 0) free_regs.push_back(reg[k]);  // dead value
    }
    P.n_instr = ni;
    P.n_outs = (int)outs.size();
    st.out_slot.clear();
    for (size_t k = 0; k < outs.size(); ++k) {
      VmOut& vo = P.out[k];
      vo.ptr = nullptr;
      vo.offset = outs[k].offset;
      vo.elem = elem_of(outs[k].dt);
      vo.reg = (uint8_t)reg[outs[k].vnode];
      bool lin = true;
      for (int d = 0; d < P.rank; ++d) {
        vo.stride[d] = sp.ostride[k][d];
        lin = lin && vo.stride[d] == cstr[d];
      }
      vo.linear = lin ? 1 : 0;
      if (!lin && result_vnode < 0) P.all_linear = 0;  // a reduction's output is a single store per group
      st.out_slot.push_back(outs[k].slot);
    }
    P.result_reg = result_vnode >= 0 ? reg[result_vnode] : 0;
    asm_pinned_regs.clear();
    for (int v : asm_pinned) asm_pinned_regs.push_back(reg[v]);
    st.outer = st.red_n = st.inner = 1;
    // reduction classes after normalisation -> [outer][red][inner]
    if (!cls.empty() && std::find(cls.begin(), cls.end(), 1) != cls.end()) {
      std::vector<int> c = sp.cls;
      // strip to run-lengths: K* R+ K*
      size_t a = 0;
      while (a < c.size() && c[a] == 0) ++a;
      size_t b = a;
      while (b < c.size() && c[b] == 1) ++b;
      for (size_t q = b; q < c.size(); ++q)
        if (c[q] == 1) throw Error(RX_ERR_PLAN, "reduce over non-adjacent dimensions is not supported");
      if (a > 1 || b - a > 1 || c.size() - b > 1) {
        // more than one dim per group survived collapsing: strided group, handled by the generic kernels via rank-4 indexing
      }
      st.prog.fast_id = FAST_NONE;
    }
    L.nodes = original_nodes;
    detect_fast(st, L, result_vnode >= 0 ? result_vnode : (outs.empty() ? -1 : outs[0].vnode));
    if (L.wide) {
      if (L.wconsts.size() > (size_t)kVmMaxWideConsts) throw Error(RX_ERR_PLAN, "fusion group uses more than " + std::to_string(kVmMaxWideConsts) + " distinct f64 constants");
      P.wide = 1;
      P.n_wconst = (int)L.wconsts.size();
      for (size_t k = 0; k < L.wconsts.size(); ++k) P.wconst[k] = L.wconsts[k];
      P.fast_id = FAST_NONE;  // the hand-fused kernels are f32
    }
    cls_after = sp.cls;
  }
  std::vector<int> cls_after;

  // Recognise chains that have compile-time-fused kernels.
  void detect_fast(Step& st, Lowering& L, int root) {
    VmProgram& P = st.prog;
    P.fast_id = FAST_NONE;
    if (root < 0) return;
    auto is_f32_leaf = [&](int v) { return v >= 0 && L.nodes[v].leaf >= 0 && L.leaves[L.nodes[v].leaf].dt == DT::F32; };
    const VNode& r = L.nodes[root];
    if (is_f32_leaf(root) && L.leaves.size() == 1) { P.fast_id = FAST_IDENTITY; return; }
    if (r.op == VM_ADD && L.leaves.size() == 2) {
      for (int sw = 0; sw < 2; ++sw) {
        int s = sw ? r.b : r.a, o = sw ? r.a : r.b;
        if (s >= 0 && L.nodes[s].op == VM_SIN && is_f32_leaf(L.nodes[s].a) && is_f32_leaf(o) && L.nodes[s].a != o) {
          // leaf 0 must be the sine operand
          if (L.nodes[L.nodes[s].a].leaf == 1) swap_leaves(st, 0, 1);
          P.fast_id = FAST_SIN_ADD;
          return;
        }
      }
    }
    if (r.op == VM_EXP && L.leaves.size() == 2) {
      const VNode& sub = L.nodes[r.a];
      if (sub.op == VM_SUB && is_f32_leaf(sub.a) && is_f32_leaf(sub.b) && sub.a != sub.b) {
        if (L.nodes[sub.a].leaf == 1) swap_leaves(st, 0, 1);
        P.fast_id = FAST_EXP_SUB;
        return;
      }
    }
    if (r.op == VM_MUL && L.leaves.size() == 5) {
      for (int sw = 0; sw < 2; ++sw) {
        int c = sw ? r.b : r.a, x = sw ? r.a : r.b;
        if (c < 0 || x < 0 || L.nodes[c].op != VM_CONST || L.nodes[c].leaf >= 0) continue;
        // x = ((((l_a + l_b) + l_c) + l_d) + l_e), left-leaning
        std::vector<int> chain;
        int curv = x;
        bool ok = true;
        for (int depth = 0; depth < 4 && ok; ++depth) {
          const VNode& a = L.nodes[curv];
          if (a.op != VM_ADD || !is_f32_leaf(a.b)) { ok = false; break; }
          chain.push_back(L.nodes[a.b].leaf);
          curv = a.a;
        }
        if (!ok || !is_f32_leaf(curv)) continue;
        chain.push_back(L.nodes[curv].leaf);
        std::reverse(chain.begin(), chain.end());
        std::set<int> uniq(chain.begin(), chain.end());
        if (uniq.size() != 5) continue;
        // reorder leaves into evaluation order
        std::vector<VmLeaf> nl;
        std::vector<int> ns;
        for (int q : chain) { nl.push_back(P.leaf[q]); ns.push_back(st.leaf_slot[q]); }
        for (int q = 0; q < 5; ++q) { P.leaf[q] = nl[q]; st.leaf_slot[q] = ns[q]; }
        // the interpreter form stays valid: leaf.reg travels with the leaf
        memcpy(&P.fast_c, &L.nodes[c].imm, 4);
        P.fast_id = FAST_STENCIL5_MUL;
        return;
      }
    }
  }
  void swap_leaves(Step& st, int a, int b) {
    std::swap(st.prog.leaf[a], st.prog.leaf[b]);
    std::swap(st.leaf_slot[a], st.leaf_slot[b]);
  }

  // ---- step emitters -------------------------------------------------------
  // out[shape-indexed] = expr, written at `offset` with `ostride` into `slot`.
  // What the most recently emitted Map step computes, kept so that the next map can be merged into it.
  struct LastMap {
    std::vector<Step>* where = nullptr;
    size_t index = 0;
    struct Out { int slot; ExprP expr; int64_t offset; std::vector<int64_t> stride; };
    std::vector<Out> outs;
  } last_map;

  // Replace every whole-slot read of `slot` in `e` by `repl`.  *blocked is set if `slot` is also read in a way that
  // cannot be replaced (a window of it): the reader must then stay a separate launch after the writer.
  ExprP subst_slot(const ExprP& e, int slot, const ExprP& repl, std::map<const Expr*, ExprP>& memo, bool* found, bool* blocked) {
    auto it = memo.find(e.get());
    if (it != memo.end()) return it->second;
    ExprP r = e;
    if (e->k == Expr::Leaf) {
      if (e->slot == slot) {
        if (whole_slot(e) && e->shape == repl->shape && e->dt == repl->dt) { r = repl; *found = true; }
        else *blocked = true;
      }
    } else if (e->k == Expr::Op || e->k == Expr::View) {
      std::vector<ExprP> kids;
      bool changed = false;
      for (auto& k : e->kids) {
        kids.push_back(subst_slot(k, slot, repl, memo, found, blocked));
        changed = changed || kids.back() != k;
      }
      if (changed) {
        auto c = std::make_shared<Expr>(*e);
        c->kids = kids;
        r = c;
      }
    }
    memo[e.get()] = r;
    return r;
  }
  // Is `slot` read by a value that an op after `op` (or the enclosing region's result) still uses?  Values are lazy
  // expressions, so a value that has been consumed only by ops planned so far no longer matters: whatever it fed
  // either became a step already emitted or lives on inside another value, which is examined in its own right.
  bool read_later(int slot, const Op& op) {
    for (size_t w = 0; w < env.size(); ++w) {
      if (!env[w]) continue;
      int left = remaining[w] - (int)std::count(op.in.begin(), op.in.end(), (int)w);
      if (left <= 0) continue;
      std::set<const Expr*> seen;
      if (reads_slot(env[w], slot, seen)) return true;
    }
    return false;
  }
  bool reads_slot(const ExprP& e, int slot, std::set<const Expr*>& seen) {
    if (!seen.insert(e.get()).second) return false;
    if (e->k == Expr::Leaf) return e->slot == slot;
    for (auto& k : e->kids)
      if (reads_slot(k, slot, seen)) return true;
    return false;
  }

  // ---- elementwise and reduction work fused into the epilogue of the GEMM that produces its operand ---------------
  // After a dot_general has been emitted as a Gemm step, maps and additive reductions over the [M][N] result whose
  // other operands are per-element ([M][N], any row stride), per-column ([N], broadcast along m) or scalars join
  // that step: the chain runs on the accumulator while it is still on chip.  What joins must not depend on any
  // step emitted after the GEMM.  D itself stays a result of the step until the end of planning, when it is dropped
  // if nothing else reads it.  Only at the top level of @main (steps of a loop body are not revisited), on shapes the
  // two-CTA tensor-core kernel takes, and when run-time compilation is available (RX_GEMM_EPILOGUE=0 switches it off).
  struct GemmFusion {
    std::vector<Step>* where = nullptr;
    size_t index = 0;
    int d_slot = -1;
    DT dt = DT::BF16;
    int64_t M = 0, N = 0;
    std::string base_note;
    struct Out { int slot; ExprP expr; std::string note; };
    std::vector<Out> outs;
    struct Sum { int partial_slot; ExprP expr; bool col; std::string note; };
    std::vector<Sum> sums;
    int finish_index = -1;
  };
  std::vector<GemmFusion> fusions;  // every fused GEMM of the plan; the last one is the one that can still grow
  bool fusion_open = false;

  static bool epilogue_enabled() {
    const bool on = !(getenv("RX_GEMM_EPILOGUE") && atoi(getenv("RX_GEMM_EPILOGUE")) == 0) && !getenv("RX_GEMM_SIMT") && !getenv("RX_GEMM_1CTA");
    return on && jit_available();
  }
  GemmFusion* open_fusion() { return fusion_open && !fusions.empty() && fusions.back().where == cur ? &fusions.back() : nullptr; }

  // (Re)build the GEMM step's epilogue program from the fusion record.  false: it does not fit the kernel (too many
  // operands / results / live values, an operand with a stride the epilogue cannot walk, ...); the step is unchanged.
  bool lower_fusion(GemmFusion& g, bool keep_d) {
    Step tmp = (*g.where)[g.index];
    Lowering L(std::vector<int64_t>{g.M, g.N});
    const RMap id = Lowering::identity(2);
    const std::vector<int64_t> dense = {g.N, 1};
    Type dtype{g.dt, {g.M, g.N}};
    std::vector<OutSpec> outs;
    const int acc_v = L.lower(leaf(g.d_slot, dtype), id);
    if (keep_d) outs.push_back(OutSpec{g.d_slot, g.dt, 0, dense, acc_v});
    for (auto& o : g.outs) outs.push_back(OutSpec{o.slot, plan.slots[o.slot].type.dt, 0, dense, L.lower(o.expr, id)});
    std::vector<int> pinned;
    for (auto& su : g.sums) pinned.push_back(L.lower(su.expr, id));
    if (L.has_iota || outs.empty() && pinned.empty()) return false;
    asm_pinned = pinned;
    asm_fixed_space = true;
    std::vector<int> regs;
    try {
      assemble(tmp, L, outs, -1, std::vector<int>{0, 0}, true);
      regs = asm_pinned_regs;
    } catch (const Error& e) {
      asm_pinned.clear();
      asm_fixed_space = false;
      if (e.code != RX_ERR_PLAN) throw;
      return false;
    }
    asm_pinned.clear();
    asm_fixed_space = false;
    VmProgram& P = tmp.prog;
    P.fast_id = FAST_NONE;
    int acc_leaf = -1;
    for (int k = 0; k < P.n_leaves; ++k) {
      const VmLeaf& l = P.leaf[k];
      if (l.elem != EL_F32 && l.elem != EL_BF16) return false;
      if (tmp.leaf_slot[k] == g.d_slot) {
        if (acc_leaf >= 0 || l.offset != 0 || l.stride[0] != g.N || l.stride[1] != 1) return false;  // read other than at (m, n)
        acc_leaf = k;
      } else if (l.stride[1] != 0 && l.stride[1] != 1) {
        return false;
      }
    }
    if (acc_leaf < 0) return false;
    for (int k = 0; k < P.n_outs; ++k)
      if (P.out[k].elem != EL_F32 && P.out[k].elem != EL_BF16) return false;
    GemmDesc& gd = tmp.gemm;
    gd.has_epilogue = true;
    gd.acc_leaf = acc_leaf;
    gd.n_leaves = P.n_leaves;
    gd.n_col = gd.n_full = 0;
    for (size_t q = 0; q < g.sums.size(); ++q) {
      if (g.sums[q].col) {
        if (gd.n_col == 2) return false;
        gd.col_reg[gd.n_col] = regs[q];
        gd.col_slot[gd.n_col++] = g.sums[q].partial_slot;
      } else {
        if (gd.n_full == 2) return false;
        gd.full_reg[gd.n_full] = regs[q];
        gd.full_slot[gd.n_full++] = g.sums[q].partial_slot;
      }
    }
    std::string note = g.base_note + " + epilogue[";
    bool first = true;
    auto add = [&](const std::string& t) { note += (first ? "" : "; ") + t; first = false; };
    if (keep_d) add("product");
    for (auto& o : g.outs) add(o.note);
    for (auto& su : g.sums) add(su.note);
    tmp.note = note + "]";
    (*g.where)[g.index] = std::move(tmp);
    return true;
  }

  // Slots that steps emitted after the GEMM read or write: nothing that joins the epilogue may touch them.
  bool touched_after(const GemmFusion& g, const std::set<int>& slots) {
    for (size_t q = g.index + 1; q < g.where->size(); ++q) {
      const Step& t = (*g.where)[q];
      if (t.kind == StepK::Loop) return true;
      std::vector<int> all = t.leaf_slot;
      all.insert(all.end(), t.out_slot.begin(), t.out_slot.end());
      for (int w : {t.src_slot, t.dst_slot, t.gemm.a_slot, t.gemm.b_slot, t.gemm.d_slot}) all.push_back(w);
      for (auto& j : t.sums) { all.push_back(j.src_slot); all.push_back(j.dst_slot); }
      for (int w : all)
        if (w >= 0 && slots.count(w)) {
          // the partial buffers of this very fusion are written by the GEMM and read by its SumPartials step
          bool own_partial = false;
          for (auto& su : g.sums) own_partial = own_partial || su.partial_slot == w;
          if (!own_partial) return true;
        }
    }
    return false;
  }
  bool fusable_expr(GemmFusion& g, const ExprP& e) {
    if (e->shape != std::vector<int64_t>{g.M, g.N}) return false;
    std::set<const Expr*> seen;
    if (!reads_slot(e, g.d_slot, seen)) return false;
    std::vector<const Expr*> lv;
    std::set<const Expr*> seen2;
    collect_leaves(e, lv, seen2);
    std::set<int> slots;
    for (auto* l : lv)
      if (l->slot != g.d_slot) slots.insert(l->slot);
    return !touched_after(g, slots);
  }
  bool try_fuse_map(const ExprP& e, int slot, int64_t offset, const std::vector<int64_t>& ostride, const std::string& note) {
    GemmFusion* g = open_fusion();
    if (!g || offset != 0 || !fusable_expr(*g, e)) return false;
    if (ostride != canon_strides(e->shape) || prod(e->shape) != plan.slots[slot].type.numel() || slot == g->d_slot) return false;
    for (auto& o : g->outs)
      if (o.slot == slot) return false;
    if (touched_after(*g, std::set<int>{slot})) return false;
    g->outs.push_back({slot, e, note});
    if (!lower_fusion(*g, true)) {
      g->outs.pop_back();
      return false;
    }
    return true;
  }
  // sum over dim 0 (per column) or over both dims of an [M][N] chain value; returns the slot of the result or -1
  int try_fuse_sum(const ExprP& X, const std::vector<int64_t>& dims, const Type& rt, double init_f) {
    GemmFusion* g = open_fusion();
    if (!g || X->dt != DT::F32 || rt.dt != DT::F32 || !fusable_expr(*g, X)) return -1;
    const bool col = dims == std::vector<int64_t>{0}, full = dims == std::vector<int64_t>{0, 1};
    if (!col && !full) return -1;
    const int64_t tiles = ((g->M + 255) / 256) * ((g->N + 255) / 256);
    const size_t n_slots = plan.slots.size();
    Type pt{DT::F32, col ? std::vector<int64_t>{g->M / 32, g->N} : std::vector<int64_t>{tiles * 16}};  // one partial per (tile, CTA, epilogue warp)
    const int partial = new_slot(pt);
    g->sums.push_back({partial, X, col, col ? "column sums" : "full sum"});
    if (!lower_fusion(*g, true)) {
      g->sums.pop_back();
      plan.slots.resize(n_slots);
      return -1;
    }
    const int dst = new_slot(rt);
    SumJob job;
    job.src_slot = partial;
    job.dst_slot = dst;
    job.rows = col ? g->M / 32 : tiles * 16;
    job.n = col ? g->N : 1;
    job.init = init_f;
    if (g->finish_index >= 0 && (size_t)g->finish_index + 1 == g->where->size() && (*g->where)[g->finish_index].sums.size() < 4) {
      (*g->where)[g->finish_index].sums.push_back(job);
    } else {
      Step fin;
      fin.kind = StepK::SumPartials;
      fin.note = "ordered sum of the epilogue partials";
      fin.sums.push_back(job);
      g->where->push_back(std::move(fin));
      g->finish_index = (int)g->where->size() - 1;
    }
    last_map.where = nullptr;
    return dst;
  }
  // End of planning: a fused GEMM whose product nobody else reads does not store it.
  void finalize_fusions() {
    std::function<bool(const std::vector<Step>&, int, const Step*)> reads = [&](const std::vector<Step>& steps, int slot, const Step* self) {
      for (const Step& t : steps) {
        if (&t == self) continue;
        for (int w : t.leaf_slot) if (w == slot) return true;
        for (int w : {t.src_slot, t.gemm.a_slot, t.gemm.b_slot}) if (w == slot) return true;
        if (t.kind == StepK::AllReduce && t.dst_slot == slot) return true;
        for (auto& j : t.sums) if (j.src_slot == slot) return true;
        for (int w : t.state_slots) if (w == slot) return true;
        for (int w : t.yield_slots) if (w == slot) return true;
        if (reads(t.body, slot, self)) return true;
      }
      return false;
    };
    for (auto& g : fusions) {
      Step* self = &(*g.where)[g.index];
      if (!self->gemm.has_epilogue) continue;
      bool needed = reads(plan.steps, g.d_slot, self);
      for (auto& rb : plan.results) needed = needed || rb.slot == g.d_slot;
      if (needed) continue;
      if (lower_fusion(g, false)) plan.slots[g.d_slot].dead = true;
    }
  }

  // ---- step emitters -------------------------------------------------------
  // out[shape-indexed] = expr, written at `offset` with `ostride` into `slot`.
  //
  // Merging: when this map reads, element for element, what the map emitted just before it wrote (a value that
  // was materialised because it has several consumers, e.g. the activation that both the next layer and the
  // backward pass need), the two become ONE launch with both outputs: the shared value is computed once in
  // registers, stored, and used -- it is not written and read back, and the operands the two chains have in common
  // are loaded once.  Results are identical: the register holds exactly the value that is stored.
  // does any value of the expression have type f64?  (Such a group is lowered as a wide program.)
  static bool expr_wide(const ExprP& e, std::set<const Expr*>& seen) {
    if (!seen.insert(e.get()).second) return false;
    if (e->dt == DT::F64) return true;
    for (auto& k : e->kids)
      if (expr_wide(k, seen)) return true;
    return false;
  }

  void emit_map(const ExprP& e, int slot, int64_t offset, const std::vector<int64_t>& ostride, const std::string& note) {
    if (try_fuse_map(e, slot, offset, ostride, note)) {
      last_map.where = nullptr;
      return;
    }
    static const bool merge_off = getenv("RX_NO_MAP_MERGE") != nullptr;
    if (!merge_off && last_map.where == cur && last_map.index < cur->size() && (*cur)[last_map.index].kind == StepK::Map &&
        last_map.outs.size() + 1 <= (size_t)kVmMaxOuts && !last_map.outs.empty() && last_map.outs[0].expr->shape == e->shape) {
      ExprP merged = e;
      bool found = false, blocked = false;
      {
        // an f64 group and a 32-bit group stay two launches: merged, the narrow one's floats would be computed as doubles
        std::set<const Expr*> seen;
        const bool wide_here = expr_wide(e, seen) || plan.slots[slot].type.dt == DT::F64;
        blocked = wide_here != ((*cur)[last_map.index].prog.wide != 0);
      }
      for (auto& o : last_map.outs) {
        std::map<const Expr*, ExprP> memo;
        merged = subst_slot(merged, o.slot, o.expr, memo, &found, &blocked);
        std::set<const Expr*> seen;
        blocked = blocked || reads_slot(o.expr, slot, seen) || o.slot == slot;  // the earlier chain must not read what this one writes
      }
      // steps emitted since that map (reductions of its result, say) stay where they are; this map moves up in front
      // of them, which is fine as long as none of them writes anything it reads
      if (found && !blocked) {
        std::set<int> written;
        for (size_t q = last_map.index + 1; q < cur->size(); ++q) {
          const Step& t = (*cur)[q];
          if (t.kind == StepK::Loop || t.kind == StepK::Stencil) blocked = true;
          for (int w : t.out_slot) written.insert(w);
          for (int w : {t.dst_slot, t.gemm.d_slot})
            if (w >= 0) written.insert(w);
        }
        for (int w : written) {
          std::set<const Expr*> seen;
          blocked = blocked || w == slot || reads_slot(merged, w, seen);
        }
      }
      if (found && !blocked) {
        Step st;
        st.kind = StepK::Map;
        st.note = (*cur)[last_map.index].note + " + " + note;
        try {
          Lowering L(e->shape);
          std::vector<OutSpec> outs;
          for (auto& o : last_map.outs)
            outs.push_back(OutSpec{o.slot, plan.slots[o.slot].type.dt, o.offset, o.stride, L.lower(o.expr, Lowering::identity(e->shape.size()))});
          outs.push_back(OutSpec{slot, plan.slots[slot].type.dt, offset, ostride, L.lower(merged, Lowering::identity(e->shape.size()))});
          std::vector<int> cls(e->shape.size(), 0);
          assemble(st, L, outs, -1, cls, true);
          (*cur)[last_map.index] = std::move(st);
          last_map.outs.push_back({slot, merged, offset, ostride});
          return;
        } catch (const Error& err) {
          if (err.code != RX_ERR_PLAN) throw;  // too many operands / instructions / registers for one group: keep two launches
        }
      }
    }
    Step st;
    st.kind = StepK::Map;
    st.note = note;
    Lowering L(e->shape);
    int root = L.lower(e, Lowering::identity(e->shape.size()));
    DT odt = plan.slots[slot].type.dt;
    std::vector<int> cls(e->shape.size(), 0);
    assemble(st, L, {OutSpec{slot, odt, offset, ostride, root}}, -1, cls, true);
    classify_stencil(st);
    const bool plain = st.kind == StepK::Map;
    cur->push_back(std::move(st));
    last_map.where = nullptr;
    if (plain && offset == 0 && ostride == canon_strides(e->shape) && prod(e->shape) == plan.slots[slot].type.numel()) {
      last_map.where = cur;
      last_map.index = cur->size() - 1;
      last_map.outs.clear();
      last_map.outs.push_back({slot, e, offset, ostride});
    }
  }

  // A map whose operands are shifted windows of one row-major 2-D array and whose
  // output is a window of another: run it through the shared-memory tiled kernel.
  void classify_stencil(Step& st) {
    VmProgram& P = st.prog;
    if (P.rank != 2 || P.n_leaves < 2 || P.n_outs != 1) return;
    if (P.out[0].stride[1] != 1 || P.out[0].elem != EL_F32) return;
    int64_t ld = P.leaf[0].stride[0];
    int64_t base = INT64_MAX;
    for (int k = 0; k < P.n_leaves; ++k) {
      if (st.leaf_slot[k] != st.leaf_slot[0] || P.leaf[k].elem != EL_F32) return;
      if (P.leaf[k].stride[0] != ld || P.leaf[k].stride[1] != 1) return;
      base = std::min(base, P.leaf[k].offset);
    }
    if (ld < P.dim[1]) return;
    st.st_dy.clear();
    st.st_dx.clear();
    int radius = 0;
    // offsets relative to the window origin; dx recovered as the remainder closest to zero
    int64_t row0 = base / ld, col0 = INT64_MAX;
    for (int k = 0; k < P.n_leaves; ++k) col0 = std::min(col0, P.leaf[k].offset % ld);
    for (int k = 0; k < P.n_leaves; ++k) {
      int64_t dy = P.leaf[k].offset / ld - row0, dx = P.leaf[k].offset % ld - col0;
      if (dy < 0 || dy > 8 || dx < 0 || dx > 8) return;
      st.st_dy.push_back((int)dy);
      st.st_dx.push_back((int)dx);
      radius = std::max(radius, (int)std::max(dy, dx));
    }
    if (st.leaf_slot[0] == st.out_slot[0]) return;  // in-place shifted update is not a stencil step
    st.kind = StepK::Stencil;
    st.st_rows = P.dim[0];
    st.st_cols = P.dim[1];
    st.st_src_ld = ld;
    st.st_src_off = row0 * ld + col0;
    st.st_dst_ld = P.out[0].stride[0];
    st.st_dst_off = P.out[0].offset;
    st.st_radius = radius;
  }

  int materialise(const ExprP& e, const std::string& why) {
    if (whole_slot(e)) return e->slot;
    Type t;
    t.dt = e->dt;
    t.shape = e->shape;
    int slot = new_slot(t);
    emit_map(e, slot, 0, canon_strides(e->shape), why);
    return slot;
  }
  ExprP materialised(const ExprP& e, const std::string& why) {
    if (e->k == Expr::Leaf) return e;
    Type t;
    t.dt = e->dt;
    t.shape = e->shape;
    return leaf(materialise(e, why), t);
  }

  // ---- op handlers -----------------------------------------------------------
  int join_shard(const Op& op, const std::vector<int>& ins) {
    int s = -1;
    for (int v : ins) {
      if (shard[v] < 0) continue;
      if (s >= 0 && s != shard[v]) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op " + op.name + ": operands sharded along different dimensions");
      s = shard[v];
    }
    if (s >= 0)
      for (int v : ins)
        if (shard[v] < 0 && !is_splat(env[v]) && !invariant_along(env[v], s))
          throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op " + op.name + ": a replicated operand that varies along the sharded dimension is combined with a sharded one");
    return s;
  }

  int convert_op(DT from, DT to) {
    auto cls = [](DT d) { return dt_is_float(d) ? 0 : (d == DT::PRED ? 2 : 1); };
    int a = cls(from), b = cls(to);
    if (a == 0 && b == 0) return to == DT::BF16 && from != DT::BF16 ? VM_RBF16 : VM_MOV;
    if (a == 1 && b == 0) return VM_I2F;
    if (a == 0 && b == 1) return VM_F2I;
    if (a == 2 && b == 0) return VM_P2F;
    if (a == 0 && b == 2) return VM_F2P;
    if (a == 1 && b == 2) return VM_I2P;
    return VM_MOV;  // pred->int, int->int of the same width
  }
  void check_dt(const Op& op, DT dt) {
    if (dt == DT::F32 || dt == DT::BF16 || dt == DT::S32 || dt == DT::PRED || dt == DT::F64) return;
    throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type " + std::string(dt_name(dt)) + " in " + op.name);
  }
  // bf16 arithmetic is evaluated in f32 and rounded once per op, as XLA's CPU backend does
  ExprP round_if_bf16(const ExprP& e) {
    if (e->dt != DT::BF16 || e->k != Expr::Op || e->vmop == VM_RBF16 || e->vmop == VM_MOV || e->vmop == VM_SELECT) return e;
    Type t{e->dt, e->shape};
    return mkop(VM_RBF16, t, {e});
  }

  void maybe_spill(int v) {
    // Values with several consumers are computed once when recomputation would be costly.
    ExprP e = env[v];
    // A replicated value that does not vary along some dim may later meet a tensor sharded along that dim, where
    // each device evaluates it on its own index range; a materialised copy would no longer show that it is
    // invariant, so such values stay expressions and are recomputed.
    if (nparts > 1 && shard[v] < 0)
      for (size_t d = 0; d < e->shape.size(); ++d)
        if (e->shape[d] > 1 && invariant_along(e, (int)d)) return;
    if (uses[v] > 1 && e->k != Expr::Leaf && !is_splat(e) && prod(e->shape) > 1024 && e->cost > 12) {
      // a value computed from the result of the GEMM just emitted is evaluated inside that GEMM's epilogue by each of
      // its consumers that joins it (one evaluation per element there, shared between them) and recomputed by the others
      if (GemmFusion* g = open_fusion()) {
        std::set<const Expr*> seen;
        if (e->shape == std::vector<int64_t>{g->M, g->N} && reads_slot(e, g->d_slot, seen)) return;
      }
      env[v] = materialised(e, "shared value " + m.values[v].name);
    }
  }

  void plan_elementwise(const Op& op) {
    int v = op.out[0];
    shard[v] = join_shard(op, op.in);
    Type t = local_type(v);
    bool scalar_int = t.shape.empty() && (t.dt == DT::S64 || t.dt == DT::S32 || t.dt == DT::U32 || t.dt == DT::U64);
    if (!scalar_int && op.kind != OpK::Compare) check_dt(op, t.dt);
    DT idt = m.values[op.in[0]].type.dt;
    bool fl = dt_is_float(idt);
    std::vector<ExprP> k;
    for (int x : op.in) k.push_back(env[x]);
    ExprP e;
    switch (op.kind) {
      case OpK::Unary: {
        int vop = op.ew;
        if (!fl) {
          if (vop == VM_NEG) vop = VM_INEG;
          else if (vop == VM_ABS) vop = VM_IABS;
          else if (vop == VM_NOT) vop = idt == DT::PRED ? VM_LNOT : VM_NOT;
          else if (vop != VM_MOV && vop != VM_SIGN) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op " + op.name + " on integers");
        }
        e = mkop(vop, t, k);
        break;
      }
      case OpK::Binary: {
        int vop = op.ew;
        if (!fl) {
          switch (vop) {
            case VM_ADD: vop = VM_IADD; break;
            case VM_SUB: vop = VM_ISUB; break;
            case VM_MUL: vop = VM_IMUL; break;
            case VM_DIV: vop = VM_IDIV; break;
            case VM_MAX: vop = idt == DT::PRED ? VM_OR : VM_IMAX; break;
            case VM_MIN: vop = idt == DT::PRED ? VM_AND : VM_IMIN; break;
            case VM_AND: case VM_OR: case VM_XOR: break;
            default: throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op " + op.name + " on integers");
          }
        } else if (vop == VM_AND || vop == VM_OR || vop == VM_XOR) {
          throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op " + op.name + " on floats");
        }
        // m + log(sumexp) where both come from one logsumexp pass: already computed
        if (vop == VM_ADD) {
          for (int sw = 0; sw < 2; ++sw) {
            const ExprP& a = k[sw];
            const ExprP& b = k[1 - sw];
            if (a->k == Expr::Leaf && b->k == Expr::Op && b->vmop == VM_LOG && b->kids[0]->k == Expr::Leaf && whole_slot(a) && whole_slot(b->kids[0])) {
              auto it = lse_of_sum.find(b->kids[0]->slot);
              if (it != lse_of_sum.end() && it->second.m_slot == a->slot) {
                env[v] = leaf(it->second.lse_slot, t);
                return;
              }
            }
          }
        }
        e = mkop(vop, t, k);
        break;
      }
      case OpK::Convert: {
        if (scalar_int) { e = mkop(VM_MOV, t, k); break; }
        check_dt(op, idt);
        // f64 and narrower floats never share a fusion group (a wide program computes every float as a double):
        // a value that is widened is materialised in its own type first and read as an operand, a value that is
        // narrowed is stored (rounded once, which is the conversion) and read back by whatever follows
        const bool from_wide = idt == DT::F64, to_wide = t.dt == DT::F64;
        if (to_wide && !from_wide && dt_is_float(idt)) k[0] = materialised(k[0], "value widened to f64");
        e = mkop(convert_op(idt, t.dt), t, k);
        if (from_wide && !to_wide && dt_is_float(t.dt)) e = materialised(e, "f64 value rounded to " + std::string(dt_name(t.dt)));
        break;
      }
      case OpK::Compare: {
        bool sc = m.values[op.in[0]].type.shape.empty() && !fl;
        if (!sc) check_dt(op, idt);
        e = mkop(fl ? VM_FCMP : VM_ICMP, t, k, op.ew);
        break;
      }
      case OpK::Select: {
        ExprP p = k[0];
        if (p->shape.empty() && !t.shape.empty()) {  // scalar predicate broadcasts
          RMap mp;
          Type pt{DT::PRED, t.shape};
          p = view(p, pt, mp);
        }
        e = mkop(VM_SELECT, t, {p, k[1], k[2]});
        break;
      }
      case OpK::Clamp: {
        bool f = dt_is_float(t.dt);
        auto bc = [&](const ExprP& x) {
          if (x->shape.empty() && !t.shape.empty()) { Type xt{x->dt, t.shape}; return view(x, xt, RMap{}); }
          return x;
        };
        ExprP lo = bc(k[0]), hi = bc(k[2]);
        e = mkop(f ? VM_MIN : VM_IMIN, t, {mkop(f ? VM_MAX : VM_IMAX, t, {k[1], lo}), hi});
        break;
      }
      default: throw Error(RX_ERR_PLAN, "internal: not elementwise");
    }
    env[v] = round_if_bf16(e);
    maybe_spill(v);
  }

  void plan_constant(const Op& op) {
    int v = op.out[0];
    Type t = m.values[v].type;
    if (op.splat) {
      env[v] = konst(t, op.fval, op.ival);
      return;
    }
    int slot = new_slot(t, SlotK::Const);
    plan.slots[slot].init = op.dense;
    env[v] = leaf(slot, t);
  }

  // Operand of a contraction: a strided 2-D (or batched) view of a bf16/f32 slot.
  struct MatView { int slot; int64_t off; std::vector<int64_t> stride; };
  bool as_strided_leaf(const ExprP& e, MatView* mv) {
    Lowering L(e->shape);
    int r = L.lower(e, Lowering::identity(e->shape.size()));
    if (L.nodes[r].leaf < 0 || L.leaves.size() != 1 || L.nodes.size() != 1) return false;
    mv->slot = L.leaves[0].slot;
    mv->off = L.leaves[0].offset;
    mv->stride = L.leaves[0].stride;
    return true;
  }

  void plan_view(const Op& op) {
    int v = op.out[0], x = op.in[0];
    ExprP kid = env[x];
    const Type& gt_in = m.values[x].type;
    RMap mp(gt_in.shape.size());
    switch (op.kind) {
      case OpK::BroadcastInDim:
        if (shard[x] >= 0) shard[v] = (int)op.dims[shard[x]];
        for (size_t d = 0; d < gt_in.shape.size(); ++d) {
          int od = (int)op.dims[d];
          if (gt_in.shape[d] == 1 && m.values[v].type.shape[od] != 1) mp[d] = {-1, 0, 0};
          else mp[d] = {od, 1, 0};
        }
        break;
      case OpK::Transpose:
        for (size_t j = 0; j < op.dims.size(); ++j) {
          mp[op.dims[j]] = {(int)j, 1, 0};
          if (shard[x] == (int)op.dims[j]) shard[v] = (int)j;
        }
        break;
      case OpK::Slice:
        if (shard[x] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.slice of a sharded tensor");
        for (size_t d = 0; d < gt_in.shape.size(); ++d) mp[d] = {(int)d, op.stride[d], op.start[d]};
        break;
      default: break;
    }
    env[v] = simplify(view(kid, local_type(v), mp));
  }

  // A view that merely relabels unit dims of a contiguous leaf is itself a contiguous leaf.
  ExprP simplify(const ExprP& e) {
    if (e->k != Expr::View) return e;
    const Expr* base = e.get();
    while (base->k == Expr::View) base = base->kids[0].get();
    if (base->k != Expr::Leaf) return e;
    MatView mv;
    if (!as_strided_leaf(e, &mv)) return e;
    std::vector<int64_t> cs = canon_strides(e->shape);
    for (size_t d = 0; d < e->shape.size(); ++d)
      if (e->shape[d] != 1 && mv.stride[d] != cs[d]) return e;
    auto l = leaf(mv.slot, Type{e->dt, e->shape});
    l->loffset = mv.off;
    return l;
  }

  void plan_reshape(const Op& op) {
    int v = op.out[0], x = op.in[0];
    if (shard[x] >= 0) {
      // only unit-dim insertion/removal keeps the sharded dim identifiable
      const auto& is = m.values[x].type.shape;
      const auto& os = m.values[v].type.shape;
      int64_t before = 1;
      for (int d = 0; d < shard[x]; ++d) before *= is[d];
      int64_t acc = 1;
      shard[v] = -1;
      for (size_t d = 0; d < os.size(); ++d) {
        if (acc == before && os[d] == is[shard[x]]) { shard[v] = (int)d; break; }
        acc *= os[d];
      }
      if (shard[v] < 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reshape regrouping a sharded dimension");
    }
    Type t = local_type(v);
    ExprP kid = env[x];
    if (kid->k == Expr::Const) { env[v] = konst(t, kid->f, kid->i); return; }
    if (contiguous_leaf(kid)) {
      auto e = leaf(kid->slot, t);
      e->loffset = kid->loffset;
      env[v] = e;
      return;
    }
    // unit-dim insert/remove: a pure index relabelling
    std::vector<int> in_nz, out_nz;
    for (size_t d = 0; d < kid->shape.size(); ++d) if (kid->shape[d] != 1) in_nz.push_back((int)d);
    for (size_t d = 0; d < t.shape.size(); ++d) if (t.shape[d] != 1) out_nz.push_back((int)d);
    bool same = in_nz.size() == out_nz.size();
    for (size_t q = 0; same && q < in_nz.size(); ++q) same = kid->shape[in_nz[q]] == t.shape[out_nz[q]];
    if (same) {
      RMap mp(kid->shape.size(), DimMap{-1, 0, 0});
      for (size_t q = 0; q < in_nz.size(); ++q) mp[in_nz[q]] = {out_nz[q], 1, 0};
      env[v] = view(kid, t, mp);
      return;
    }
    ExprP mat = materialised(kid, "reshape operand " + m.values[x].name);
    if (!contiguous_leaf(mat)) {
      int s = new_slot(Type{mat->dt, mat->shape});
      emit_map(mat, s, 0, canon_strides(mat->shape), "reshape operand " + m.values[x].name);
      mat = leaf(s, Type{mat->dt, mat->shape});
    }
    auto e = leaf(mat->slot, t);
    e->loffset = mat->loffset;
    env[v] = e;
  }

  void plan_iota(const Op& op) {
    int v = op.out[0];
    auto e = std::make_shared<Expr>();
    e->k = Expr::Iota;
    e->dt = m.values[v].type.dt;
    e->shape = m.values[v].type.shape;
    e->iota_dim = (int)op.dims[0];
    e->cost = 1;
    if (e->dt != DT::S32 && e->dt != DT::F32) throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type " + std::string(dt_name(e->dt)) + " in stablehlo.iota");
    env[v] = e;
  }

  void plan_reduce(const Op& op) {
    int v = op.out[0], x = op.in[0];
    ExprP X = env[x], init = env[op.in[1]];
    if (init->k != Expr::Const) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce with a non-constant init value");
    DT dt = X->dt;
    check_dt(op, dt);
    bool needs_allreduce = false;
    if (shard[x] >= 0) {
      bool over = std::find(op.dims.begin(), op.dims.end(), (int64_t)shard[x]) != op.dims.end();
      if (over) {
        if (op.red != RedK::Add) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce (non-additive) over a sharded dimension");
        needs_allreduce = true;
        shard[v] = -1;
      } else {
        int shift = 0;
        for (auto d : op.dims) if (d < shard[x]) ++shift;
        shard[v] = shard[x] - shift;
      }
    }
    Type rt = local_type(v);
    std::vector<int64_t> dims = op.dims;
    std::sort(dims.begin(), dims.end());
    env[v] = reduce_any(op, X, dims, rt, init->f, init->i, needs_allreduce);
  }

  // stablehlo.reduce_window in the cumulative form Reactant's accumulate / cumsum / cumprod emit
  // (src/TracedRArray.jl:1049-1107): the window covers one whole dimension, padded low by its extent minus one,
  // unit strides and dilations -- an inclusive scan along that dimension, combined with the init value.
  // Windows that are not scans (pooling: ext/ReactantNNlibExt/Implementations.jl, src/TracedRArray.jl:981-1047): the
  // result is the combiner applied to one strided view of the (padded) operand per window position,
  //   out[i] = x'[i * stride + k * dilation]  combined over k,
  // so it needs no kernel of its own: the views are leaves of an ordinary fused chain (the strided map kernels read
  // them in place), materialised every few positions to stay inside a chain's operand budget.  Padding is written
  // once, with the combiner's identity.  Positions are combined in row-major window order.
  void plan_general_window(const Op& op) {
    int v = op.out[0], x = op.in[0];
    ExprP X = env[x], init = env[op.in[1]];
    if (shard[x] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window over a sharded tensor (other than a scan along an unsharded dimension)");
    const int rank = (int)X->shape.size();
    const Type t = m.values[v].type;
    const bool flt = dt_is_float(X->dt);
    int64_t volume = 1;
    bool padded = false;
    std::vector<int64_t> pshape = X->shape;
    for (int d = 0; d < rank; ++d) {
      volume *= op.dims[d];
      if (op.start[d] < 0 || op.limit[d] < 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with negative padding");
      padded = padded || op.start[d] || op.limit[d];
      pshape[d] += op.start[d] + op.limit[d];
      // the shape rule of the op, checked because the views below rely on it
      const int64_t span = (op.dims[d] - 1) * op.dilation[d] + 1;
      const int64_t expect = pshape[d] < span ? 0 : (pshape[d] - span) / op.stride[d] + 1;
      if (t.shape[d] != expect) throw Error(RX_ERR_SHAPE, "stablehlo.reduce_window: result extent " + std::to_string(t.shape[d]) + " in dimension " + std::to_string(d) + ", the window gives " + std::to_string(expect));
    }
    if (volume > 64) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with a window of " + std::to_string(volume) + " elements (more than 64) that is not a scan");
    ExprP base;
    if (padded) {
      Type pt{X->dt, pshape};
      const int dst = new_slot(pt);
      const std::vector<int64_t> cs = canon_strides(pshape);
      emit_map(konst(pt, init->f, init->i), dst, 0, cs, "window padding");
      int64_t off = 0;
      for (int d = 0; d < rank; ++d) off += op.start[d] * cs[d];
      emit_map(X, dst, off, cs, "window operand inside its padding");
      base = leaf(dst, pt);
    } else {
      base = materialised(X, "window operand");
    }
    const int vop = flt ? (op.red == RedK::Add ? VM_ADD : op.red == RedK::Max ? VM_MAX : op.red == RedK::Min ? VM_MIN : VM_MUL)
                        : (op.red == RedK::Add ? VM_IADD : op.red == RedK::Max ? VM_IMAX : op.red == RedK::Min ? VM_IMIN : VM_IMUL);
    ExprP acc;
    std::vector<int64_t> k(rank, 0);
    int in_chain = 0;
    for (int64_t pos = 0; pos < volume; ++pos) {
      RMap mp(rank);
      for (int d = 0; d < rank; ++d) mp[d] = {d, op.stride[d], k[d] * op.dilation[d]};
      ExprP piece = simplify(view(base, t, mp));
      acc = acc ? mkop(vop, t, {acc, piece}) : piece;
      if (++in_chain == 6 && pos + 1 < volume) {  // keep every chain within its operand budget
        acc = materialised(acc, "window partial");
        in_chain = 1;
      }
      for (int d = rank - 1; d >= 0; --d) {
        if (++k[d] < op.dims[d]) break;
        k[d] = 0;
      }
    }
    env[v] = acc;
  }

  void plan_reduce_window(const Op& op) {
    int v = op.out[0], x = op.in[0];
    ExprP X = env[x], init = env[op.in[1]];
    if (init->k != Expr::Const) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with a non-constant init value");
    if (X->dt != DT::F32 && X->dt != DT::S32 && X->dt != DT::F64)
      throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type " + std::string(dt_name(X->dt)) + " in " + op.name);
    {
      // the padding is filled with the init value, so anything but the combiner's identity would be counted once
      // per padded position; Reactant passes the identity (src/TracedRArray.jl:1063-1070)
      const bool f = dt_is_float(X->dt);
      bool identity = false;
      switch (op.red) {
        case RedK::Add: identity = f ? init->f == 0.0 : init->i == 0; break;
        case RedK::Mul: identity = f ? init->f == 1.0 : init->i == 1; break;
        case RedK::Max: identity = f ? (std::isinf(init->f) && init->f < 0) : init->i == INT32_MIN; break;
        case RedK::Min: identity = f ? (std::isinf(init->f) && init->f > 0) : init->i == INT32_MAX; break;
        default: break;
      }
      if (!identity) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with an init value that is not the identity of its combiner");
    }
    const int rank = (int)X->shape.size();
    int axis = -1;
    bool cumulative = true;
    for (int d = 0; d < rank; ++d) {
      const bool trivial = op.dims[d] == 1 && op.start[d] == 0 && op.limit[d] == 0 && op.stride[d] == 1;
      if (trivial) continue;
      // the window and padding are written for the global shape
      const int64_t extent = m.values[x].type.shape[d];
      if (axis >= 0 || op.dims[d] != extent || op.start[d] != extent - 1 || op.limit[d] != 0 || op.stride[d] != 1 || op.dilation[d] != 1) cumulative = false;
      axis = d;
    }
    if (!cumulative) {
      plan_general_window(op);
      return;
    }
    if (axis >= 0 && shard[x] == axis) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window scanning along a sharded dimension");
    shard[v] = shard[x];
    Type t = local_type(v);
    const bool flt = dt_is_float(X->dt);
    if (axis < 0) {  // windows of one element: out = x (op) init
      int vop = flt ? (op.red == RedK::Add ? VM_ADD : op.red == RedK::Max ? VM_MAX : op.red == RedK::Min ? VM_MIN : VM_MUL)
                    : (op.red == RedK::Add ? VM_IADD : op.red == RedK::Max ? VM_IMAX : op.red == RedK::Min ? VM_IMIN : VM_IMUL);
      env[v] = mkop(vop, t, {X, konst(t, init->f, init->i)});
      return;
    }
    Step st;
    st.kind = StepK::Scan;
    st.src_slot = materialise(X, "scan operand");
    st.dst_slot = new_slot(t);
    st.red = op.red;
    st.red_dt = X->dt == DT::F64 ? DT::F64 : flt ? DT::F32 : DT::S32;
    st.init_f = init->f;
    st.init_i = init->i;
    st.outer = st.inner = 1;
    for (int d = 0; d < axis; ++d) st.outer *= X->shape[d];
    st.red_n = X->shape[axis];
    for (int d = axis + 1; d < rank; ++d) st.inner *= X->shape[d];
    st.note = std::string("inclusive scan(") + (op.red == RedK::Add ? "add" : op.red == RedK::Max ? "max" : op.red == RedK::Min ? "min" : "mul") + ") over " +
              std::to_string(st.red_n) + " x " + std::to_string(st.outer * st.inner) + " lines";
    plan.scratch_floats = std::max<int64_t>(plan.scratch_floats, 1 << 16);
    const int dst = st.dst_slot;
    cur->push_back(std::move(st));
    env[v] = leaf(dst, t);
  }

  // One step when the reduced dims form a single run of the (normalised) iteration space and the kept dims on
  // either side merge.  Otherwise (a) several reduced dims: reduce the innermost one on its own, with the
  // operation's identity as init, and go on with the rest -- valid for every supported combiner (associative and
  // commutative), each stage a streaming pass; (b) one reduced dim whose neighbours do not merge (a broadcast
  // operand along one of them): evaluate the chain into a dense temporary first, then reduce that.
  ExprP reduce_any(const Op& op, ExprP X, std::vector<int64_t> dims, const Type& rt, double init_f, int64_t init_i, bool needs_allreduce) {
    const size_t n_slots = plan.slots.size(), n_steps = cur->size();
    try {
      return reduce_core(op, X, dims, rt, init_f, init_i, needs_allreduce);
    } catch (const Error& e) {
      if (e.code != RX_ERR_PLAN) throw;
      plan.slots.resize(n_slots);
      cur->resize(n_steps);
      last_map.where = nullptr;
      if (dims.size() < 2 && whole_slot(X)) throw;
    }
    if (dims.size() < 2) {
      Type xt{X->dt, X->shape};
      return reduce_core(op, leaf(materialise(X, "reduce operand (kept dims do not merge)"), xt), dims, rt, init_f, init_i, needs_allreduce);
    }
    const int64_t d = dims.back();
    dims.pop_back();
    Type mid{X->dt, X->shape};
    mid.shape.erase(mid.shape.begin() + d);
    double idf = 0;
    int64_t idi = 0;
    switch (op.red) {
      case RedK::Add: case RedK::Or: break;
      case RedK::Max: idf = -INFINITY; idi = INT32_MIN; break;
      case RedK::Min: idf = INFINITY; idi = INT32_MAX; break;
      case RedK::Mul: case RedK::And: idf = 1; idi = 1; break;
    }
    ExprP M = reduce_any(op, X, {d}, mid, idf, idi, false);
    return reduce_any(op, M, dims, rt, init_f, init_i, needs_allreduce);
  }

  // chain X -> reduce over `dims` -> a fresh slot of type rt; returns the result as a leaf
  ExprP reduce_core(const Op& op, ExprP X, const std::vector<int64_t>& dims, const Type& rt, double init_f, int64_t init_i, bool needs_allreduce) {
    if (op.red == RedK::Add) {
      const bool late = needs_allreduce && init_f != 0.0;
      const int fused = try_fuse_sum(X, dims, rt, late ? 0.0 : init_f);
      if (fused >= 0) {
        if (needs_allreduce) emit_allreduce(fused, rt);
        if (late) emit_late_init(fused, rt, init_f);
        return leaf(fused, rt);
      }
    }
    const DT dt = X->dt;
    std::vector<int> cls(X->shape.size(), 0);
    for (auto d : dims) cls[d] = 1;
    // output strides over root dims: kept dims in order
    std::vector<int64_t> ostr(X->shape.size(), 0);
    {
      int64_t acc = 1;
      for (int d = (int)X->shape.size() - 1; d >= 0; --d)
        if (!cls[d]) { ostr[d] = acc; acc *= X->shape[d]; }
    }
    int slot = new_slot(rt);
    Step st;
    st.red = op.red;
    st.red_dt = (dt == DT::S32) ? DT::S32 : (dt == DT::PRED ? DT::PRED : dt == DT::F64 ? DT::F64 : DT::F32);
    if (dt == DT::PRED && op.red == RedK::Add) st.red = RedK::Or;  // i1 addition saturates
    // A reduce over the sharded dim is summed over the mesh afterwards: every device folding the init value into
    // its local result would count it once per device, so the local reduce starts from the identity and the init
    // value is added once, after the all-reduce.
    const bool late_init = needs_allreduce && (init_f != 0.0 || init_i != 0);
    st.init_f = late_init ? 0.0 : init_f;
    st.init_i = late_init ? 0 : init_i;
    Lowering L(X->shape);
    int root = L.lower(X, Lowering::identity(X->shape.size()));
    OutSpec os{slot, rt.dt, 0, ostr, root};
    assemble(st, L, {os}, root, cls, false);
    // shape of the collapsed space
    const VmProgram& P = st.prog;
    std::vector<int> c = cls_after;
    int nred = (int)std::count(c.begin(), c.end(), 1);
    int64_t red_n = 1, kept_n = 1;
    for (int d = 0; d < P.rank; ++d) (c[d] ? red_n : kept_n) *= P.dim[d];
    st.red_n = red_n;
    std::ostringstream note;
    note << "reduce(" << (op.red == RedK::Add ? "add" : op.red == RedK::Max ? "max" : op.red == RedK::Min ? "min" : op.red == RedK::Mul ? "mul" : op.red == RedK::Or ? "or" : "and") << ")";
    if (nred == 0) {
      // only unit dims are reduced: out = x (op) init, a plain map
      int vop = dt_is_float(st.red_dt) ? (op.red == RedK::Add ? VM_ADD : op.red == RedK::Max ? VM_MAX : op.red == RedK::Min ? VM_MIN : VM_MUL)
                                     : (st.red == RedK::Add ? VM_IADD : st.red == RedK::Max ? VM_IMAX : st.red == RedK::Min ? VM_IMIN : st.red == RedK::Mul ? VM_IMUL : st.red == RedK::Or ? VM_OR : VM_AND);
      Type xt{X->dt, X->shape};
      ExprP e = late_init ? X : round_if_bf16(mkop(vop, xt, {X, konst(xt, init_f, init_i)}));
      emit_map(e, slot, 0, ostr, "reduce over unit dimensions");
      // a sharded dim whose local extent is one still has to be summed over the mesh
      if (needs_allreduce) emit_allreduce(slot, rt);
      if (late_init) emit_late_init(slot, rt, init_f);
      return leaf(slot, rt);
    } else if (kept_n == 1) {
      st.kind = StepK::ReduceFull;
      if (P.rank != 1 && !(P.rank == 0)) {
        // several reduced dims that could not be merged: index generically
      }
    } else {
      to_outer_red_inner(st, c);
      // the reduced run is contiguous in memory for the dominant operand iff it is the innermost dim
      st.kind = st.inner == 1 ? StepK::ReduceRow : StepK::ReduceCol;
    }
    st.note = note.str() + " over " + std::to_string(st.red_n) + " of " + std::to_string(kept_n * red_n) + " elements";
    plan.scratch_floats = std::max<int64_t>(plan.scratch_floats, 1 << 16);

    // logsumexp: this is sum(exp(x - max(x))) with the max produced by an earlier row reduce of the same x
    if (op.red == RedK::Add && st.kind == StepK::ReduceRow && st.prog.fast_id == FAST_EXP_SUB && try_logsumexp(st, slot)) {
      return leaf(slot, rt);
    }
    cur->push_back(std::move(st));
    if (needs_allreduce) emit_allreduce(slot, rt);
    if (late_init) emit_late_init(slot, rt, init_f);
    return leaf(slot, rt);
  }
  // slot += init, element for element, in place (the all-reduced result of a reduce whose init is not zero)
  void emit_late_init(int slot, const Type& rt, double init_f) {
    last_map.where = nullptr;  // must stay behind the all-reduce: never merged into an earlier map
    emit_map(mkop(VM_ADD, rt, {leaf(slot, rt), konst(rt, init_f, 0)}), slot, 0, canon_strides(rt.shape), "init value added once, after the all-reduce");
    last_map.where = nullptr;
  }
  void emit_allreduce(int slot, const Type& rt) {
    Step ar;
    ar.kind = StepK::AllReduce;
    ar.dst_slot = slot;
    ar.count = rt.numel();
    ar.red_dt = rt.dt;
    ar.note = "all_reduce(sum) over the mesh axis";
    if (rt.dt != DT::F32) throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type for all_reduce");
    cur->push_back(std::move(ar));
  }

  // Rewrite prog dims/strides into exactly three dims [outer][red][inner].
  void to_outer_red_inner(Step& st, const std::vector<int>& c) {
    VmProgram& P = st.prog;
    size_t a = 0;
    while (a < c.size() && c[a] == 0) ++a;
    size_t b = a;
    while (b < c.size() && c[b] == 1) ++b;
    if (a > 1 || b - a > 1 || c.size() - b > 1)
      throw Error(RX_ERR_PLAN, "reduction over a strided group of dimensions is not supported");
    int64_t dim[3] = {1, 1, 1};
    int map3[3] = {-1, -1, -1};
    if (a == 1) { dim[0] = P.dim[0]; map3[0] = 0; }
    if (b - a == 1) { dim[1] = P.dim[a]; map3[1] = (int)a; }
    if (c.size() - b == 1) { dim[2] = P.dim[b]; map3[2] = (int)b; }
    auto remap = [&](int64_t* s) {
      int64_t o[kMaxRank] = {0, 0, 0, 0};
      for (int q = 0; q < 3; ++q) o[q] = map3[q] >= 0 ? s[map3[q]] : 0;
      for (int q = 0; q < kMaxRank; ++q) s[q] = o[q];
    };
    for (int k = 0; k < P.n_leaves; ++k) remap(P.leaf[k].stride);
    for (int k = 0; k < P.n_outs; ++k) remap(P.out[k].stride);
    for (int k = 0; k < P.n_instr; ++k)
      if (P.ins[k].op == VM_IOTA) {
        int nd = -1;
        for (int q = 0; q < 3; ++q) if (map3[q] == P.ins[k].a) nd = q;
        P.ins[k].a = (uint8_t)(nd < 0 ? 0 : nd);
      }
    P.rank = 3;
    P.dim[0] = st.outer = dim[0];
    P.dim[1] = st.red_n = dim[1];
    P.dim[2] = st.inner = dim[2];
    P.dim[3] = 1;
  }

  bool try_logsumexp(Step& sum_step, int sum_slot) {
    const VmProgram& S = sum_step.prog;
    // leaf 0 = x rows (contiguous along the reduced dim), leaf 1 = per-row max (broadcast along it)
    if (S.leaf[0].stride[1] != 1 || S.leaf[1].stride[1] != 0 || S.leaf[0].elem != EL_F32 || S.leaf[1].elem != EL_F32) return false;
    if (sum_step.init_f != 0.0) return false;
    int m_slot = sum_step.leaf_slot[1];
    for (size_t q = 0; q < cur->size(); ++q) {
      Step& mx = (*cur)[q];
      if (mx.kind != StepK::ReduceRow || mx.red != RedK::Max || mx.out_slot.size() != 1 || mx.out_slot[0] != m_slot) continue;
      if (mx.prog.fast_id != FAST_IDENTITY || mx.leaf_slot[0] != sum_step.leaf_slot[0]) return false;
      const VmLeaf& a = mx.prog.leaf[0];
      const VmLeaf& b = S.leaf[0];
      if (a.offset != b.offset || a.stride[0] != b.stride[0] || a.stride[1] != b.stride[1]) return false;
      if (mx.outer != sum_step.outer || mx.red_n != sum_step.red_n) return false;
      if (!(std::isinf(mx.init_f) && mx.init_f < 0)) return false;
      // max rows must be laid out like the sum rows
      if (mx.prog.out[0].stride[0] != S.out[0].stride[0] || S.leaf[1].stride[0] != mx.prog.out[0].stride[0] || S.leaf[1].offset != 0) return false;
      Step lse;
      lse.kind = StepK::LogSumExp;
      lse.prog = mx.prog;
      lse.leaf_slot = mx.leaf_slot;
      int lse_slot = new_slot(plan.slots[sum_slot].type);
      lse.out_slot = {m_slot, sum_slot, lse_slot};
      lse.outer = mx.outer;
      lse.red_n = mx.red_n;
      lse.inner = 1;
      lse.note = "logsumexp rows=" + std::to_string(lse.outer) + " cols=" + std::to_string(lse.red_n) + " (max, sum(exp(x-max)), max+log(sum) in one read)";
      (*cur)[q] = std::move(lse);
      lse_of_sum[sum_slot] = {m_slot, lse_slot};
      return true;
    }
    return false;
  }

  int loop_depth = 0;

  // stablehlo.dynamic_slice (src/Ops.jl:3680-3696; scalar indexing `a[i]` with a traced index, src/Indexing.jl:25-31).
  // Constant start indices make it a slice.  Start indices that are affine in the counter of the enclosing counted
  // loop (`fict[t]` in benchmark/polybench/stencil.jl:49) become a DynSlice step: the host knows the iteration it is
  // enqueueing, so the slice is a small device-to-device copy from a computed offset into a temporary, and everything
  // downstream sees an ordinary array.  The slice must be contiguous in the operand (a scalar, a row, whole trailing
  // dims); anything else is refused by name.
  void plan_dynamic_slice(const Op& op) {
    int v = op.out[0], x = op.in[0];
    if (shard[x] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_slice of a sharded tensor");
    const Type& tin = m.values[x].type;
    const Type t = m.values[v].type;
    const int rank = (int)tin.shape.size();
    if ((int)op.in.size() != 1 + rank || (int)op.dims.size() != rank) throw Error(RX_ERR_PARSE, "stablehlo.dynamic_slice: start indices or sizes do not match the operand rank");
    std::vector<int64_t> a(rank), b(rank);
    int depth = 0;
    for (int d = 0; d < rank; ++d) {
      int dd = 0;
      if (!affine_int(env[op.in[1 + d]], &a[d], &b[d], &dd))
        throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_slice with a start index that is not affine in a loop counter");
      if (dd && depth && dd != depth) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_slice indexed by the counters of two loops");
      if (dd) depth = dd;
      if (op.dims[d] < 0 || op.dims[d] > tin.shape[d]) throw Error(RX_ERR_SHAPE, "stablehlo.dynamic_slice: slice size exceeds the operand");
    }
    if (depth == 0) {  // all constant: an ordinary slice, clamped as the op specifies
      RMap mp(rank);
      for (int d = 0; d < rank; ++d) mp[d] = {d, 1, std::max<int64_t>(0, std::min<int64_t>(b[d], tin.shape[d] - op.dims[d]))};
      env[v] = simplify(view(env[x], t, mp));
      return;
    }
    if (depth != loop_depth) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_slice indexed by the counter of an outer loop");
    // contiguous: sizes are 1 up to some dim, then one partial dim, then whole dims
    int first = 0;
    while (first < rank && op.dims[first] == 1) ++first;
    for (int d = first + 1; d < rank; ++d)
      if (op.dims[d] != tin.shape[d]) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_slice with loop-variant start indices whose slice is not contiguous in the operand");
    check_dt(op, t.dt);
    Step st;
    st.kind = StepK::DynSlice;
    st.src_slot = materialise(env[x], "dynamic_slice operand");
    st.dst_slot = new_slot(t);
    st.dyn_elem_bytes = (int64_t)dt_size(t.dt);
    st.bytes = t.numel() * st.dyn_elem_bytes;
    const std::vector<int64_t> cs = canon_strides(tin.shape);
    for (int d = 0; d < rank; ++d) {
      st.dyn_a.push_back(a[d]);
      st.dyn_b.push_back(b[d]);
      st.dyn_hi.push_back(tin.shape[d] - op.dims[d]);
      st.dyn_stride.push_back(cs[d]);
    }
    st.note = "dynamic slice at an offset that follows the loop counter (" + std::to_string(st.bytes) + " bytes per iteration)";
    const int dst = st.dst_slot;
    cur->push_back(std::move(st));
    env[v] = leaf(dst, t);
  }

  void plan_dus(const Op& op) {
    int v = op.out[0], o = op.in[0], u = op.in[1];
    for (int x : op.in) if (shard[x] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_update_slice of a sharded tensor");
    ExprP U = env[u];
    Type t = m.values[v].type;
    std::vector<int64_t> starts;
    for (size_t k = 2; k < op.in.size(); ++k) {
      int64_t s;
      if (!const_int(env[op.in[k]], &s)) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dynamic_update_slice with non-constant start indices");
      int d = (int)k - 2;
      s = std::max<int64_t>(0, std::min<int64_t>(s, t.shape[d] - U->shape[d]));  // clamped, as the op specifies
      starts.push_back(s);
    }
    plan_update_window(op, v, env[o], U, starts);
  }

  // value v = the array O with the window at `starts` replaced by U (`op` is the op being planned: a
  // dynamic_update_slice, or the select of the pad + select spelling)
  void plan_update_window(const Op& op, int v, ExprP O, ExprP U, const std::vector<int64_t>& starts) {
    Type t = m.values[v].type;
    int dst = -1;
    // In place when nothing that is still to be evaluated reads the target's storage: the target itself has no later
    // use, and every expression that looked at it (the slices of the previous half-step, say) has already been
    // turned into a step that runs before this one.
    bool in_place = whole_slot(O) && slot_writable(O->slot) && !read_later(O->slot, op);
    std::vector<int64_t> cs = canon_strides(t.shape);
    int64_t off = 0;
    for (size_t d = 0; d < starts.size(); ++d) off += starts[d] * cs[d];
    if (in_place) {
      // the update may read the destination only at the very position it writes (A[w] = A[w] - ..., the in-place
      // field updates of fdtd_2d, benchmark/polybench/stencil.jl:52-66): every element then depends on its own old
      // value only, whatever order the kernel takes them in
      Lowering L(U->shape);
      L.lower(U, Lowering::identity(U->shape.size()));
      for (auto& lf : L.leaves) {
        if (lf.slot != O->slot) continue;
        bool same = lf.offset == off;
        for (size_t d = 0; d < cs.size() && same; ++d)
          if (U->shape[d] != 1 && lf.stride[d] != cs[d]) same = false;
        if (!same) in_place = false;
      }
    }
    if (in_place) {
      dst = O->slot;
    } else {
      dst = new_slot(t);
      if (O->k == Expr::Leaf && whole_slot(O)) {
        Step cp;
        cp.kind = StepK::Copy;
        cp.src_slot = O->slot;
        cp.dst_slot = dst;
        cp.bytes = plan.slots[dst].bytes();
        cp.note = "copy (update target still live)";
        cur->push_back(std::move(cp));
      } else {
        emit_map(O, dst, 0, canon_strides(t.shape), "materialise update target");
      }
    }
    emit_map(U, dst, off, cs, "update window at offset " + std::to_string(off));
    env[v] = leaf(dst, t);
  }

  void plan_pad(const Op& op) {
    int v = op.out[0];
    if (shard[op.in[0]] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.pad of a sharded tensor");
    for (auto i : op.stride) if (i != 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.pad with interior padding");
    for (auto i : op.start) if (i < 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.pad with negative padding");
    for (auto i : op.limit) if (i < 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.pad with negative padding");
    ExprP X = env[op.in[0]], pv = env[op.in[1]];
    if (pv->k != Expr::Const) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.pad with a non-constant padding value");
    Type t = m.values[v].type;
    check_dt(op, t.dt);
    {
      // `true` padded with `false`: the mask of a window (see plan_masked_update)
      int64_t inside = 0, outside = 1;
      if (t.dt == DT::PRED && const_int(X, &inside) && inside != 0 && const_int(pv, &outside) && outside == 0) window_mask[v] = {op.start, op.limit};
    }
    if (const Op* sel = sole_user_if(v, OpK::Select)) {
      auto it = window_mask.find(sel->in[0]);
      if (sel->in[1] == v && sel->in[2] != v && sel->in[0] != v && it != window_mask.end() && it->second.first == op.start && it->second.second == op.limit &&
          shard[sel->in[2]] < 0) {
        deferred_pad[v] = &op;
        for (int x : op.in) ++remaining[x];  // still needed: consumed when the select is planned
        return;
      }
    }
    int dst = new_slot(t);
    emit_map(konst(t, pv->f, pv->i), dst, 0, canon_strides(t.shape), "pad fill");
    std::vector<int64_t> cs = canon_strides(t.shape);
    int64_t off = 0;
    for (size_t d = 0; d < op.start.size(); ++d) off += op.start[d] * cs[d];
    emit_map(X, dst, off, cs, "pad interior");
    env[v] = leaf(dst, t);
  }

  // ---- concatenate --------------------------------------------------------------------------------------------
  // Reactant's pad / communication patterns may rewrite a dynamic_update_slice into concatenates of the untouched
  // borders of the target around the update (src/CompileOptions.jl:22-41, OptimizationPasses.jl:356-372), usually
  // nested: columns first, then rows.  A concatenate whose only user is another concatenate is not materialised;
  // the outer one places all pieces at their N-d offsets.  Pieces that are the target's own contents at the position
  // they already occupy are not copied: when every such piece comes from one writable array that nothing reads
  // later, the rest is written into that array in place -- the same plan the dynamic_update_slice form gets.
  struct ConcatPiece { ExprP e; std::vector<int64_t> at; };
  std::map<int, const Op*> deferred_concat;
  const Region* cur_region = nullptr;

  const Op* sole_user_if(int v, OpK kind) const {
    if (uses[v] != 1 || !cur_region) return nullptr;
    for (auto& op : cur_region->ops)
      for (int x : op.in)
        if (x == v) return op.kind == kind ? &op : nullptr;
    return nullptr;  // a result of the region, or used inside a nested one
  }
  const Op* sole_user_if_concat(int v) const { return sole_user_if(v, OpK::Concatenate); }

  // ---- pad + select ---------------------------------------------------------------------------------------------
  // The other spelling the communication patterns leave of a dynamic_update_slice (src/compiler/OptimizationPasses.jl:
  // 356-372): select(mask, pad(update), target), where mask is `true` padded with `false` by the same amounts (a
  // constant, usually hoisted out of the loop).  The padded update is not materialised; the select is planned as the
  // window update it is, in place under the same conditions as a dynamic_update_slice.
  std::map<int, std::pair<std::vector<int64_t>, std::vector<int64_t>>> window_mask;  // value -> (low, high) padding
  std::map<int, const Op*> deferred_pad;

  bool plan_masked_update(const Op& op) {
    auto it = deferred_pad.find(op.in[1]);
    if (it == deferred_pad.end()) return false;
    const Op* pad = it->second;
    deferred_pad.erase(it);
    plan_update_window(op, op.out[0], env[op.in[2]], env[pad->in[0]], pad->start);
    for (int x : pad->in) --remaining[x];
    return true;
  }
  void concat_pieces(const Op& op, const std::vector<int64_t>& base, std::vector<ConcatPiece>& out, std::vector<const Op*>& inner) {
    const int d = (int)op.dims[0];
    int64_t pos = 0;
    for (int x : op.in) {
      std::vector<int64_t> at = base;
      at[d] += pos;
      auto it = deferred_concat.find(x);
      if (it != deferred_concat.end()) {
        inner.push_back(it->second);
        concat_pieces(*it->second, at, out, inner);
      } else {
        out.push_back({env[x], at});
      }
      pos += m.values[x].type.shape[d];
    }
  }

  void plan_concat(const Op& op) {
    int v = op.out[0];
    Type t = m.values[v].type;
    check_dt(op, t.dt);
    for (int x : op.in)
      if (shard[x] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.concatenate of a sharded tensor");
    if (sole_user_if_concat(v)) {
      deferred_concat[v] = &op;
      for (int x : op.in) ++remaining[x];  // still needed: consumed when the outer concatenate is planned
      return;
    }
    std::vector<ConcatPiece> pieces;
    std::vector<const Op*> inner;
    concat_pieces(op, std::vector<int64_t>(t.shape.size(), 0), pieces, inner);
    const std::vector<int64_t> cs = canon_strides(t.shape);
    auto offset_of = [&](const ConcatPiece& p) {
      int64_t off = 0;
      for (size_t d = 0; d < cs.size(); ++d) off += p.at[d] * cs[d];
      return off;
    };
    // which pieces already sit where they belong, and in which array
    int target = -1;
    std::vector<bool> in_place_piece(pieces.size(), false);
    for (size_t k = 0; k < pieces.size(); ++k) {
      MatView mv;
      if (!as_strided_leaf(pieces[k].e, &mv)) continue;
      if (target >= 0 && mv.slot != target) continue;
      const Slot& sl = plan.slots[mv.slot];
      if (sl.type.dt != t.dt || sl.type.shape != t.shape || mv.off != offset_of(pieces[k])) continue;
      bool same_layout = true;
      for (size_t d = 0; d < cs.size(); ++d)
        if (pieces[k].e->shape[d] != 1 && mv.stride[d] != cs[d]) same_layout = false;
      if (!same_layout) continue;
      target = mv.slot;
      in_place_piece[k] = true;
    }
    bool in_place = target >= 0 && slot_writable(target);
    if (in_place) {
      // nothing still to be evaluated may read the target, apart from the operands consumed here
      std::vector<int> consumed(op.in.begin(), op.in.end());
      for (const Op* q : inner) consumed.insert(consumed.end(), q->in.begin(), q->in.end());
      for (size_t w = 0; w < env.size() && in_place; ++w) {
        if (!env[w]) continue;
        int left = remaining[w] - (int)std::count(consumed.begin(), consumed.end(), (int)w);
        if (left <= 0) continue;
        std::set<const Expr*> seen;
        if (reads_slot(env[w], target, seen)) in_place = false;
      }
      // and the pieces that are written may not read it at all (they would see rows already replaced)
      for (size_t k = 0; k < pieces.size() && in_place; ++k) {
        if (in_place_piece[k]) continue;
        std::vector<const Expr*> lv;
        std::set<const Expr*> seen;
        collect_leaves(pieces[k].e, lv, seen);
        for (auto* l : lv)
          if (l->slot == target) in_place = false;
      }
    }
    int dst = in_place ? target : new_slot(t);
    for (size_t k = 0; k < pieces.size(); ++k) {
      if (in_place && in_place_piece[k]) continue;
      emit_map(pieces[k].e, dst, offset_of(pieces[k]), cs, in_place ? "concatenate piece, written in place" : "concatenate piece");
    }
    for (const Op* q : inner) {
      for (int x : q->in) --remaining[x];
      deferred_concat.erase(q->out[0]);
    }
    env[v] = leaf(dst, t);
  }

  void plan_dot(const Op& op) {
    int v = op.out[0], a = op.in[0], b = op.in[1];
    ExprP A = env[a], B = env[b];
    // SPMD rule for contractions on a 1-D mesh: a sharded free dimension stays sharded in the result;
    // a contraction over a dimension sharded in both operands gives per-device partial products that
    // are summed with an all-reduce; anything else is not expressible without resharding.
    bool partial_sum = false;
    shard[v] = -1;
    if (shard[a] >= 0 || shard[b] >= 0) {
      if (op.lcontract.size() != 1 || !op.lbatch.empty()) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general: sharded batched contraction");
      int lc0 = (int)op.lcontract[0], rc0 = (int)op.rcontract[0];
      bool a_c = shard[a] == lc0, b_c = shard[b] == rc0;
      if (a_c && b_c) partial_sum = true;
      else if (a_c || b_c) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general: contraction dimension sharded in only one operand");
      else if (shard[a] >= 0 && shard[b] >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general: both operands sharded along free dimensions");
      else if (shard[a] >= 0) shard[v] = 0;                                  // result dims are (lhs free, rhs free)
      else shard[v] = (int)A->shape.size() - 1;
    }
    Type rt = local_type(v);
    if (!(A->dt == B->dt && (A->dt == DT::BF16 || A->dt == DT::F32 || (A->dt == DT::F64 && rt.dt == DT::F64))))
      throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element types for stablehlo.dot_general: " + std::string(dt_name(A->dt)) + " x " + dt_name(B->dt));
    if (op.lcontract.size() != 1 || op.lbatch.size() > 1)
      throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general with several contracting or batching dimensions");
    size_t nb = op.lbatch.size();
    if (A->shape.size() != 2 + nb || B->shape.size() != 2 + nb)
      throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general on operands that are not (batched) matrices");
    MatView av, bv;
    auto get = [&](int val, MatView* mv, const char* why) {
      if (as_strided_leaf(env[val], mv)) return;
      ExprP mat = materialised(env[val], why);
      if (!as_strided_leaf(mat, mv)) throw Error(RX_ERR_PLAN, "internal: materialised operand is not a leaf");
      env[val] = mat;  // later consumers read the materialised copy
    };
    get(a, &av, "contraction lhs");
    get(b, &bv, "contraction rhs");
    int lc = (int)op.lcontract[0], rc = (int)op.rcontract[0];
    int lb = nb ? (int)op.lbatch[0] : -1, rb = nb ? (int)op.rbatch[0] : -1;
    int lf = -1, rf = -1;
    for (int d = 0; d < (int)A->shape.size(); ++d) if (d != lc && d != lb) lf = d;
    for (int d = 0; d < (int)B->shape.size(); ++d) if (d != rc && d != rb) rf = d;
    Step st;
    st.kind = StepK::Gemm;
    GemmDesc& g = st.gemm;
    g.M = A->shape[lf];
    g.K = A->shape[lc];
    g.N = B->shape[rf];
    if (B->shape[rc] != g.K) throw Error(RX_ERR_SHAPE, "stablehlo.dot_general: contracting dimensions differ");
    g.batch = nb ? A->shape[lb] : 1;
    g.a_slot = av.slot;
    g.b_slot = bv.slot;
    g.a_sm = av.stride[lf];
    g.a_sk = av.stride[lc];
    g.b_sk = bv.stride[rc];
    g.b_sn = bv.stride[rf];
    g.a_sb = nb ? av.stride[lb] : 0;
    g.b_sb = nb ? bv.stride[rb] : 0;
    g.in_dt = A->dt;
    g.out_dt = rt.dt;
    g.a_off = av.off;
    g.b_off = bv.off;
    int dst = new_slot(rt);
    g.d_slot = dst;
    g.d_sb = g.M * g.N;
    st.leaf_slot = {av.slot, bv.slot};
    st.out_slot = {dst};
    std::ostringstream note;
    note << "gemm M=" << g.M << " N=" << g.N << " K=" << g.K << (g.batch > 1 ? " batch=" + std::to_string(g.batch) : "")
         << " A(" << (g.a_sk == 1 ? "k-major" : "m-major") << ") B(" << (g.b_sk == 1 ? "k-major" : "n-major") << ") "
         << dt_name(g.in_dt) << "->" << dt_name(g.out_dt) << (g.in_dt == DT::F64 ? " fp64 accumulate" : " fp32 accumulate");
    st.note = note.str();
    // can elementwise work on the product join this step?  (what the two-CTA tensor-core kernel with a compiled epilogue takes)
    const bool majors_ok = (g.a_sk == 1 || g.a_sm == 1) && (g.b_sk == 1 || g.b_sn == 1);
    const int64_t a_pitch = g.a_sk == 1 ? g.a_sm : g.a_sk, b_pitch = g.b_sk == 1 ? g.b_sn : g.b_sk;
    const bool fusable = !partial_sum && cur == &plan.steps && epilogue_enabled() && g.in_dt == DT::BF16 && (g.out_dt == DT::BF16 || g.out_dt == DT::F32) &&
                         g.batch == 1 && g.M >= 256 && g.N >= 256 && g.M % 32 == 0 && g.N % 32 == 0 && g.K >= 1 && majors_ok && a_pitch > 0 && b_pitch > 0 &&
                         a_pitch % 8 == 0 && b_pitch % 8 == 0 && av.off % 8 == 0 && bv.off % 8 == 0 && g.M < (1LL << 31) && g.N < (1LL << 31) && g.K < (1LL << 31);
    fusion_open = false;
    if (fusable) {
      GemmFusion gf;
      gf.where = cur;
      gf.index = cur->size();
      gf.d_slot = dst;
      gf.dt = rt.dt;
      gf.M = g.M;
      gf.N = g.N;
      gf.base_note = st.note;
      fusions.push_back(std::move(gf));
      fusion_open = true;
    }
    cur->push_back(std::move(st));
    if (partial_sum) {
      if (rt.dt != DT::F32 && rt.dt != DT::BF16) throw Error(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type for all_reduce");
      Step ar;
      ar.kind = StepK::AllReduce;
      ar.dst_slot = dst;
      ar.count = rt.numel();
      ar.red_dt = rt.dt;
      ar.note = "all_reduce(sum) of per-device partial products";
      cur->push_back(std::move(ar));
    }
    env[v] = leaf(dst, rt);
  }

  void plan_while(const Op& op) {
    size_t n = op.in.size();
    for (int v : op.in) --remaining[v];  // the operands are consumed on entry: the loop's storage takes their place
    const Region& cond = op.regions[0];
    const Region& body = op.regions[1];
    // Carried arrays split into row blocks over the mesh (tensor dim 0 of 2-D f32 arrays): accepted when the body turns
    // out to be slice-and-add (stencil) updates only -- what XLA's partitioner turns into collective-permutes of the
    // boundary rows (test/core/sharding/optimize_comm.jl:48-56).  The body is then planned on the global arrays.
    bool row_sharded = false;
    for (int x : op.in) {
      if (shard[x] < 0) continue;
      const Type& t = m.values[x].type;
      if (shard[x] != 0 || t.shape.size() != 2 || t.dt != DT::F32 || cur != &plan.steps)
        throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while carrying sharded tensors other than 2-D f32 arrays split along their first tensor dimension");
      row_sharded = true;
    }
    // ---- trip count: cond is `compare LT|LE, counter, bound`, body steps counter by a constant
    int64_t trip = -1;
    int counter = -1;
    int64_t counter_init = 0, counter_step = 0;
    {
      if (cond.ops.empty() || cond.yields.size() != 1) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: condition is not a comparison");
      // bind cond args symbolically
      for (size_t k = 0; k < n; ++k) {
        auto s = std::make_shared<Expr>();
        s->k = Expr::Sym;
        s->dt = m.values[cond.args[k]].type.dt;
        s->shape = m.values[cond.args[k]].type.shape;
        s->slot = (int)k;
        env[cond.args[k]] = s;
      }
      const Op* cmp = nullptr;
      for (auto& c : cond.ops) {
        if (c.kind == OpK::Constant) plan_constant(c);
        else if (c.kind == OpK::Compare && c.out[0] == cond.yields[0]) cmp = &c;
        else throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: condition contains " + c.name);
      }
      if (!cmp) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: condition is not a comparison");
      ExprP l = env[cmp->in[0]], r = env[cmp->in[1]];
      int64_t bound;
      if (l->k != Expr::Sym || !const_int(r, &bound) || (cmp->ew != CMP_LT && cmp->ew != CMP_LE))
        throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: only `counter < constant` loops are supported");
      counter = l->slot;
      int64_t init;
      if (!const_int(env[op.in[counter]], &init)) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: counter does not start at a constant");
      // step: body yield of counter = counter + c
      int yv = body.yields[counter];
      int64_t step = 0;
      for (auto& bo : body.ops)
        if (bo.out.size() == 1 && bo.out[0] == yv && bo.kind == OpK::Binary && bo.ew == VM_ADD) {
          for (int sw = 0; sw < 2; ++sw)
            if (bo.in[sw] == body.args[counter]) {
              // the other operand must be constant: look it up among constants defined so far or in the body
              int other = bo.in[1 - sw];
              if (env[other] && const_int(env[other], &step)) {}
              else
                for (auto& bc : body.ops)
                  if (bc.kind == OpK::Constant && bc.out[0] == other && bc.splat) step = bc.ival;
            }
        }
      if (step <= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: counter is not advanced by a positive constant");
      if (cmp->ew == CMP_LE) bound += 1;
      trip = bound <= init ? 0 : (bound - init + step - 1) / step;
      counter_init = init;
      counter_step = step;
    }
    // ---- loop-carried tensors live in slots
    Step loop;
    loop.kind = StepK::Loop;
    loop.trip = trip;
    std::vector<int> state_slot(n, -1);
    for (size_t k = 0; k < n; ++k) {
      if ((int)k == counter) continue;
      int x = op.in[k];
      Type t = m.values[x].type;
      ExprP e = env[x];
      if (t.shape.empty() && !dt_is_float(t.dt)) continue;  // integer scalar bookkeeping stays symbolic
      if (row_sharded) {
        if (shard[x] != 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: a row-sharded loop carries a tensor that is not sharded the same way");
        int s = new_slot(t);  // the global type; allocated per device as its row block plus halos
        plan.slots[s].row_block = true;
        Step in;
        in.kind = StepK::RowsIn;
        in.src_slot = materialise(e, "row block of a loop-carried array");
        in.dst_slot = s;
        in.note = "row block + neighbours' halo rows into loop storage";
        cur->push_back(std::move(in));
        state_slot[k] = s;
        continue;
      }
      bool reuse = whole_slot(e) && uses[x] == 1 && slot_writable(e->slot);
      if (reuse) {
        state_slot[k] = e->slot;
      } else {
        int s = new_slot(t);
        if (whole_slot(e)) {
          Step cp;
          cp.kind = StepK::Copy;
          cp.src_slot = e->slot;
          cp.dst_slot = s;
          cp.bytes = plan.slots[s].bytes();
          cp.note = "copy loop-carried value into loop storage";
          cur->push_back(std::move(cp));
        } else {
          emit_map(e, s, 0, canon_strides(t.shape), "initialise loop-carried value");
        }
        state_slot[k] = s;
      }
    }
    // ---- body
    std::vector<Step>* saved = cur;
    cur = &loop.body;
    ++loop_depth;
    for (size_t k = 0; k < n; ++k) {
      int arg = body.args[k];
      if (state_slot[k] >= 0) {
        env[arg] = leaf(state_slot[k], m.values[arg].type);
      } else {
        auto s = std::make_shared<Expr>();
        s->k = Expr::Sym;
        s->dt = m.values[arg].type.dt;
        s->shape = m.values[arg].type.shape;
        if ((int)k == counter) {  // its value in iteration `it` is known: init + it * step
          s->sym_depth = loop_depth;
          s->sym_a = counter_step;
          s->sym_b = counter_init;
        }
        env[arg] = s;
      }
    }
    int first_body_slot = (int)plan.slots.size();
    const int64_t saved_parts = nparts;
    if (row_sharded) nparts = 1;  // inside the body the arrays are the global ones (local_type() must not divide them)
    try {
      plan_region(body);
    } catch (...) {
      nparts = saved_parts;
      --loop_depth;
      throw;
    }
    nparts = saved_parts;
    --loop_depth;
    std::vector<int> yslot(n, -1);
    for (size_t k = 0; k < n; ++k) {
      if (state_slot[k] < 0) continue;
      ExprP y = env[body.yields[k]];
      if (!whole_slot(y)) y = leaf(materialise(y, "loop-carried result"), m.values[body.yields[k]].type);
      // a value defined outside the loop (and not itself loop-carried) must not be rotated into the loop's storage
      bool is_state = std::find(state_slot.begin(), state_slot.end(), y->slot) != state_slot.end();
      if (!is_state && y->slot < first_body_slot) y = leaf(materialise_copy(y), m.values[body.yields[k]].type);
      yslot[k] = y->slot;
    }
    cur = saved;
    // two carried values must not end up in one buffer
    {
      std::set<int> seen;
      for (size_t k = 0; k < n; ++k)
        if (yslot[k] >= 0 && !seen.insert(yslot[k]).second)
          throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while: two loop-carried values alias one result");
    }
    for (size_t k = 0; k < n; ++k)
      if (state_slot[k] >= 0) {
        loop.state_slots.push_back(state_slot[k]);
        loop.yield_slots.push_back(yslot[k]);
      }
    loop.note = "counted loop x" + std::to_string(trip);
    if (row_sharded) {
      // every step of the body must be a stencil update from one carried array into another; the rows a device needs
      // from its neighbours follow from the window offsets
      int up = 0, down = 0;
      int64_t rows = 0;
      for (int x : op.in)
        if (shard[x] == 0) rows = m.values[x].type.shape[0];
      for (const Step& b : loop.body) {
        const bool carried = b.kind == StepK::Stencil && !b.leaf_slot.empty() && b.out_slot.size() == 1 && plan.slots[b.leaf_slot[0]].row_block &&
                             plan.slots[b.out_slot[0]].row_block && b.st_src_ld == b.st_dst_ld;
        if (!carried)
          throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while carrying sharded tensors: the body is not made of slice-and-add updates between the carried arrays only (step: " + b.note + ")");
        int max_dy = 0;
        for (int dy : b.st_dy) max_dy = std::max(max_dy, dy);
        const int64_t row0 = b.st_src_off / b.st_src_ld, drow0 = b.st_dst_off / b.st_dst_ld;
        up = std::max<int>(up, (int)(drow0 - row0));
        down = std::max<int>(down, (int)(row0 + max_dy - drow0));
      }
      // a radius-1 loop gets two halo rows on each side, so that the executor may do two sweeps per pass over memory
      if (up == 1 && down == 1 && rows / saved_parts >= 2) up = down = 2;
      if (up < 0 || down < 0 || up > 2 || down > 2 || rows % saved_parts != 0 || rows / saved_parts < std::max(up, down) || rows / saved_parts < 1)
        throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while carrying sharded tensors: halo of more than 2 rows, or row blocks smaller than the halo");
      for (int s : loop.state_slots) {
        plan.slots[s].halo_up = up;
        plan.slots[s].halo_down = down;
      }
      for (int s : loop.yield_slots) {
        if (!plan.slots[s].row_block) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.while carrying sharded tensors: a carried value leaves the loop's own storage");
      }
      loop.row_sharded = true;
      loop.note += " over row blocks (halo " + std::to_string(up) + " up, " + std::to_string(down) + " down)";
    }
    cur->push_back(std::move(loop));
    // ---- results
    for (size_t k = 0; k < n; ++k) {
      int r = op.out[k];
      if (row_sharded && state_slot[k] >= 0) {
        shard[r] = 0;
        Type lt = local_type(r);
        Step out;
        out.kind = StepK::RowsOut;
        out.src_slot = state_slot[k];
        out.dst_slot = new_slot(lt);
        out.note = "row block out of loop storage";
        const int dst = out.dst_slot;
        cur->push_back(std::move(out));
        env[r] = leaf(dst, lt);
        continue;
      }
      if (state_slot[k] >= 0) env[r] = leaf(state_slot[k], m.values[r].type);
      else {
        auto s = std::make_shared<Expr>();  // final scalar values are not consumed by tensor code on the path
        s->k = Expr::Sym;
        s->dt = m.values[r].type.dt;
        env[r] = s;
      }
    }
  }
  int materialise_copy(const ExprP& e) {
    Type t{e->dt, e->shape};
    int s = new_slot(t);
    emit_map(e, s, 0, canon_strides(e->shape), "copy");
    return s;
  }

  void plan_region(const Region& r) {
    const Region* outer_region = cur_region;
    cur_region = &r;
    for (auto& op : r.ops) {
      switch (op.kind) {
        case OpK::Constant: plan_constant(op); break;
        case OpK::Iota: plan_iota(op); break;
        case OpK::Select:
          if (plan_masked_update(op)) break;
          plan_elementwise(op); break;
        case OpK::Unary: case OpK::Binary: case OpK::Convert: case OpK::Compare: case OpK::Clamp:
          plan_elementwise(op); break;
        case OpK::BroadcastInDim: case OpK::Transpose: case OpK::Slice: plan_view(op); break;
        case OpK::Reshape: plan_reshape(op); break;
        case OpK::Reduce: plan_reduce(op); break;
        case OpK::ReduceWindow: plan_reduce_window(op); break;
        case OpK::DynamicSlice: plan_dynamic_slice(op); break;
        case OpK::DynamicUpdateSlice: plan_dus(op); break;
        case OpK::Pad: plan_pad(op); break;
        case OpK::Concatenate: plan_concat(op); break;
        case OpK::DotGeneral: plan_dot(op); break;
        case OpK::While: plan_while(op); break;
        default: throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported op " + op.name);
      }
      if (op.kind != OpK::While)
        for (int v : op.in) --remaining[v];
    }
    cur_region = outer_region;
  }

  void run() {
    const Func& f = m.funcs.at("main");
    nparts = m.num_partitions;
    plan.num_partitions = nparts;
    count_uses(f.body);
    remaining = uses;
    int64_t mesh_size = 1;
    for (auto& kv : m.meshes)
      for (auto& ax : kv.second) mesh_size *= ax.second;
    if (nparts > 1 && !m.meshes.empty() && mesh_size != nparts)
      throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported: mesh size does not match mhlo.num_partitions");
    if (nparts > 1)
      for (auto& kv : m.meshes)
        if (kv.second.size() != 1) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported: only 1-D meshes are supported");
    for (size_t k = 0; k < f.body.args.size(); ++k) {
      int v = f.body.args[k];
      const ArgAttr& at = f.arg_attrs[k];
      if (nparts > 1 && !at.sharding_mesh.empty()) {
        int sd = -1;
        for (size_t d = 0; d < at.dim_axes.size(); ++d)
          if (!at.dim_axes[d].empty()) {
            if (sd >= 0) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported: argument sharded along several dimensions");
            sd = (int)d;
          }
        // A dimension that the mesh does not divide is not padded: Reactant asks XLA for a sharding that fits and
        // uses that (src/Sharding.jl:582-654, 895-926; the padded form of src/xla/Sharding.jl:236-244 is only a
        // probe).  Here such an argument is held in full by every device, and reported so by the sharding getters.
        if (sd >= 0 && m.values[v].type.shape[sd] % nparts != 0) sd = -1;
        shard[v] = sd;
      }
      Type lt = local_type(v);
      int slot = new_slot(lt, SlotK::Arg);
      plan.slots[slot].arg_index = (int)k;
      plan.slots[slot].writable = at.aliasing_output >= 0;
      plan.arg_types.push_back(lt);
      plan.arg_global_types.push_back(m.values[v].type);
      plan.arg_sharded_dim.push_back(shard[v]);
      plan.arg_alias.push_back(at.aliasing_output);
      env[v] = leaf(slot, lt);
    }
    cur = &plan.steps;
    plan_region(f.body);
    for (size_t k = 0; k < f.body.yields.size(); ++k) {
      int v = f.body.yields[k];
      ExprP e = env[v];
      if (!e || e->k == Expr::Sym) throw Error(RX_ERR_UNSUPPORTED_OP, "unsupported: @main returns a loop counter");
      Type lt = local_type(v);
      int slot;
      if (whole_slot(e) && plan.slots[e->slot].kind != SlotK::Const) slot = e->slot;
      else {
        slot = new_slot(lt);
        emit_map(e, slot, 0, canon_strides(lt.shape), "result " + std::to_string(k));
      }
      ResultBinding rb;
      rb.slot = slot;
      rb.type = lt;
      rb.sharded_dim = shard[v];
      plan.results.push_back(rb);
    }
    finalize_fusions();
    // a temp slot handed out twice would be freed twice: give later duplicates their own copy
    std::set<int> seen;
    for (auto& rb : plan.results) {
      if (plan.slots[rb.slot].kind == SlotK::Temp && !seen.insert(rb.slot).second) {
        int s = new_slot(rb.type);
        Step cp;
        cp.kind = StepK::Copy;
        cp.src_slot = rb.slot;
        cp.dst_slot = s;
        cp.bytes = plan.slots[s].bytes();
        cp.note = "duplicate result";
        plan.steps.push_back(std::move(cp));
        rb.slot = s;
      }
    }
  }
};

const char* step_name(StepK k) {
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

const char* fast_name(int id) {
  switch (id) {
    case FAST_SIN_ADD: return "sin_add";
    case FAST_IDENTITY: return "identity";
    case FAST_EXP_SUB: return "exp_sub";
    case FAST_STENCIL5_MUL: return "stencil5_mul";
    default: return "vm";
  }
}

void describe_steps(std::ostringstream& os, const std::vector<Step>& steps) {
  os << "[";
  for (size_t k = 0; k < steps.size(); ++k) {
    const Step& s = steps[k];
    if (k) os << ",";
    os << "{\"kind\":\"" << step_name(s.kind) << "\",\"note\":\"" << s.note << "\"";
    if (s.kind == StepK::Map || s.kind == StepK::ReduceFull || s.kind == StepK::ReduceRow || s.kind == StepK::ReduceCol || s.kind == StepK::Stencil || s.kind == StepK::LogSumExp) {
      os << ",\"chain\":\"" << fast_name(s.prog.fast_id) << "\",\"instrs\":" << s.prog.n_instr << ",\"leaves\":" << s.prog.n_leaves
         << ",\"linear\":" << s.prog.all_linear << ",\"rank\":" << s.prog.rank << ",\"dims\":[";
      for (int d = 0; d < s.prog.rank; ++d) os << (d ? "," : "") << s.prog.dim[d];
      os << "]";
      if (s.prog.wide) os << ",\"wide\":1";
    }
    if (s.kind == StepK::Gemm && s.gemm.has_epilogue)
      os << ",\"epilogue\":{\"instrs\":" << s.prog.n_instr << ",\"leaves\":" << s.prog.n_leaves << ",\"results\":" << s.prog.n_outs << ",\"column_sums\":" << s.gemm.n_col
         << ",\"full_sums\":" << s.gemm.n_full << "}";
    if (s.kind == StepK::SumPartials) os << ",\"jobs\":" << s.sums.size();
    if (s.kind == StepK::Loop) {
      os << ",\"trip\":" << s.trip << ",\"body\":";
      describe_steps(os, s.body);
    }
    os << "}";
  }
  os << "]";
}

}  // namespace

std::string Plan::describe() const {
  std::ostringstream os;
  os << "{\"num_partitions\":" << num_partitions << ",\"slots\":" << slots.size() << ",\"args\":" << arg_types.size()
     << ",\"results\":" << results.size() << ",\"steps\":";
  describe_steps(os, steps);
  os << "}";
  return os.str();
}

std::unique_ptr<Plan> build_plan(const Module& m) {
  auto p = std::make_unique<Plan>();
  Planner pl(m, *p);
  pl.run();
  return p;
}

}  // namespace rx
