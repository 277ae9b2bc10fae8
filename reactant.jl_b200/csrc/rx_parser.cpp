// Recursive-descent parser for the MLIR pretty form of the StableHLO subset on
// the hot path.  The op spellings accepted here are the ones Reactant's op
// emitters produce (src/Ops.jl: unary :398-460, binary :536-589, transpose
// :724-737, pad :739-759, slice :761-793, dot_general :1075-1200,
// broadcast_in_dim :1320-1357, compare/select/convert :1865-1961, while
// :2349-2447, reduce :3491-3622, dynamic_update_slice :3662-3678) after the
// module has been printed with MLIR's default printer
// (src/mlir/IR/Operation.jl:30-47).  Everything else raises
// RX_ERR_UNSUPPORTED_OP naming the op: there is no fallback executor.
#include <string.h>
#include <cmath>
#include <cstdlib>
#include <sstream>

#include "rx_ir.h"
#include "rx_vm.h"

namespace rx {

size_t dt_size(DT t) {
  switch (t) {
    case DT::PRED: case DT::S8: case DT::U8: return 1;
    case DT::S16: case DT::U16: case DT::F16: case DT::BF16: return 2;
    case DT::S32: case DT::U32: case DT::F32: return 4;
    case DT::S64: case DT::U64: case DT::F64: case DT::C64: return 8;
    case DT::C128: return 16;
    default: return 0;
  }
}

const char* dt_name(DT t) {
  switch (t) {
    case DT::PRED: return "i1"; case DT::S8: return "i8"; case DT::S16: return "i16";
    case DT::S32: return "i32"; case DT::S64: return "i64"; case DT::U8: return "ui8";
    case DT::U16: return "ui16"; case DT::U32: return "ui32"; case DT::U64: return "ui64";
    case DT::F16: return "f16"; case DT::F32: return "f32"; case DT::F64: return "f64";
    case DT::BF16: return "bf16"; case DT::C64: return "complex<f32>"; case DT::C128: return "complex<f64>";
    default: return "?";
  }
}

std::string Type::str() const {
  std::string s = "tensor<";
  for (auto d : shape) s += std::to_string(d) + "x";
  return s + dt_name(dt) + ">";
}

namespace {

struct UnaryName { const char* n; int op; };
const UnaryName kUnary[] = {
    {"sine", VM_SIN}, {"cosine", VM_COS}, {"exponential", VM_EXP}, {"log", VM_LOG},
    {"tanh", VM_TANH}, {"sqrt", VM_SQRT}, {"rsqrt", VM_RSQRT}, {"negate", VM_NEG},
    {"abs", VM_ABS}, {"log_plus_one", VM_LOG1P}, {"exponential_minus_one", VM_EXPM1},
    {"floor", VM_FLOOR}, {"ceil", VM_CEIL}, {"sign", VM_SIGN}, {"logistic", VM_LOGISTIC},
    {"not", VM_NOT}, {"tan", VM_TAN}, {"cbrt", VM_CBRT}, {"round_nearest_even", VM_RINT}, {"round_nearest_afz", VM_ROUND},
    {"is_finite", VM_ISFINITE}};
const UnaryName kBinary[] = {
    {"add", VM_ADD}, {"subtract", VM_SUB}, {"multiply", VM_MUL}, {"divide", VM_DIV},
    {"maximum", VM_MAX}, {"minimum", VM_MIN}, {"power", VM_POW},
    {"and", VM_AND}, {"or", VM_OR}, {"xor", VM_XOR}, {"atan2", VM_ATAN2}, {"remainder", VM_REM}};

struct Parser {
  const std::string& s;
  size_t p = 0;
  Module* m;
  std::vector<std::map<std::string, int>> scopes;

  Parser(const std::string& text, Module* mod) : s(text), m(mod) {}

  int line_at(size_t pos) const {
    int l = 1;
    for (size_t i = 0; i < pos && i < s.size(); ++i) l += s[i] == '\n';
    return l;
  }
  [[noreturn]] void fail(int code, const std::string& msg) const {
    throw Error(code, "line " + std::to_string(line_at(p)) + ": " + msg);
  }
  void ws() {
    for (;;) {
      while (p < s.size() && isspace((unsigned char)s[p])) ++p;
      if (p + 1 < s.size() && s[p] == '/' && s[p + 1] == '/') {
        while (p < s.size() && s[p] != '\n') ++p;
        continue;
      }
      if (s.compare(p, 4, "loc(") == 0) {  // trailing location: skip balanced
        p += 3;
        skip_balanced('(', ')');
        continue;
      }
      break;
    }
  }
  bool eof() { ws(); return p >= s.size(); }
  bool peek(const char* t) {
    ws();
    return s.compare(p, strlen(t), t) == 0;
  }
  bool accept(const char* t) {
    if (peek(t)) { p += strlen(t); return true; }
    return false;
  }
  void expect(const char* t) {
    if (!accept(t)) fail(RX_ERR_PARSE, std::string("expected '") + t + "' near '" + s.substr(p, 24) + "'");
  }
  // keyword match: must not be followed by an identifier character
  bool accept_kw(const char* t) {
    ws();
    size_t n = strlen(t);
    if (s.compare(p, n, t) != 0) return false;
    char c = p + n < s.size() ? s[p + n] : ' ';
    if (isalnum((unsigned char)c) || c == '_' || c == '.') return false;
    p += n;
    return true;
  }
  void skip_balanced(char open, char close) {
    ws();
    if (p >= s.size() || s[p] != open) fail(RX_ERR_PARSE, std::string("expected '") + open + "'");
    int depth = 0;
    bool in_str = false;
    for (; p < s.size(); ++p) {
      char c = s[p];
      if (in_str) {
        if (c == '\\') ++p;
        else if (c == '"') in_str = false;
        continue;
      }
      if (c == '"') in_str = true;
      else if (c == open) ++depth;
      else if (c == close && --depth == 0) { ++p; return; }
    }
    fail(RX_ERR_PARSE, "unbalanced delimiter");
  }
  std::string balanced_text(char open, char close) {
    ws();
    size_t b = p;
    skip_balanced(open, close);
    return s.substr(b + 1, p - b - 2);
  }
  std::string ident() {
    ws();
    size_t b = p;
    while (p < s.size() && (isalnum((unsigned char)s[p]) || s[p] == '_' || s[p] == '.' || s[p] == '$' || s[p] == '-')) ++p;
    if (b == p) fail(RX_ERR_PARSE, "expected identifier near '" + s.substr(p, 24) + "'");
    return s.substr(b, p - b);
  }
  std::string value_name() {
    ws();
    if (p >= s.size() || s[p] != '%') fail(RX_ERR_PARSE, "expected SSA value near '" + s.substr(p, 24) + "'");
    size_t b = p++;
    while (p < s.size() && (isalnum((unsigned char)s[p]) || s[p] == '_' || s[p] == '.' || s[p] == '$' || s[p] == '-' || s[p] == '#')) ++p;
    return s.substr(b, p - b);
  }
  int64_t integer() {
    ws();
    size_t b = p;
    if (p < s.size() && (s[p] == '-' || s[p] == '+')) ++p;
    while (p < s.size() && isdigit((unsigned char)s[p])) ++p;
    if (b == p) fail(RX_ERR_PARSE, "expected integer near '" + s.substr(p, 24) + "'");
    return strtoll(s.substr(b, p - b).c_str(), nullptr, 10);
  }
  std::vector<int64_t> int_list() {  // [a, b, c]
    std::vector<int64_t> v;
    expect("[");
    if (accept("]")) return v;
    do v.push_back(integer()); while (accept(","));
    expect("]");
    return v;
  }

  DT elem_type(const std::string& t) {
    static const std::pair<const char*, DT> tbl[] = {
        {"f32", DT::F32}, {"f64", DT::F64}, {"bf16", DT::BF16}, {"f16", DT::F16}, {"i1", DT::PRED},
        {"i8", DT::S8}, {"i16", DT::S16}, {"i32", DT::S32}, {"i64", DT::S64},
        {"ui8", DT::U8}, {"ui16", DT::U16}, {"ui32", DT::U32}, {"ui64", DT::U64},
        {"si8", DT::S8}, {"si16", DT::S16}, {"si32", DT::S32}, {"si64", DT::S64}};
    for (auto& e : tbl)
      if (t == e.first) return e.second;
    fail(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type '" + t + "'");
  }
  Type type() {
    ws();
    if (!accept("tensor<")) fail(RX_ERR_UNSUPPORTED_TYPE, "expected tensor type near '" + s.substr(p, 24) + "'");
    Type t;
    for (;;) {
      ws();
      if (p < s.size() && isdigit((unsigned char)s[p])) {
        t.shape.push_back(integer());
        if (p >= s.size() || s[p] != 'x') fail(RX_ERR_PARSE, "malformed tensor shape");
        ++p;
      } else if (p < s.size() && s[p] == '?') {
        fail(RX_ERR_UNSUPPORTED_TYPE, "dynamic shapes are not supported");
      } else {
        break;
      }
    }
    size_t b = p;
    while (p < s.size() && s[p] != '>' && s[p] != ',') ++p;
    std::string et = s.substr(b, p - b);
    while (!et.empty() && isspace((unsigned char)et.back())) et.pop_back();
    t.dt = elem_type(et);
    if (accept(",")) {  // encoding attribute: skip
      int depth = 1;
      while (p < s.size() && depth) {
        if (s[p] == '<') ++depth;
        if (s[p] == '>') --depth;
        ++p;
      }
    } else {
      expect(">");
    }
    return t;
  }
  std::vector<Type> type_list_paren() {  // (t, t) or ()
    std::vector<Type> v;
    expect("(");
    if (accept(")")) return v;
    do {
      v.push_back(type());
      if (peek("{")) skip_balanced('{', '}');  // result attrs
    } while (accept(","));
    expect(")");
    return v;
  }
  // ": (ins) -> outs" or ": t[, t...]".  Returns result types (last types for the short form).
  void signature(std::vector<Type>* ins, std::vector<Type>* outs) {
    expect(":");
    if (peek("(")) {
      *ins = type_list_paren();
      expect("->");
      if (peek("(")) *outs = type_list_paren();
      else outs->push_back(type());
    } else {
      do outs->push_back(type()); while (accept(","));
    }
  }
  void maybe_attr_dict() {
    if (peek("{")) skip_balanced('{', '}');
  }

  int lookup(const std::string& name) {
    for (int i = (int)scopes.size() - 1; i >= 0; --i) {
      auto it = scopes[i].find(name);
      if (it != scopes[i].end()) return it->second;
    }
    fail(RX_ERR_PARSE, "use of undefined value " + name);
  }
  int use() { return lookup(value_name()); }
  int define(const std::string& name, const Type& t) {
    int id = m->new_value(t, name);
    scopes.back()[name] = id;
    return id;
  }

  // ---- attribute helpers -------------------------------------------------
  static std::vector<std::string> split_top(const std::string& t) {
    std::vector<std::string> out;
    int depth = 0;
    bool in_str = false;
    std::string cur;
    for (char c : t) {
      if (in_str) { cur += c; if (c == '"') in_str = false; continue; }
      if (c == '"') in_str = true;
      if (c == '<' || c == '(' || c == '[' || c == '{') ++depth;
      if (c == '>' || c == ')' || c == ']' || c == '}') --depth;
      if (c == ',' && depth == 0) { out.push_back(cur); cur.clear(); }
      else cur += c;
    }
    if (!cur.empty()) out.push_back(cur);
    return out;
  }
  static std::string trim(std::string t) {
    size_t b = t.find_first_not_of(" \t\n\r");
    if (b == std::string::npos) return "";
    size_t e = t.find_last_not_of(" \t\n\r");
    return t.substr(b, e - b + 1);
  }
  ArgAttr arg_attr(const std::string& dict) {
    ArgAttr a;
    for (auto& kv : split_top(dict)) {
      size_t eq = kv.find('=');
      std::string k = trim(eq == std::string::npos ? kv : kv.substr(0, eq));
      std::string v = eq == std::string::npos ? "" : trim(kv.substr(eq + 1));
      if (k == "tf.aliasing_output") a.aliasing_output = atoi(v.c_str());
      if (k == "sdy.sharding") {
        // #sdy.sharding<@mesh, [{"x"}, {}]>
        size_t at = v.find('@');
        size_t comma = v.find(',', at);
        if (at != std::string::npos && comma != std::string::npos) a.sharding_mesh = trim(v.substr(at + 1, comma - at - 1));
        size_t lb = v.find('[', comma);
        size_t rb = v.rfind(']');
        if (lb != std::string::npos && rb != std::string::npos && rb > lb) {
          for (auto& d : split_top(v.substr(lb + 1, rb - lb - 1))) {
            std::vector<std::string> axes;
            size_t q = 0;
            while ((q = d.find('"', q)) != std::string::npos) {
              size_t e = d.find('"', q + 1);
              axes.push_back(d.substr(q + 1, e - q - 1));
              q = e + 1;
            }
            a.dim_axes.push_back(axes);
          }
        }
      }
    }
    return a;
  }

  // ---- constants ---------------------------------------------------------
  static void put_elem(std::vector<uint8_t>& out, DT dt, double f, int64_t i, bool is_float_tok) {
    auto push = [&](const void* ptr, size_t n) { out.insert(out.end(), (const uint8_t*)ptr, (const uint8_t*)ptr + n); };
    switch (dt) {
      case DT::F32: { float v = is_float_tok ? (float)f : (float)i; push(&v, 4); break; }
      case DT::F64: { double v = is_float_tok ? f : (double)i; push(&v, 8); break; }
      case DT::BF16: {
        float v = is_float_tok ? (float)f : (float)i;
        uint32_t u; memcpy(&u, &v, 4);
        uint16_t h = (uint16_t)((u + 0x7FFF + ((u >> 16) & 1)) >> 16);
        push(&h, 2); break;
      }
      case DT::PRED: case DT::S8: case DT::U8: { int8_t v = (int8_t)(is_float_tok ? (int64_t)f : i); push(&v, 1); break; }
      case DT::S16: case DT::U16: { int16_t v = (int16_t)(is_float_tok ? (int64_t)f : i); push(&v, 2); break; }
      case DT::S32: case DT::U32: { int32_t v = (int32_t)(is_float_tok ? (int64_t)f : i); push(&v, 4); break; }
      case DT::S64: case DT::U64: { int64_t v = is_float_tok ? (int64_t)f : i; push(&v, 8); break; }
      default: break;
    }
  }
  // One scalar token of a dense<> payload -> (f, i).  Hex tokens carry raw bits.
  void scalar_token(const std::string& tok, DT dt, double* f, int64_t* i, bool* is_float) {
    *is_float = dt_is_float(dt);
    if (tok == "true") { *i = 1; *f = 1; return; }
    if (tok == "false") { *i = 0; *f = 0; return; }
    if (tok.size() > 2 && tok[0] == '0' && (tok[1] == 'x' || tok[1] == 'X')) {
      uint64_t bits = strtoull(tok.c_str() + 2, nullptr, 16);
      if (dt == DT::F32) { uint32_t u = (uint32_t)bits; float v; memcpy(&v, &u, 4); *f = v; }
      else if (dt == DT::F64) { double v; memcpy(&v, &bits, 8); *f = v; }
      else if (dt == DT::BF16) { uint32_t u = (uint32_t)bits << 16; float v; memcpy(&v, &u, 4); *f = v; }
      else { *i = (int64_t)bits; *f = (double)bits; }
      return;
    }
    if (*is_float) { *f = strtod(tok.c_str(), nullptr); *i = (int64_t)*f; }
    else { *i = strtoll(tok.c_str(), nullptr, 10); *f = (double)*i; }
  }
  void constant(Op& op, const Type& t, const std::string& payload) {
    std::string pl = trim(payload);
    size_t esz = dt_size(t.dt);
    if (!pl.empty() && pl[0] == '"') {  // hex blob: "0x...."
      std::string hex = pl.substr(1, pl.size() - 2);
      if (hex.compare(0, 2, "0x") != 0 && hex.compare(0, 2, "0X") != 0) fail(RX_ERR_PARSE, "malformed dense hex blob");
      std::vector<uint8_t> raw;
      for (size_t k = 2; k + 1 < hex.size(); k += 2) raw.push_back((uint8_t)strtoul(hex.substr(k, 2).c_str(), nullptr, 16));
      if (raw.size() == esz && t.numel() != 1) {
        // single element = splat
        op.dense = raw;
      } else if ((int64_t)raw.size() != t.numel() * (int64_t)esz) {
        fail(RX_ERR_PARSE, "dense hex blob size does not match the tensor type");
      } else {
        op.dense = raw;
      }
      if (raw.size() == esz) {
        op.splat = true;
        uint64_t bits = 0;
        memcpy(&bits, raw.data(), esz);
        char buf[32];
        snprintf(buf, sizeof buf, "0x%llx", (unsigned long long)bits);
        bool isf;
        scalar_token(buf, t.dt, &op.fval, &op.ival, &isf);
        op.dense.clear();
      } else {
        op.splat = false;
      }
      return;
    }
    // scalar or nested list of scalars
    std::vector<std::string> toks;
    std::string cur;
    for (char c : pl) {
      if (c == '[' || c == ']' || c == ',' || isspace((unsigned char)c)) {
        if (!cur.empty()) { toks.push_back(cur); cur.clear(); }
      } else {
        cur += c;
      }
    }
    if (!cur.empty()) toks.push_back(cur);
    if (toks.empty()) fail(RX_ERR_PARSE, "empty dense attribute");
    if (toks.size() == 1) {
      bool isf;
      op.splat = true;
      scalar_token(toks[0], t.dt, &op.fval, &op.ival, &isf);
      return;
    }
    if ((int64_t)toks.size() != t.numel()) fail(RX_ERR_PARSE, "dense element count does not match the tensor type");
    op.splat = false;
    for (auto& tk : toks) {
      double f = 0; int64_t i = 0; bool isf;
      scalar_token(tk, t.dt, &f, &i, &isf);
      put_elem(op.dense, t.dt, f, i, isf);
    }
  }

  // ---- ops -----------------------------------------------------------------
  void finish(Op& op, const std::vector<std::string>& res_names, const std::vector<Type>& outs) {
    if (res_names.size() != outs.size())
      fail(RX_ERR_PARSE, op.name + ": " + std::to_string(res_names.size()) + " result names for " + std::to_string(outs.size()) + " result types");
    for (size_t k = 0; k < outs.size(); ++k) op.out.push_back(define(res_names[k], outs[k]));
  }

  void parse_region_body(Region& r, bool* saw_return) {
    // caller consumed '{'; parse ops until the matching '}'
    *saw_return = false;
    for (;;) {
      ws();
      if (accept("}")) return;
      if (p >= s.size()) fail(RX_ERR_PARSE, "unterminated region");
      if (peek("^")) {  // block label
        while (p < s.size() && s[p] != '\n') ++p;
        continue;
      }
      parse_op(r, saw_return);
    }
  }

  // "stablehlo.reduce_window"(%x, %init) <{padding = dense<..> : tensor<Rx2xi64>, window_dimensions = array<i64: ..>, ..}> ({
  //   ^bb0(%a: tensor<T>, %b: tensor<T>):  %s = stablehlo.add %a, %b : tensor<T>  stablehlo.return %s : tensor<T>
  // }) : (tensor<..>, tensor<T>) -> tensor<..>
  // -- the generic form MLIR prints for the op Reactant's scans emit (src/Ops.jl:3967-4010).
  void parse_reduce_window(Region& region, const std::vector<std::string>& res, int line) {
    Op op;
    op.name = "stablehlo.reduce_window";
    op.kind = OpK::ReduceWindow;
    op.line = line;
    expect("(");
    op.in.push_back(use());
    expect(",");
    op.in.push_back(use());
    if (accept(",")) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with several operands");
    expect(")");
    ws();
    size_t a0 = p;
    skip_balanced('<', '>');
    const std::string attrs = s.substr(a0, p - a0);
    auto ints_after = [&](const std::string& key, bool required) {
      std::vector<int64_t> v;
      size_t k = attrs.find(key);
      if (k == std::string::npos) {
        if (required) fail(RX_ERR_PARSE, "stablehlo.reduce_window without " + key);
        return v;
      }
      size_t b = attrs.find('<', k);  // dense<...> or array<i64: ...>
      if (b == std::string::npos) fail(RX_ERR_PARSE, "stablehlo.reduce_window: malformed " + key);
      ++b;
      size_t e2 = b;
      for (int depth = 0; e2 < attrs.size() && !(attrs[e2] == '>' && depth == 0); ++e2) {
        if (attrs[e2] == '<') ++depth;
        if (attrs[e2] == '>') --depth;
      }
      if (key != "padding") {  // skip the element type of array<i64: ...>
        size_t colon = attrs.find(':', b);
        if (colon == std::string::npos || colon > e2) fail(RX_ERR_PARSE, "stablehlo.reduce_window: malformed " + key);
        b = colon + 1;
      }
      const std::string body = attrs.substr(b, e2 - b);
      for (size_t q = 0; q < body.size();) {
        if (isdigit((unsigned char)body[q]) || (body[q] == '-' && q + 1 < body.size() && isdigit((unsigned char)body[q + 1]))) {
          size_t used = 0;
          v.push_back(std::stoll(body.substr(q), &used));
          q += used;
        } else {
          ++q;
        }
      }
      return v;
    };
    op.dims = ints_after("window_dimensions", true);
    const size_t rank = op.dims.size();
    std::vector<int64_t> pad = ints_after("padding", false);
    if (pad.empty()) pad.assign(2 * rank, 0);
    if (pad.size() == 1) pad.assign(2 * rank, pad[0]);  // splat
    if (pad.size() != 2 * rank) fail(RX_ERR_PARSE, "stablehlo.reduce_window: padding does not match the window rank");
    for (size_t d = 0; d < rank; ++d) {
      op.start.push_back(pad[2 * d]);
      op.limit.push_back(pad[2 * d + 1]);
    }
    op.stride = ints_after("window_strides", false);
    op.dilation = ints_after("window_dilations", false);
    if (op.stride.empty()) op.stride.assign(rank, 1);
    if (op.dilation.empty()) op.dilation.assign(rank, 1);
    if (op.stride.size() != rank || op.dilation.size() != rank) fail(RX_ERR_PARSE, "stablehlo.reduce_window: strides or dilations do not match the window rank");
    for (size_t d = 0; d < rank; ++d)
      if (op.stride[d] < 1 || op.dilation[d] < 1 || op.dims[d] < 1) fail(RX_ERR_PARSE, "stablehlo.reduce_window: non-positive window size, stride or dilation");
    for (int64_t v : ints_after("base_dilations", false))
      if (v != 1) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with base_dilations other than 1");
    expect("(");
    expect("{");
    scopes.emplace_back();
    ws();
    if (peek("^")) {
      while (p < s.size() && s[p] != '(') ++p;
      expect("(");
      do {
        std::string n = value_name();
        expect(":");
        define(n, type());
      } while (accept(","));
      expect(")");
      expect(":");
    }
    Region body;
    bool ret;
    parse_region_body(body, &ret);
    scopes.pop_back();
    expect(")");
    if (body.ops.size() != 1 || body.yields.size() != 1 || body.ops[0].out[0] != body.yields[0])
      fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window with a multi-op body");
    static const std::pair<const char*, RedK> reds[] = {
        {"stablehlo.add", RedK::Add}, {"stablehlo.maximum", RedK::Max}, {"stablehlo.minimum", RedK::Min}, {"stablehlo.multiply", RedK::Mul}};
    bool ok = false;
    for (auto& r : reds)
      if (body.ops[0].name == r.first) { op.red = r.second; ok = true; }
    if (!ok) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce_window applying " + body.ops[0].name);
    std::vector<Type> ins, outs;
    signature(&ins, &outs);
    if (rank != m->values[op.in[0]].type.shape.size()) fail(RX_ERR_PARSE, "stablehlo.reduce_window: window rank does not match the operand");
    finish(op, res, outs);
    region.ops.push_back(std::move(op));
  }

  // enzymexla.math.gelu (what NNlib's gelu / gelu_tanh / gelu_sigmoid trace to: ext/ReactantNNlibExt/Implementations.jl:12-25,
  // src/Ops.jl:4153-4175).  Reactant's own pipeline lowers it to elementwise ops before the runtime sees the module
  // (`lower-enzymexla-math`, src/compiler/Compiler.jl:417); a module that still carries it is expanded here the same
  // way, so that it fuses like any other chain:
  //   TANH     0.5 * x * (1 + tanh(sqrt(2/pi) * (x + 0.044715 * x^3)))
  //   SIGMOID  x * logistic(1.702 * x)
  // The exact form (NONE) needs erf, which the chain machine does not have: refused by name.
  void parse_math_gelu(Region& region, const std::vector<std::string>& res, int line, bool generic) {
    int x;
    std::string attrs;
    if (generic) {
      expect("(");
      x = use();
      expect(")");
      ws();
      if (peek("<")) { expect("<"); attrs = balanced_text('{', '}'); expect(">"); }
      else if (peek("{")) attrs = balanced_text('{', '}');
    } else {
      x = use();
      ws();
      if (peek("{")) attrs = balanced_text('{', '}');
    }
    std::vector<Type> ins, outs;
    signature(&ins, &outs);
    if (res.size() != 1 || outs.size() != 1) fail(RX_ERR_PARSE, "enzymexla.math.gelu has one result");
    const Type t = outs[0];
    if (!dt_is_float(t.dt)) fail(RX_ERR_UNSUPPORTED_TYPE, "unsupported element type in enzymexla.math.gelu");
    const bool tanh_form = attrs.find("TANH") != std::string::npos, sigmoid_form = attrs.find("SIGMOID") != std::string::npos;
    if (!tanh_form && !sigmoid_form) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op enzymexla.math.gelu with gelu_approximation NONE (erf)");
    int counter = 0;
    auto fresh = [&]() { return m->new_value(t, res[0] + "$gelu" + std::to_string(counter++)); };
    auto konst = [&](double v) {
      Op c;
      c.kind = OpK::Constant;
      c.name = "stablehlo.constant";
      c.line = line;
      c.splat = true;
      c.fval = v;
      c.out.push_back(fresh());
      region.ops.push_back(c);
      return c.out[0];
    };
    auto emit = [&](OpK kind, const char* name, int vmop, std::vector<int> in, int out = -1) {
      Op o;
      o.kind = kind;
      o.name = name;
      o.line = line;
      o.ew = vmop;
      o.in = std::move(in);
      o.out.push_back(out >= 0 ? out : fresh());
      region.ops.push_back(o);
      return o.out[0];
    };
    const int result = define(res[0], t);
    if (tanh_form) {
      int x2 = emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {x, x});
      int x3 = emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {x2, x});
      int t0 = emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {konst(0.044715), x3});
      int t1 = emit(OpK::Binary, "stablehlo.add", VM_ADD, {x, t0});
      int t2 = emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {konst(0.7978845608028654), t1});
      int th = emit(OpK::Unary, "stablehlo.tanh", VM_TANH, {t2});
      int t3 = emit(OpK::Binary, "stablehlo.add", VM_ADD, {konst(1.0), th});
      int t4 = emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {konst(0.5), x});
      emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {t4, t3}, result);
    } else {
      int t0 = emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {konst(1.702), x});
      int sg = emit(OpK::Unary, "stablehlo.logistic", VM_LOGISTIC, {t0});
      emit(OpK::Binary, "stablehlo.multiply", VM_MUL, {x, sg}, result);
    }
  }

  void parse_op(Region& region, bool* saw_return) {
    ws();
    int line = line_at(p);
    std::vector<std::string> res;
    if (peek("%")) {
      do {
        std::string n = value_name();
        if (accept(":")) {
          int64_t cnt = integer();
          for (int64_t k = 0; k < cnt; ++k) res.push_back(n + "#" + std::to_string(k));
        } else {
          res.push_back(n);
        }
      } while (accept(","));
      expect("=");
    }
    ws();
    if (peek("\"")) {
      size_t e = s.find('"', p + 1);
      std::string quoted = s.substr(p, e - p + 1);
      p = e + 1;
      if (quoted == "\"enzymexla.math.gelu\"") {
        parse_math_gelu(region, res, line, true);
        return;
      }
      if (quoted != "\"stablehlo.reduce_window\"") fail(RX_ERR_UNSUPPORTED_OP, "unsupported op (generic form) " + quoted);
      parse_reduce_window(region, res, line);
      return;
    }
    std::string name = ident();
    if (name == "enzymexla.math.gelu") {
      parse_math_gelu(region, res, line, false);
      return;
    }
    Op op;
    op.name = name;
    op.line = line;
    std::vector<Type> ins, outs;

    if (name == "return" || name == "func.return" || name == "stablehlo.return") {
      op.kind = OpK::Return;
      if (peek("%")) {
        do op.in.push_back(use()); while (accept(","));
        maybe_attr_dict();
        signature(&ins, &outs);
      }
      region.yields = op.in;
      *saw_return = true;
      return;
    }
    if (name.compare(0, 10, "stablehlo.") != 0 && name != "sdy.sharding_constraint")
      fail(RX_ERR_UNSUPPORTED_OP, "unsupported op " + name);
    std::string shortn = name == "sdy.sharding_constraint" ? name : name.substr(10);

    if (shortn == "sdy.sharding_constraint") {
      // identity on values; the sharding of arguments is what the planner uses
      op.kind = OpK::Unary;
      op.ew = VM_MOV;
      op.in.push_back(use());
      if (peek("<")) skip_balanced('<', '>');
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "constant") {
      op.kind = OpK::Constant;
      maybe_attr_dict();
      ws();
      if (!accept("dense")) fail(RX_ERR_PARSE, "only dense<> constants are supported");
      std::string payload = balanced_text('<', '>');
      expect(":");
      Type t = type();
      constant(op, t, payload);
      finish(op, res, {t});
    } else if (shortn == "iota") {
      op.kind = OpK::Iota;
      expect("dim");
      expect("=");
      op.dims.push_back(integer());
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "convert") {
      op.kind = OpK::Convert;
      op.in.push_back(use());
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "compare") {
      op.kind = OpK::Compare;
      std::string dir = ident();
      static const std::pair<const char*, int> dirs[] = {{"EQ", CMP_EQ}, {"NE", CMP_NE}, {"LT", CMP_LT}, {"LE", CMP_LE}, {"GT", CMP_GT}, {"GE", CMP_GE}};
      op.ew = -1;
      for (auto& d : dirs) if (dir == d.first) op.ew = d.second;
      if (op.ew < 0) fail(RX_ERR_PARSE, "unknown comparison direction " + dir);
      expect(",");
      op.in.push_back(use());
      expect(",");
      op.in.push_back(use());
      if (accept(",")) {
        std::string ct = ident();
        if (ct == "UNSIGNED") fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.compare with UNSIGNED comparison");
      }
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "select" || shortn == "clamp") {
      op.kind = shortn == "select" ? OpK::Select : OpK::Clamp;
      op.in.push_back(use()); expect(",");
      op.in.push_back(use()); expect(",");
      op.in.push_back(use());
      maybe_attr_dict();
      signature(&ins, &outs);
      if (ins.empty() && outs.size() > 1) outs.erase(outs.begin(), outs.end() - 1);
      finish(op, res, outs);
    } else if (shortn == "broadcast_in_dim" || shortn == "transpose") {
      op.kind = shortn == "transpose" ? OpK::Transpose : OpK::BroadcastInDim;
      op.in.push_back(use());
      expect(",");
      expect("dims");
      expect("=");
      op.dims = int_list();
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "reshape") {
      op.kind = OpK::Reshape;
      op.in.push_back(use());
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "slice") {
      op.kind = OpK::Slice;
      op.in.push_back(use());
      expect("[");
      do {
        op.start.push_back(integer());
        expect(":");
        op.limit.push_back(integer());
        op.stride.push_back(accept(":") ? integer() : 1);
      } while (accept(","));
      expect("]");
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "dynamic_slice") {
      // %r = stablehlo.dynamic_slice %x, %i0, %i1, sizes = [1, 4] : (tensor<..>, tensor<i32>, tensor<i32>) -> tensor<..>
      op.kind = OpK::DynamicSlice;
      for (;;) {
        op.in.push_back(use());
        expect(",");
        if (accept_kw("sizes")) break;
      }
      expect("=");
      op.dims = int_list();
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "dynamic_update_slice") {
      op.kind = OpK::DynamicUpdateSlice;
      do op.in.push_back(use()); while (accept(","));
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "pad") {
      op.kind = OpK::Pad;
      op.in.push_back(use()); expect(",");
      op.in.push_back(use()); expect(",");
      expect("low"); expect("="); op.start = int_list(); expect(",");
      expect("high"); expect("="); op.limit = int_list(); expect(",");
      expect("interior"); expect("="); op.stride = int_list();
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "concatenate") {
      op.kind = OpK::Concatenate;
      for (;;) {
        op.in.push_back(use());
        expect(",");
        if (accept_kw("dim")) break;
      }
      expect("=");
      op.dims.push_back(integer());
      maybe_attr_dict();
      signature(&ins, &outs);
      finish(op, res, outs);
    } else if (shortn == "dot_general") {
      op.kind = OpK::DotGeneral;
      op.in.push_back(use()); expect(",");
      op.in.push_back(use()); expect(",");
      if (accept_kw("batching_dims")) {
        expect("="); op.lbatch = int_list(); expect("x"); op.rbatch = int_list(); expect(",");
      }
      expect("contracting_dims"); expect("=");
      op.lcontract = int_list(); expect("x"); op.rcontract = int_list();
      std::string algorithm;
      bool has_algorithm = false;
      while (accept(",")) {
        if (accept_kw("precision")) {
          expect("=");
          std::string pr = balanced_text('[', ']');
          for (auto& e : split_top(pr))
            if (trim(e) != "DEFAULT") fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general with precision " + trim(e));
        } else if (accept_kw("algorithm")) {
          expect("=");
          std::string al = balanced_text('<', '>');
          algorithm = al;
          has_algorithm = true;
        } else {
          fail(RX_ERR_PARSE, "unexpected dot_general attribute near '" + s.substr(p, 24) + "'");
        }
      }
      maybe_attr_dict();
      signature(&ins, &outs);
      if (has_algorithm) {
        // What the kernels compute is one pass over the operands in their own element type with float32
        // accumulation: the presets F32_F32_F32 on f32 operands and BF16_BF16_F32 on bf16 operands
        // (src/Configuration.jl:216-238, 346-348).  Multi-pass (X3 / X6 / X9), reduced-precision accumulation and
        // mismatched operand types are refused.
        auto field = [&](const char* key) {
          size_t q = algorithm.find(std::string(key) + " = ");
          if (q == std::string::npos) return std::string();
          q += strlen(key) + 3;
          size_t e = algorithm.find_first_of(",>", q);
          return trim(algorithm.substr(q, e == std::string::npos ? std::string::npos : e - q));
        };
        const std::string want = ins.empty() ? "" : dt_name(ins[0].dt);
        const bool ok = field("accumulation_type") == "f32" && field("lhs_precision_type") == want && field("rhs_precision_type") == want &&
                        field("lhs_component_count") == "1" && field("rhs_component_count") == "1" && field("num_primitive_operations") == "1" &&
                        field("allow_imprecise_accumulation") == "false";
        if (!ok) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.dot_general with algorithm <" + algorithm + "> on " + want + " operands");
      }
      finish(op, res, outs);
    } else if (shortn == "reduce") {
      op.kind = OpK::Reduce;
      expect("(");
      op.in.push_back(use());
      expect("init"); expect(":");
      op.in.push_back(use());
      if (accept(",")) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce with several operands");
      expect(")");
      std::string applied;
      if (accept_kw("applies")) applied = ident();
      expect("across"); expect("dimensions"); expect("=");
      op.dims = int_list();
      maybe_attr_dict();
      signature(&ins, &outs);
      if (applied.empty()) {
        expect("reducer");
        scopes.emplace_back();
        expect("(");
        std::vector<int> rargs;
        do {
          std::string n = value_name();
          expect(":");
          rargs.push_back(define(n, type()));
        } while (accept(","));
        expect(")");
        expect("{");
        Region body;
        bool ret;
        parse_region_body(body, &ret);
        scopes.pop_back();
        if (body.ops.size() != 1 || body.yields.size() != 1 || body.ops[0].out[0] != body.yields[0])
          fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce with a multi-op reducer");
        applied = body.ops[0].name;
      }
      static const std::pair<const char*, RedK> reds[] = {
          {"stablehlo.add", RedK::Add}, {"stablehlo.maximum", RedK::Max}, {"stablehlo.minimum", RedK::Min},
          {"stablehlo.multiply", RedK::Mul}, {"stablehlo.or", RedK::Or}, {"stablehlo.and", RedK::And}};
      bool ok = false;
      for (auto& r : reds) if (applied == r.first) { op.red = r.second; ok = true; }
      if (!ok) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op stablehlo.reduce applying " + applied);
      finish(op, res, outs);
    } else if (shortn == "while") {
      op.kind = OpK::While;
      expect("(");
      std::vector<std::string> iter_names;
      if (!accept(")")) {
        do {
          iter_names.push_back(value_name());
          expect("=");
          op.in.push_back(use());
        } while (accept(","));
        expect(")");
      }
      expect(":");
      do outs.push_back(type()); while (accept(","));
      if (accept_kw("attributes")) skip_balanced('{', '}');
      if (outs.size() != iter_names.size()) fail(RX_ERR_PARSE, "stablehlo.while: type count does not match operands");
      op.regions.resize(2);
      for (int r = 0; r < 2; ++r) {
        expect(r == 0 ? "cond" : "do");
        expect("{");
        scopes.emplace_back();
        for (size_t k = 0; k < iter_names.size(); ++k) op.regions[r].args.push_back(define(iter_names[k], outs[k]));
        bool ret;
        parse_region_body(op.regions[r], &ret);
        scopes.pop_back();
      }
      finish(op, res, outs);
    } else {
      bool done = false;
      for (auto& u : kUnary)
        if (shortn == u.n) {
          op.kind = OpK::Unary;
          op.ew = u.op;
          op.in.push_back(use());
          maybe_attr_dict();
          signature(&ins, &outs);
          finish(op, res, outs);
          done = true;
          break;
        }
      if (!done)
        for (auto& b : kBinary)
          if (shortn == b.n) {
            op.kind = OpK::Binary;
            op.ew = b.op;
            op.in.push_back(use()); expect(",");
            op.in.push_back(use());
            maybe_attr_dict();
            signature(&ins, &outs);
            finish(op, res, outs);
            done = true;
            break;
          }
      if (!done) fail(RX_ERR_UNSUPPORTED_OP, "unsupported op " + name);
    }
    region.ops.push_back(std::move(op));
  }

  void parse_func() {
    // after "func.func"
    accept_kw("public") || accept_kw("private");
    expect("@");
    Func f;
    f.name = ident();
    scopes.emplace_back();
    expect("(");
    if (!accept(")")) {
      do {
        std::string n = value_name();
        expect(":");
        Type t = type();
        ArgAttr a;
        if (peek("{")) a = arg_attr(balanced_text('{', '}'));
        f.body.args.push_back(define(n, t));
        f.arg_attrs.push_back(a);
      } while (accept(","));
      expect(")");
    }
    if (accept("->")) {
      if (peek("(")) {
        expect("(");
        if (!accept(")")) {
          do {
            f.result_types.push_back(type());
            ArgAttr a;
            if (peek("{")) a = arg_attr(balanced_text('{', '}'));
            f.res_attrs.push_back(a);
          } while (accept(","));
          expect(")");
        }
      } else {
        f.result_types.push_back(type());
        f.res_attrs.emplace_back();
      }
    }
    if (accept_kw("attributes")) skip_balanced('{', '}');
    expect("{");
    bool ret;
    parse_region_body(f.body, &ret);
    scopes.pop_back();
    if (f.body.yields.size() != f.result_types.size())
      fail(RX_ERR_PARSE, "@" + f.name + ": returns " + std::to_string(f.body.yields.size()) + " values, signature declares " + std::to_string(f.result_types.size()));
    m->funcs[f.name] = std::move(f);
  }

  void parse_module_attrs(const std::string& dict) {
    for (auto& kv : split_top(dict)) {
      size_t eq = kv.find('=');
      if (eq == std::string::npos) continue;
      std::string k = trim(kv.substr(0, eq)), v = trim(kv.substr(eq + 1));
      if (k == "mhlo.num_partitions") m->num_partitions = atoll(v.c_str());
      if (k == "mhlo.num_replicas") m->num_replicas = atoll(v.c_str());
    }
  }

  void parse_top() {
    bool in_module = false;
    if (accept_kw("module") || accept_kw("builtin.module")) {
      in_module = true;
      if (accept("@")) m->name = ident();
      if (accept_kw("attributes")) parse_module_attrs(balanced_text('{', '}'));
      expect("{");
    }
    for (;;) {
      ws();
      if (p >= s.size()) break;
      if (in_module && accept("}")) break;
      if (accept_kw("func.func")) {
        parse_func();
      } else if (accept_kw("sdy.mesh")) {
        expect("@");
        std::string name = ident();
        expect("=");
        std::string body = balanced_text('<', '>');
        std::vector<std::pair<std::string, int64_t>> axes;
        size_t q = 0;
        while ((q = body.find('"', q)) != std::string::npos) {
          size_t e = body.find('"', q + 1);
          std::string ax = body.substr(q + 1, e - q - 1);
          size_t eq = body.find('=', e);
          axes.push_back({ax, atoll(body.c_str() + eq + 1)});
          q = e + 1;
        }
        m->meshes[name] = axes;
      } else {
        fail(RX_ERR_UNSUPPORTED_OP, "unsupported top-level construct near '" + s.substr(p, 32) + "'");
      }
    }
    if (!m->funcs.count("main")) fail(RX_ERR_PARSE, "module has no @main function");
  }
};

}  // namespace

std::unique_ptr<Module> parse_module(const std::string& text) {
  auto m = std::make_unique<Module>();
  Parser ps(text, m.get());
  ps.parse_top();
  return m;
}

}  // namespace rx
