// Chain specialiser: VmProgram -> CUDA source -> NVRTC (sm_100a cubin) -> driver module.
#include "rx_jit.h"

#include <cuda.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <vector>

#include "rx_b200.h"

namespace rx {

void set_last_error(int code, const std::string& msg);

namespace {

// The device headers, embedded at build time (build.py writes this file from the sources
// beside it) so that run-time compilation needs no file system access and no CUDA headers.
#include "rx_jit_embed.inc"

// ---- NVRTC, loaded on first use ---------------------------------------------------------
struct Nvrtc {
  void* lib = nullptr;
  int (*CreateProgram)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*DestroyProgram)(void**) = nullptr;
  int (*CompileProgram)(void*, int, const char* const*) = nullptr;
  int (*GetProgramLogSize)(void*, size_t*) = nullptr;
  int (*GetProgramLog)(void*, char*) = nullptr;
  int (*GetCUBINSize)(void*, size_t*) = nullptr;
  int (*GetCUBIN)(void*, char*) = nullptr;
  int (*AddNameExpression)(void*, const char*) = nullptr;
  int (*GetLoweredName)(void*, const char*, const char**) = nullptr;
  bool ok = false;
};

const Nvrtc& nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"};
    for (const char* nm : names) {
      n.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (n.lib) break;
    }
    if (!n.lib) return;
    auto sym = [&](const char* s) { return dlsym(n.lib, s); };
    n.CreateProgram = (decltype(n.CreateProgram))sym("nvrtcCreateProgram");
    n.DestroyProgram = (decltype(n.DestroyProgram))sym("nvrtcDestroyProgram");
    n.CompileProgram = (decltype(n.CompileProgram))sym("nvrtcCompileProgram");
    n.GetProgramLogSize = (decltype(n.GetProgramLogSize))sym("nvrtcGetProgramLogSize");
    n.GetProgramLog = (decltype(n.GetProgramLog))sym("nvrtcGetProgramLog");
    n.GetCUBINSize = (decltype(n.GetCUBINSize))sym("nvrtcGetCUBINSize");
    n.GetCUBIN = (decltype(n.GetCUBIN))sym("nvrtcGetCUBIN");
    n.AddNameExpression = (decltype(n.AddNameExpression))sym("nvrtcAddNameExpression");
    n.GetLoweredName = (decltype(n.GetLoweredName))sym("nvrtcGetLoweredName");
    n.ok = n.CreateProgram && n.DestroyProgram && n.CompileProgram && n.GetProgramLogSize && n.GetProgramLog && n.GetCUBINSize && n.GetCUBIN &&
           n.AddNameExpression && n.GetLoweredName;
  });
  return n;
}

// ---- driver entry points (the library links the CUDA runtime only) --------------------------
struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
  CUresult (*Occupancy)(int*, CUfunction, int, size_t) = nullptr;
  CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;  // optional
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;             // optional
  bool ok = false;
};

const Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* s) -> void* {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(s, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
      cudaGetLastError();
      return p;
    };
    d.ModuleLoadData = (decltype(d.ModuleLoadData))get("cuModuleLoadData");
    d.ModuleGetFunction = (decltype(d.ModuleGetFunction))get("cuModuleGetFunction");
    d.LaunchKernel = (decltype(d.LaunchKernel))get("cuLaunchKernel");
    d.Occupancy = (decltype(d.Occupancy))get("cuOccupancyMaxActiveBlocksPerMultiprocessor");
    d.LaunchKernelEx = (decltype(d.LaunchKernelEx))get("cuLaunchKernelEx");
    d.FuncSetAttribute = (decltype(d.FuncSetAttribute))get("cuFuncSetAttribute");
    d.ok = d.ModuleLoadData && d.ModuleGetFunction && d.LaunchKernel && d.Occupancy;
  });
  return d;
}

// ---- op expression text, from the same tables the interpreter expands ----------------------
struct OpText {
  const char* unary[VM_NUM_OPS] = {};
  const char* binary[VM_NUM_OPS] = {};
  OpText() {
#define RX_X(op, expr) unary[op] = #expr;
    RX_VM_UNARY_OPS(RX_X)
#undef RX_X
#define RX_X(op, expr) binary[op] = #expr;
    RX_VM_BINARY_OPS(RX_X)
#undef RX_X
  }
};
const OpText& op_text() {
  static OpText t;
  return t;
}

std::string hex32(uint32_t v) {
  char b[16];
  snprintf(b, sizeof b, "0x%08xu", v);
  return b;
}

std::mutex g_mu;
// RX_JIT_MIN_ELEMS overrides the default threshold (e.g. 0 to specialise every launch, -1 for none)
int64_t g_min_elems = getenv("RX_JIT_MIN_ELEMS") ? atoll(getenv("RX_JIT_MIN_ELEMS")) : (int64_t)1 << 20;
int64_t g_compiled = 0, g_hits = 0, g_failed = 0, g_disk_hits = 0;
std::map<std::string, std::vector<char>> g_cubins;              // source -> cubin
std::map<std::string, std::string> g_lowered;                   // source -> lowered kernel name
std::map<std::pair<int, std::string>, JitKernel> g_kernels;     // (device, source) -> loaded kernel

bool compile(const std::string& src, const std::string& name_expr, std::vector<char>* cubin, std::string* lowered, std::string* log) {
  const Nvrtc& n = nvrtc();
  void* prog = nullptr;
  if (n.CreateProgram(&prog, src.c_str(), "rx_chain.cu", kEmbedCount, kEmbedSrc, kEmbedNames) != 0) {
    *log = "nvrtcCreateProgram failed";
    return false;
  }
  n.AddNameExpression(prog, name_expr.c_str());
  // RX_JIT_VERBOSE=1 prints each generated source and ptxas' resource summary to stderr
  static const bool verbose = getenv("RX_JIT_VERBOSE") && atoi(getenv("RX_JIT_VERBOSE")) > 0;
  // RX_JIT_DEFINES="-DNAME=value -D..." is handed to the compiler as is (tuning experiments)
  std::vector<std::string> extra;
  if (const char* defs = getenv("RX_JIT_DEFINES")) {
    std::string t(defs), cur;
    for (char c : t + " ") {
      if (c == ' ') { if (!cur.empty()) extra.push_back(cur); cur.clear(); }
      else cur += c;
    }
  }
  std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "-std=c++17"};
#if defined(RX_BOUNDS) && RX_BOUNDS
  opts.push_back("-DRX_BOUNDS=1");  // the bounds-checked library compiles bounds-checked chains
#endif
  for (auto& e : extra) opts.push_back(e.c_str());
  if (verbose) opts.push_back("--ptxas-options=-v");
  if (verbose) fprintf(stderr, "---- %s\n%s\n", name_expr.c_str(), src.c_str());
  int rc = n.CompileProgram(prog, (int)opts.size(), opts.data());
  size_t ls = 0;
  n.GetProgramLogSize(prog, &ls);
  if (ls > 1) {
    log->resize(ls);
    n.GetProgramLog(prog, &(*log)[0]);
  }
  if (verbose) fprintf(stderr, "%s\n", log->c_str());
  bool ok = rc == 0;
  if (ok) {
    size_t cs = 0;
    const char* lname = nullptr;
    ok = n.GetCUBINSize(prog, &cs) == 0 && cs > 0;
    if (ok) {
      cubin->resize(cs);
      ok = n.GetCUBIN(prog, cubin->data()) == 0 && n.GetLoweredName(prog, name_expr.c_str(), &lname) == 0 && lname;
      if (ok) *lowered = lname;
    }
  }
  n.DestroyProgram(&prog);
  return ok;
}

// Optional on-disk cache of compiled chains (RX_JIT_CACHE_DIR=<existing directory>): the analogue, for this
// engine's only compiled artefact, of Reactant's persistent compile cache (src/PersistentCompileCache.jl).
// A file holds the source length, a newline, the generated source, the lowered kernel name, a newline, and the
// cubin; its name is a 64-bit FNV-1a hash of the source together with its length, and the stored source is
// compared on load, so a hash collision cannot hand out the wrong kernel.
std::string cache_path(const std::string& src) {
  const char* dir = getenv("RX_JIT_CACHE_DIR");
  if (!dir || !*dir) return "";
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : src) h = (h ^ c) * 1099511628211ull;
  char name[64];
  snprintf(name, sizeof name, "/rx_chain_%016llx_%zu.bin", (unsigned long long)h, src.size());
  return std::string(dir) + name;
}
bool cache_load(const std::string& src, std::vector<char>* cubin, std::string* lowered) {
  const std::string path = cache_path(src);
  if (path.empty()) return false;
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  std::string blob;
  char buf[65536];
  size_t n;
  while ((n = fread(buf, 1, sizeof buf, f)) > 0) blob.append(buf, n);
  fclose(f);
  // layout: source length (decimal) '\n' source lowered-name '\n' cubin
  size_t nl = blob.find('\n');
  if (nl == std::string::npos) return false;
  size_t slen = strtoull(blob.substr(0, nl).c_str(), nullptr, 10);
  if (slen != src.size() || blob.size() < nl + 1 + slen || blob.compare(nl + 1, slen, src) != 0) return false;
  size_t p = nl + 1 + slen, nl2 = blob.find('\n', p);
  if (nl2 == std::string::npos) return false;
  *lowered = blob.substr(p, nl2 - p);
  cubin->assign(blob.begin() + nl2 + 1, blob.end());
  return !cubin->empty();
}
void cache_store(const std::string& src, const std::vector<char>& cubin, const std::string& lowered) {
  const std::string path = cache_path(src);
  if (path.empty()) return;
  const std::string tmp = path + ".tmp" + std::to_string((long long)getpid());
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return;
  const std::string head = std::to_string(src.size()) + "\n";
  bool ok = fwrite(head.data(), 1, head.size(), f) == head.size() && fwrite(src.data(), 1, src.size(), f) == src.size() &&
            fwrite(lowered.data(), 1, lowered.size(), f) == lowered.size() && fputc('\n', f) != EOF && fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
  ok = fclose(f) == 0 && ok;
  if (ok) rename(tmp.c_str(), path.c_str());  // atomic: readers see a whole file or none
  else remove(tmp.c_str());
}

}  // namespace

// The generated source includes the embedded device headers by name, so the same text compiles to a different
// kernel when they change (a struct passed by value grows a field, say).  Their fingerprint is part of the text,
// and with it of the key of both caches.
static const std::string& headers_fingerprint() {
  static const std::string fp = [] {
    uint64_t h = 1469598103934665603ull;
    for (int k = 0; k < kEmbedCount; ++k)
      for (const char* c = kEmbedSrc[k]; *c; ++c) h = (h ^ (unsigned char)*c) * 1099511628211ull;
    char buf[32];
    snprintf(buf, sizeof buf, "%016llx", (unsigned long long)h);
    return std::string(buf);
  }();
  return fp;
}

std::string jit_chain_source(const VmProgram& P, int red_code, const char* family, const char* extra_members) {
  const OpText& T = op_text();
  std::string s;
  s.reserve(4096);
  s += "// headers: " + headers_fingerprint() + "\n";
  // what the compiler is told besides the source is part of the text too, so that the caches never hand a kernel
  // built one way to a library that asks for the other
#if defined(RX_BOUNDS) && RX_BOUNDS
  s += "// options: -DRX_BOUNDS=1\n";
#endif
  if (const char* defs = getenv("RX_JIT_DEFINES")) s += std::string("// options: ") + defs + "\n";
  s += "// family: ";
  s += family;
  s += "\n#define RX_CHAIN_SPECIALISED 1\n#include \"rx_chain_kernels.cuh\"\n";
  if (!strncmp(family, "k_gemm_pair", 11)) s += "#include \"rx_gemm_pair.cuh\"\n";
  s += "namespace rx {\nstruct SpecChain {\n";
  if (extra_members) s += extra_members;
  int max_reg = P.result_reg;
  for (int k = 0; k < P.n_leaves; ++k) max_reg = std::max<int>(max_reg, P.leaf[k].reg);
  for (int k = 0; k < P.n_outs; ++k) max_reg = std::max<int>(max_reg, P.out[k].reg);
  for (int k = 0; k < P.n_instr; ++k) {
    const VmInstr& in = P.ins[k];
    if (in.flags & VMF_STORE) max_reg = std::max<int>(max_reg, in.dst);
  }
  auto I = [](int v) { return std::to_string(v); };
  auto L = [](int64_t v) { return std::to_string((long long)v) + "LL"; };
  // The general map kernel spends most of its instructions on index arithmetic (unravelling the row, one offset per
  // operand from 64-bit strides): for it the rank, the dims and every stride are written into the source, so that
  // the loops over dims fold, divisions are by constants and operands with equal strides share their products.
  // (One compilation per shape; the other families stay shape-independent.)
  const bool shaped = !strncmp(family, "k_map_runs", 10);
  s += "  static constexpr int kRegs = " + I(max_reg + 1) + ";\n";
  s += "  static __device__ __forceinline__ int rank(const VmProgram& P) { return " + (shaped ? I(P.rank) : std::string("P.rank")) + "; }\n";
  s += "  static __device__ __forceinline__ int64_t dim(const VmProgram& P, int d) {\n";
  if (shaped) {
    s += "    switch (d) {\n";
    for (int d = 0; d < P.rank; ++d) s += "      case " + I(d) + ": return " + L(P.dim[d]) + ";\n";
    s += "    }\n    return 1;\n  }\n";
  } else {
    s += "    return P.dim[d];\n  }\n";
  }
  s += "  static __device__ __forceinline__ int n_leaves(const VmProgram&) { return " + I(P.n_leaves) + "; }\n";
  s += "  static __device__ __forceinline__ int n_outs(const VmProgram&) { return " + I(P.n_outs) + "; }\n";
  s += "  static __device__ __forceinline__ int result_reg(const VmProgram&) { return " + I(P.result_reg) + "; }\n";
  s += "  static __device__ __forceinline__ int red_code(int c) { return " + (red_code >= 0 ? I(red_code) : std::string("c")) + "; }\n";
  s += "  static __device__ __forceinline__ int leaf_reg(const VmProgram&, int k) {\n    switch (k) {\n";
  for (int k = 0; k < P.n_leaves; ++k) s += "      case " + I(k) + ": return " + I(P.leaf[k].reg) + ";\n";
  s += "    }\n    return 0;\n  }\n";
  s += "  static __device__ __forceinline__ int out_reg(const VmProgram&, int k) {\n    switch (k) {\n";
  for (int k = 0; k < P.n_outs; ++k) s += "      case " + I(k) + ": return " + I(P.out[k].reg) + ";\n";
  s += "    }\n    return 0;\n  }\n";
  s += "  static __device__ __forceinline__ VmLeaf leaf(const VmProgram& P, int k) {\n    VmLeaf l = P.leaf[k];\n    switch (k) {\n";
  for (int k = 0; k < P.n_leaves; ++k) {
    s += "      case " + I(k) + ": l.elem = " + I(P.leaf[k].elem) + "; l.linear = " + I(P.leaf[k].linear) + ";";
    if (shaped)
      for (int d = 0; d < kMaxRank; ++d) s += " l.stride[" + I(d) + "] = " + L(d < P.rank ? P.leaf[k].stride[d] : 0) + ";";
    s += " break;\n";
  }
  s += "    }\n    return l;\n  }\n";
  s += "  static __device__ __forceinline__ VmOut out(const VmProgram& P, int k) {\n    VmOut o = P.out[k];\n    switch (k) {\n";
  for (int k = 0; k < P.n_outs; ++k) {
    s += "      case " + I(k) + ": o.elem = " + I(P.out[k].elem) + ";";
    if (shaped)
      for (int d = 0; d < kMaxRank; ++d) s += " o.stride[" + I(d) + "] = " + L(d < P.rank ? P.out[k].stride[d] : 0) + ";";
    s += " break;\n";
  }
  s += "    }\n    return o;\n  }\n";
  s += "  template <int V>\n  static __device__ __forceinline__ void exec(const VmProgram& P, uint32_t (*R)[V], const int64_t* idx) {\n";
  s += "#pragma unroll\n    for (int v = 0; v < V; ++v) {\n      uint32_t acc = 0;\n";
  for (int k = 0; k < P.n_instr; ++k) {
    const VmInstr& in = P.ins[k];
    const std::string rb = "R[" + I(in.b) + "][v]", rc = "R[" + I(in.c) + "][v]";
    if (in.op == VM_LD) {
      s += "      acc = " + rb + ";\n";
    } else if (in.op == VM_IOTA) {
      s += "      acc = (uint32_t)(int32_t)(idx[" + I(in.a) + "] + (" + I(in.a) + " == P.rank - 1 ? v : 0));\n";
    } else if (in.op == VM_SELECT) {
      s += "      acc = acc ? " + rb + " : " + rc + ";\n";
    } else if (in.op == VM_MULADD) {
      s += "      acc = f2u(__fadd_rn(__fmul_rn(u2f(acc), u2f(" + rb + ")), u2f(" + rc + ")));\n";
    } else if (in.op == VM_MULADD_C) {
      s += "      acc = f2u(__fadd_rn(__fmul_rn(u2f(" + rb + "), u2f(" + rc + ")), u2f(acc)));\n";
    } else if (T.unary[in.op]) {
      // A constant that starts a value is read from the program (a kernel parameter), not written as a literal:
      // with a literal the compiler evaluates tanhf(c), expf(c) ... itself, and its value can differ in the last
      // bit from the one the device code computes in the interpreter.  Immediates of the exactly rounded ops
      // (add, multiply, divide, min, max) stay literals.
      const std::string immv = in.op == VM_CONST ? "P.ins[" + I(k) + "].imm" : hex32(in.imm);
      s += "      { const uint32_t ua = acc, imm = " + immv + "; const float a = u2f(ua), fimm = u2f(imm); const int32_t ia = (int32_t)ua; acc = (" +
           T.unary[in.op] + "); }\n";
    } else if (T.binary[in.op]) {
      s += "      { const uint32_t ua = acc, ub = " + rb + "; const float a = u2f(ua), b = u2f(ub); const int32_t ia = (int32_t)ua, ib = (int32_t)ub; const int cdir = " +
           I(in.c) + "; acc = (" + T.binary[in.op] + "); }\n";
    } else {
      s += "      // op " + I(in.op) + " has no effect\n";
    }
    if (in.flags & VMF_STORE) s += "      R[" + I(in.dst) + "][v] = acc;\n";
  }
  s += "    }\n  }\n};\n}  // namespace rx\n";
  return s;
}

bool jit_available() { return nvrtc().ok; }

int64_t jit_compile_only(const VmProgram& P, int red_code, const char* family, std::string* log, const char* extra_members) {
  if (!nvrtc().ok) {
    *log = "NVRTC library not found";
    return -1;
  }
  std::vector<char> cubin;
  std::string lowered;
  if (!compile(jit_chain_source(P, red_code, family, extra_members), std::string("rx::") + family, &cubin, &lowered, log)) return -1;
  return (int64_t)cubin.size();
}

void jit_set_min_elems(int64_t n) {
  std::lock_guard<std::mutex> g(g_mu);
  g_min_elems = n;
}

void jit_stats(int64_t out[5]) {
  std::lock_guard<std::mutex> g(g_mu);
  out[0] = g_compiled;
  out[1] = g_hits;
  out[2] = g_failed;
  out[3] = (nvrtc().ok && driver().ok) ? 0 : 1;
  out[4] = g_disk_hits;
}

const JitKernel* jit_chain_kernel(int device, const VmProgram& P, const char* family, int red_code, int64_t work_elems, bool* failed,
                                  const char* extra_members, bool force) {
  *failed = false;
  if (!force) {
    std::lock_guard<std::mutex> g(g_mu);
    if (g_min_elems < 0 || work_elems < g_min_elems) return nullptr;
  }
  if (!nvrtc().ok || !driver().ok) return nullptr;
  const std::string src = jit_chain_source(P, red_code, family, extra_members);
  auto key = std::make_pair(device, src);
  bool have_cubin = false;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_kernels.find(key);
    if (it != g_kernels.end()) {
      ++g_hits;
      return &it->second;  // entries are never erased: the pointer stays valid
    }
    have_cubin = g_cubins.count(src) != 0;
  }
  auto fail = [&](const std::string& msg) -> const JitKernel* {
    std::lock_guard<std::mutex> g(g_mu);
    ++g_failed;
    *failed = true;
    set_last_error(RX_ERR_CUDA, "chain specialisation (" + std::string(family) + "): " + msg);
    return nullptr;
  };
  if (!have_cubin) {
    // compile without holding the lock (a tenth of a second or more); two threads may compile the same chain at the
    // same time, the second result is dropped
    std::vector<char> cubin;
    std::string lowered, log;
    const bool from_disk = cache_load(src, &cubin, &lowered);
    if (!from_disk) {
      if (!compile(src, std::string("rx::") + family, &cubin, &lowered, &log)) return fail("NVRTC: " + log);
      cache_store(src, cubin, lowered);
    }
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_cubins.count(src)) {
      g_cubins[src] = std::move(cubin);
      g_lowered[src] = lowered;
      if (from_disk) ++g_disk_hits;
      else ++g_compiled;
    }
  }
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_kernels.find(key);
  if (it != g_kernels.end()) return &it->second;
  const Driver& d = driver();
  CUmodule mod = nullptr;
  CUfunction fn = nullptr;
  CUresult r = d.ModuleLoadData(&mod, g_cubins[src].data());
  if (r == CUDA_SUCCESS) r = d.ModuleGetFunction(&fn, mod, g_lowered[src].c_str());
  if (r != CUDA_SUCCESS) {
    ++g_failed;
    *failed = true;
    set_last_error(RX_ERR_CUDA, "chain specialisation (" + std::string(family) + "): loading " + g_lowered[src] + " returned " + std::to_string((int)r));
    return nullptr;
  }
  JitKernel k;
  k.fn = (void*)fn;
  int occ = 0;
  if (d.Occupancy(&occ, fn, 256, 0) != CUDA_SUCCESS || occ < 1) occ = 4;
  k.occupancy = occ;
  return &(g_kernels[key] = k);
}

cudaError_t jit_launch_cluster(const JitKernel* k, unsigned grid_x, unsigned block_x, unsigned cluster_x, size_t smem_bytes, void** args, cudaStream_t stream,
                               bool pdl) {
  const Driver& d = driver();
  if (!d.LaunchKernelEx || !d.FuncSetAttribute) return cudaErrorNotSupported;
  {
    std::lock_guard<std::mutex> g(g_mu);
    if (k->smem_limit < (int)smem_bytes) {
      CUresult r = d.FuncSetAttribute((CUfunction)k->fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem_bytes);
      if (r != CUDA_SUCCESS) return (cudaError_t)r;
      k->smem_limit = (int)smem_bytes;
    }
  }
  CUlaunchConfig cfg{};
  cfg.gridDimX = grid_x; cfg.gridDimY = 1; cfg.gridDimZ = 1;
  cfg.blockDimX = block_x; cfg.blockDimY = 1; cfg.blockDimZ = 1;
  cfg.sharedMemBytes = (unsigned)smem_bytes;
  cfg.hStream = (CUstream)stream;
  CUlaunchAttribute at[2];
  at[0].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
  at[0].value.clusterDim.x = cluster_x;
  at[0].value.clusterDim.y = 1;
  at[0].value.clusterDim.z = 1;
  at[1].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
  at[1].value.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 2 : 1;
  CUresult r = d.LaunchKernelEx(&cfg, (CUfunction)k->fn, args, nullptr);
  return r == CUDA_SUCCESS ? cudaSuccess : (cudaError_t)r;
}

cudaError_t jit_launch(const JitKernel* k, dim3 grid, dim3 block, void** args, cudaStream_t stream, bool pdl) {
  if (pdl && driver().LaunchKernelEx) {
    CUlaunchConfig cfg{};
    cfg.gridDimX = grid.x; cfg.gridDimY = grid.y; cfg.gridDimZ = grid.z;
    cfg.blockDimX = block.x; cfg.blockDimY = block.y; cfg.blockDimZ = block.z;
    cfg.hStream = (CUstream)stream;
    CUlaunchAttribute at[1];
    at[0].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    at[0].value.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CUresult r = driver().LaunchKernelEx(&cfg, (CUfunction)k->fn, args, nullptr);
    return r == CUDA_SUCCESS ? cudaSuccess : (cudaError_t)r;
  }
  CUresult r = driver().LaunchKernel((CUfunction)k->fn, grid.x, grid.y, grid.z, block.x, block.y, block.z, 0, (CUstream)stream, args, nullptr);
  return r == CUDA_SUCCESS ? cudaSuccess : (cudaError_t)r;
}

}  // namespace rx
