// Run-time fusion of element-wise chains: an expression over same-shape tensors
// ("selu((a+b)*(c+d))") is parsed, differentiated in reverse mode on the host,
// emitted as CUDA C (one forward kernel, one reverse kernel that recomputes the
// intermediates and produces every leaf gradient in a single pass), compiled
// by NVRTC for sm_100a and cached by (expression, dtype).  The generated
// kernels have the same shape as the static element-wise kernels: 128-bit
// streaming accesses, one trip per CTA, fp32 arithmetic for r16/r32.
//
// The reference links nvrtc (build.zig:139) but never calls it; its op wrappers
// launch one kernel per op (src/ops/*.zig).  The grammar accepted here covers
// the flat ops of that layer: + - * (addition, subtraction, hadamard), unary -
// (negate), literal operands (translate, dilate), relu(x), selu(x).
//
// NVRTC and the driver's module API are resolved at run time (dlopen /
// cudaGetDriverEntryPoint), so the library still loads where they are absent.
#include "mp_common.cuh"
#include "../../include/mp_jit.h"

#include <dlfcn.h>
#include <string.h>

#include <map>
#include <tuple>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace {

// ------------------------------ expression --------------------------------
enum class Kind { Leaf, Const, Add, Sub, Mul, Neg, Selu, Relu };
struct Node {
  Kind kind;
  int a = -1, b = -1;  // operand node ids
  int leaf = -1;       // Leaf: index into leaves
  double value = 0.0;  // Const
};

struct Expr {
  std::vector<Node> nodes;  // topological order: operands precede users
  std::vector<std::string> leaves;
  int root = -1;
  std::string error;
};

class Parser {
 public:
  Parser(const char* text, Expr& e) : p_(text), e_(e) {}
  bool parse() {
    e_.root = sum();
    skip();
    if (e_.error.empty() && *p_ != '\0') e_.error = std::string("unexpected '") + *p_ + "'";
    return e_.error.empty() && e_.root >= 0;
  }

 private:
  void skip() { while (*p_ == ' ' || *p_ == '\t' || *p_ == '\n') ++p_; }
  int add(Node n) { e_.nodes.push_back(n); return static_cast<int>(e_.nodes.size()) - 1; }
  int fail(const std::string& m) { if (e_.error.empty()) e_.error = m; return -1; }
  int sum() {
    int lhs = product();
    for (;;) {
      skip();
      if (lhs < 0) return lhs;
      if (*p_ == '+' || *p_ == '-') {
        const char op = *p_++;
        const int rhs = product();
        if (rhs < 0) return rhs;
        Node n; n.kind = op == '+' ? Kind::Add : Kind::Sub; n.a = lhs; n.b = rhs;
        lhs = add(n);
      } else {
        return lhs;
      }
    }
  }
  int product() {
    int lhs = unary();
    for (;;) {
      skip();
      if (lhs < 0) return lhs;
      if (*p_ == '*') {
        ++p_;
        const int rhs = unary();
        if (rhs < 0) return rhs;
        Node n; n.kind = Kind::Mul; n.a = lhs; n.b = rhs;
        lhs = add(n);
      } else {
        return lhs;
      }
    }
  }
  int unary() {
    skip();
    if (*p_ == '-') {
      ++p_;
      const int a = unary();
      if (a < 0) return a;
      Node n; n.kind = Kind::Neg; n.a = a;
      return add(n);
    }
    return atom();
  }
  int atom() {
    skip();
    if (*p_ == '(') {
      ++p_;
      const int v = sum();
      skip();
      if (*p_ != ')') return fail("expected ')'");
      ++p_;
      return v;
    }
    if ((*p_ >= '0' && *p_ <= '9') || *p_ == '.') {
      char* end = nullptr;
      const double v = strtod(p_, &end);
      if (end == p_) return fail("bad number");
      p_ = end;
      Node n; n.kind = Kind::Const; n.value = v;
      return add(n);
    }
    if ((*p_ >= 'a' && *p_ <= 'z') || (*p_ >= 'A' && *p_ <= 'Z') || *p_ == '_') {
      std::string id;
      while ((*p_ >= 'a' && *p_ <= 'z') || (*p_ >= 'A' && *p_ <= 'Z') || (*p_ >= '0' && *p_ <= '9') || *p_ == '_') id += *p_++;
      skip();
      if (*p_ == '(') {
        ++p_;
        const int a = sum();
        skip();
        if (*p_ != ')') return fail("expected ')' after the argument of " + id);
        ++p_;
        if (a < 0) return a;
        Node n; n.a = a;
        if (id == "selu") n.kind = Kind::Selu;
        else if (id == "relu") n.kind = Kind::Relu;
        else return fail("unknown function " + id);
        return add(n);
      }
      int idx = -1;
      for (size_t i = 0; i < e_.leaves.size(); ++i) if (e_.leaves[i] == id) idx = static_cast<int>(i);
      if (idx < 0) { e_.leaves.push_back(id); idx = static_cast<int>(e_.leaves.size()) - 1; }
      Node n; n.kind = Kind::Leaf; n.leaf = idx;
      return add(n);
    }
    return fail(*p_ ? std::string("unexpected '") + *p_ + "'" : "unexpected end of expression");
  }
  const char* p_;
  Expr& e_;
};

// ------------------------------ code generation ---------------------------
struct TypeInfo { const char* storage; const char* acc; int pack; int bytes; };
const TypeInfo kTypes[3] = {{"unsigned short", "float", 8, 2}, {"float", "float", 4, 4}, {"double", "double", 2, 8}};

std::string lit(double v, const char* acc) {
  std::ostringstream o;
  o.precision(17);
  o << "(" << acc << ")(" << v << (std::string(acc) == "float" ? "" : "") << ")";
  return o.str();
}

// Straight-line forward evaluation: A v<k> = ... for every node.
std::string gen_forward(const Expr& e, const char* acc, const std::string& indent) {
  std::ostringstream o;
  for (size_t k = 0; k < e.nodes.size(); ++k) {
    const Node& n = e.nodes[k];
    o << indent << "const A v" << k << " = ";
    switch (n.kind) {
      case Kind::Leaf: o << "x" << n.leaf; break;
      case Kind::Const: o << lit(n.value, acc); break;
      case Kind::Add: o << "v" << n.a << " + v" << n.b; break;
      case Kind::Sub: o << "v" << n.a << " - v" << n.b; break;
      case Kind::Mul: o << "v" << n.a << " * v" << n.b; break;
      case Kind::Neg: o << "-v" << n.a; break;
      case Kind::Selu: o << "(v" << n.a << " > (A)0 ? SELU_L * v" << n.a << " : SELU_LA * (mp_exp(v" << n.a << ") - (A)1))"; break;
      case Kind::Relu: o << "(v" << n.a << " >= (A)0 ? v" << n.a << " : (A)0)"; break;
    }
    o << ";\n";
  }
  return o.str();
}

// Adjoint sweep in reverse topological order; leaf adjoints end up in g<leaf>.
std::string gen_reverse(const Expr& e, const std::string& indent) {
  std::ostringstream o;
  for (size_t k = 0; k < e.nodes.size(); ++k) o << indent << "A d" << k << " = (A)0;\n";
  o << indent << "d" << e.root << " = gout;\n";
  for (int k = static_cast<int>(e.nodes.size()) - 1; k >= 0; --k) {
    const Node& n = e.nodes[k];
    switch (n.kind) {
      case Kind::Leaf: o << indent << "g" << n.leaf << " += d" << k << ";\n"; break;
      case Kind::Const: break;
      case Kind::Add: o << indent << "d" << n.a << " += d" << k << "; d" << n.b << " += d" << k << ";\n"; break;
      case Kind::Sub: o << indent << "d" << n.a << " += d" << k << "; d" << n.b << " -= d" << k << ";\n"; break;
      case Kind::Mul: o << indent << "d" << n.a << " += d" << k << " * v" << n.b << "; d" << n.b << " += d" << k << " * v" << n.a << ";\n"; break;
      case Kind::Neg: o << indent << "d" << n.a << " -= d" << k << ";\n"; break;
      case Kind::Selu: o << indent << "d" << n.a << " += d" << k << " * (v" << n.a << " > (A)0 ? SELU_L : SELU_LA * mp_exp(v" << n.a << "));\n"; break;
      case Kind::Relu: o << indent << "d" << n.a << " += d" << k << " * (v" << n.a << " >= (A)0 ? (A)1 : (A)0);\n"; break;
    }
  }
  return o.str();
}

constexpr int JIT_THREADS = 512;

std::string gen_source(const Expr& e, int dtype) {
  const TypeInfo& t = kTypes[dtype];
  const int L = static_cast<int>(e.leaves.size());
  const int U = L <= 2 ? 2 : 1;  // 16-byte packs per thread and stream
  std::ostringstream o;
  o << "typedef " << t.storage << " T;\ntypedef " << t.acc << " A;\n";
  o << "#define PN " << t.pack << "\n#define UNROLL " << U << "\n#define THREADS " << JIT_THREADS << "\n";
  o << "#define SELU_L ((A)1.0507009873554805)\n#define SELU_LA ((A)(1.0507009873554805 * 1.6732632423543772))\n";
  o << "typedef unsigned long long u64;\n";
  o << "struct __align__(16) Pack { T v[PN]; };\n";
  o << R"(
__device__ __forceinline__ float mp_exp(float x) { return expf(x); }
__device__ __forceinline__ double mp_exp(double x) { return exp(x); }
__device__ __forceinline__ Pack ld_pack(const T* p, u64 i) {
  union { uint4 u; Pack k; } x;
  const uint4* a = reinterpret_cast<const uint4*>(p) + i;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x.u.x), "=r"(x.u.y), "=r"(x.u.z), "=r"(x.u.w) : "l"(a));
  return x.k;
}
__device__ __forceinline__ void st_pack(T* p, u64 i, const Pack& k) {
  union { uint4 u; Pack k; } x;
  x.k = k;
  uint4* a = reinterpret_cast<uint4*>(p) + i;
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(a), "r"(x.u.x), "r"(x.u.y), "r"(x.u.z), "r"(x.u.w) : "memory");
}
)";
  if (dtype == 0) {
    o << R"(
__device__ __forceinline__ A up(T h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ T down(A f) { T h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
)";
  } else {
    o << "__device__ __forceinline__ A up(T v) { return v; }\n__device__ __forceinline__ T down(A v) { return v; }\n";
  }

  // ---- per-element bodies ---------------------------------------------------
  std::ostringstream fwd_body, rev_body;
  fwd_body << gen_forward(e, t.acc, "      ");
  rev_body << gen_forward(e, t.acc, "      ");
  for (int l = 0; l < L; ++l) rev_body << "      A g" << l << " = (A)0;\n";
  rev_body << gen_reverse(e, "      ");

  // ---- forward kernel ---------------------------------------------------------
  auto leaf_params = [&](const char* prefix, bool is_const) {
    std::ostringstream s;
    for (int l = 0; l < L; ++l) s << (is_const ? "const T* " : "T* ") << prefix << l << ", ";
    return s.str();
  };
  for (int vec = 1; vec >= 0; --vec) {
    o << "extern \"C\" __global__ void __launch_bounds__(THREADS) mp_jit_fwd_" << (vec ? "vec" : "scalar") << "("
      << leaf_params("l", true) << "T* out, u64 n) {\n";
    if (vec) {
      o << "  const u64 nvec = n / PN, trip = (u64)THREADS * UNROLL;\n"
        << "  for (u64 base = blockIdx.x * trip; base < nvec; base += (u64)gridDim.x * trip) {\n";
      for (int l = 0; l < L; ++l) o << "    Pack p" << l << "[UNROLL];\n";
      o << "#pragma unroll\n    for (int u = 0; u < UNROLL; ++u) { const u64 i = base + (u64)u * THREADS + threadIdx.x; if (i < nvec) {";
      for (int l = 0; l < L; ++l) o << " p" << l << "[u] = ld_pack(l" << l << ", i);";
      o << " } }\n#pragma unroll\n    for (int u = 0; u < UNROLL; ++u) { const u64 i = base + (u64)u * THREADS + threadIdx.x; if (i < nvec) {\n"
        << "      Pack r;\n#pragma unroll\n      for (int e = 0; e < PN; ++e) {\n";
      for (int l = 0; l < L; ++l) o << "      const A x" << l << " = up(p" << l << "[u].v[e]);\n";
      o << fwd_body.str() << "      r.v[e] = down(v" << e.root << ");\n      }\n      st_pack(out, i, r);\n    } }\n  }\n"
        << "  if (blockIdx.x == 0) { const u64 i = nvec * PN + threadIdx.x; if (i < n) {\n";
      for (int l = 0; l < L; ++l) o << "      const A x" << l << " = up(l" << l << "[i]);\n";
      o << fwd_body.str() << "      out[i] = down(v" << e.root << ");\n  } }\n}\n";
    } else {
      o << "  for (u64 i = (u64)blockIdx.x * THREADS + threadIdx.x; i < n; i += (u64)gridDim.x * THREADS) {\n";
      for (int l = 0; l < L; ++l) o << "      const A x" << l << " = up(l" << l << "[i]);\n";
      o << fwd_body.str() << "      out[i] = down(v" << e.root << ");\n  }\n}\n";
    }
  }

  // ---- reverse kernel -----------------------------------------------------------
  // gout may be null (upstream gradient of ones = the seed of a sum loss); a null
  // gradient pointer skips that leaf; alpha != 0 blends with the old gradient.
  auto rev_scalar_body = [&](const std::string& idx) {
    std::ostringstream s;
    for (int l = 0; l < L; ++l) s << "      const A x" << l << " = up(l" << l << "[" << idx << "]);\n";
    s << "      const A gout = go ? up(go[" << idx << "]) : (A)1;\n" << rev_body.str();
    for (int l = 0; l < L; ++l)
      s << "      if (g_" << l << ") g_" << l << "[" << idx << "] = down(alpha != (A)0 ? g" << l << " + alpha * up(g_" << l << "["
        << idx << "]) : g" << l << ");\n";
    return s.str();
  };
  for (int vec = 1; vec >= 0; --vec) {
    o << "extern \"C\" __global__ void __launch_bounds__(THREADS) mp_jit_rev_" << (vec ? "vec" : "scalar") << "("
      << leaf_params("l", true) << "const T* go, " << leaf_params("g_", false) << "A alpha, u64 n) {\n";
    if (vec) {
      o << "  const u64 nvec = n / PN, trip = (u64)THREADS * UNROLL;\n"
        << "  for (u64 base = blockIdx.x * trip; base < nvec; base += (u64)gridDim.x * trip) {\n";
      for (int l = 0; l < L; ++l) o << "    Pack p" << l << "[UNROLL];\n";
      o << "    Pack pg[UNROLL];\n";
      o << "#pragma unroll\n    for (int u = 0; u < UNROLL; ++u) { const u64 i = base + (u64)u * THREADS + threadIdx.x; if (i < nvec) {";
      for (int l = 0; l < L; ++l) o << " p" << l << "[u] = ld_pack(l" << l << ", i);";
      o << " if (go) pg[u] = ld_pack(go, i); } }\n"
        << "#pragma unroll\n    for (int u = 0; u < UNROLL; ++u) { const u64 i = base + (u64)u * THREADS + threadIdx.x; if (i < nvec) {\n";
      for (int l = 0; l < L; ++l) o << "      Pack r" << l << ", o" << l << ";\n";
      for (int l = 0; l < L; ++l) o << "      if (alpha != (A)0 && g_" << l << ") o" << l << " = ld_pack(g_" << l << ", i);\n";
      o << "#pragma unroll\n      for (int e = 0; e < PN; ++e) {\n";
      for (int l = 0; l < L; ++l) o << "      const A x" << l << " = up(p" << l << "[u].v[e]);\n";
      o << "      const A gout = go ? up(pg[u].v[e]) : (A)1;\n" << rev_body.str();
      for (int l = 0; l < L; ++l)
        o << "      r" << l << ".v[e] = down(alpha != (A)0 && g_" << l << " ? g" << l << " + alpha * up(o" << l << ".v[e]) : g" << l << ");\n";
      o << "      }\n";
      for (int l = 0; l < L; ++l) o << "      if (g_" << l << ") st_pack(g_" << l << ", i, r" << l << ");\n";
      o << "    } }\n  }\n  if (blockIdx.x == 0) { const u64 i = nvec * PN + threadIdx.x; if (i < n) {\n"
        << rev_scalar_body("i") << "  } }\n}\n";
    } else {
      o << "  for (u64 i = (u64)blockIdx.x * THREADS + threadIdx.x; i < n; i += (u64)gridDim.x * THREADS) {\n"
        << rev_scalar_body("i") << "  }\n}\n";
    }
  }
  return o.str();
}

// ------------------------------ NVRTC / driver ----------------------------
struct Nvrtc {
  void* lib = nullptr;
  int (*createProgram)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*compileProgram)(void*, int, const char* const*) = nullptr;
  int (*getCUBINSize)(void*, size_t*) = nullptr;
  int (*getCUBIN)(void*, char*) = nullptr;
  int (*getProgramLogSize)(void*, size_t*) = nullptr;
  int (*getProgramLog)(void*, char*) = nullptr;
  int (*destroyProgram)(void**) = nullptr;
};

Nvrtc* nvrtc() {
  static Nvrtc api;
  static std::once_flag once;
  std::call_once(once, []() {
    const char* names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so"};
    for (const char* nm : names) {
      api.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (api.lib != nullptr) break;
    }
    if (api.lib == nullptr) return;
#define MP_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.lib, name))
    MP_SYM(createProgram, "nvrtcCreateProgram");
    MP_SYM(compileProgram, "nvrtcCompileProgram");
    MP_SYM(getCUBINSize, "nvrtcGetCUBINSize");
    MP_SYM(getCUBIN, "nvrtcGetCUBIN");
    MP_SYM(getProgramLogSize, "nvrtcGetProgramLogSize");
    MP_SYM(getProgramLog, "nvrtcGetProgramLog");
    MP_SYM(destroyProgram, "nvrtcDestroyProgram");
#undef MP_SYM
  });
  if (api.lib == nullptr || api.createProgram == nullptr || api.getCUBIN == nullptr) MP_FATAL("NVRTC (libnvrtc.so.12) could not be loaded");
  return &api;
}

struct Driver {
  CUresult (*moduleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*moduleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*moduleUnload)(CUmodule) = nullptr;
  CUresult (*launchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
};

Driver* driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, []() {
    auto get = [](const char* name) {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      MP_CUDA_CHECK(cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q));
      if (p == nullptr || q != cudaDriverEntryPointSuccess) MP_FATAL("driver entry point %s is not available", name);
      return p;
    };
    d.moduleLoadData = reinterpret_cast<decltype(d.moduleLoadData)>(get("cuModuleLoadData"));
    d.moduleGetFunction = reinterpret_cast<decltype(d.moduleGetFunction)>(get("cuModuleGetFunction"));
    d.moduleUnload = reinterpret_cast<decltype(d.moduleUnload)>(get("cuModuleUnload"));
    d.launchKernel = reinterpret_cast<decltype(d.launchKernel)>(get("cuLaunchKernel"));
  });
  return &d;
}

struct JitProgram {
  uint64_t magic;
  Expr expr;
  int dtype;
  std::string source;
  CUmodule module = nullptr;
  CUfunction fwd_vec = nullptr, fwd_scalar = nullptr, rev_vec = nullptr, rev_scalar = nullptr;
  int unroll = 1;
  int refs = 1;
};
constexpr uint64_t JIT_MAGIC = 0x4d504a4954505247ull;

std::mutex g_jit_mutex;
std::map<std::tuple<std::string, int, int>, JitProgram*> g_jit_cache;   // (expression, dtype key, device)

JitProgram* as_program(void* h) {
  JitProgram* p = static_cast<JitProgram*>(h);
  if (p == nullptr || p->magic != JIT_MAGIC) MP_FATAL("not a handle from mpJitCompile");
  return p;
}

}  // namespace

// Parse + generate only (no GPU, no NVRTC): returns a malloc'ed C string the
// caller frees with mpJitFreeSource, or NULL after printing the parse error.
extern "C" char* mpJitGenerateSource(const char* expr, uint32_t dtype_key) {
  if (dtype_key > 2) { printf("mpJitGenerateSource: bad dtype key %u\n", dtype_key); return nullptr; }
  Expr e;
  Parser parser(expr, e);
  if (!parser.parse() || e.leaves.empty()) {
    printf("mpJit: cannot parse \"%s\": %s\n", expr, e.error.empty() ? "no tensor operand" : e.error.c_str());
    return nullptr;
  }
  const std::string src = gen_source(e, static_cast<int>(dtype_key));
  char* out = static_cast<char*>(malloc(src.size() + 1));
  memcpy(out, src.c_str(), src.size() + 1);
  return out;
}
extern "C" void mpJitFreeSource(char* s) { free(s); }

extern "C" void* mpJitCompile(const char* expr_text, uint32_t dtype_key) {
  if (dtype_key > 2) { printf("mpJitCompile: bad dtype key %u\n", dtype_key); return nullptr; }
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  // A loaded module belongs to the context of the device it was loaded on: the device is part of the key, so a
  // process that works on several devices gets one module per device.
  int device = -1;
  MP_CUDA_CHECK(cudaFree(nullptr));  // make sure the primary context exists and is current
  MP_CUDA_CHECK(cudaGetDevice(&device));
  const auto key = std::make_tuple(std::string(expr_text), static_cast<int>(dtype_key), device);
  auto it = g_jit_cache.find(key);
  if (it != g_jit_cache.end()) { it->second->refs++; return it->second; }

  JitProgram* prog = new JitProgram();
  prog->magic = JIT_MAGIC;
  prog->dtype = static_cast<int>(dtype_key);
  Parser parser(expr_text, prog->expr);
  if (!parser.parse() || prog->expr.leaves.empty()) {
    printf("mpJitCompile: cannot parse \"%s\": %s\n", expr_text, prog->expr.error.empty() ? "no tensor operand" : prog->expr.error.c_str());
    delete prog;
    return nullptr;
  }
  prog->source = gen_source(prog->expr, prog->dtype);
  prog->unroll = prog->expr.leaves.size() <= 2 ? 2 : 1;

  Nvrtc* rtc = nvrtc();
  void* program = nullptr;
  if (rtc->createProgram(&program, prog->source.c_str(), "mp_jit.cu", 0, nullptr, nullptr) != 0) MP_FATAL("nvrtcCreateProgram failed");
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device"};
  const int rc = rtc->compileProgram(program, 3, opts);
  if (rc != 0) {
    size_t log_size = 0;
    rtc->getProgramLogSize(program, &log_size);
    std::string log(log_size + 1, '\0');
    rtc->getProgramLog(program, &log[0]);
    printf("mpJitCompile: NVRTC failed for \"%s\":\n%s\n", expr_text, log.c_str());
    fflush(stdout);
    exit(EXIT_FAILURE);
  }
  size_t cubin_size = 0;
  if (rtc->getCUBINSize(program, &cubin_size) != 0 || cubin_size == 0) MP_FATAL("nvrtcGetCUBINSize failed");
  std::vector<char> cubin(cubin_size);
  if (rtc->getCUBIN(program, cubin.data()) != 0) MP_FATAL("nvrtcGetCUBIN failed");
  rtc->destroyProgram(&program);

  MP_CUDA_CHECK(cudaFree(nullptr));  // make sure the primary context exists and is current
  Driver* drv = driver();
  MP_CU_CHECK(drv->moduleLoadData(&prog->module, cubin.data()));
  MP_CU_CHECK(drv->moduleGetFunction(&prog->fwd_vec, prog->module, "mp_jit_fwd_vec"));
  MP_CU_CHECK(drv->moduleGetFunction(&prog->fwd_scalar, prog->module, "mp_jit_fwd_scalar"));
  MP_CU_CHECK(drv->moduleGetFunction(&prog->rev_vec, prog->module, "mp_jit_rev_vec"));
  MP_CU_CHECK(drv->moduleGetFunction(&prog->rev_scalar, prog->module, "mp_jit_rev_scalar"));
  g_jit_cache[key] = prog;
  return prog;
}

extern "C" uint32_t mpJitNumLeaves(void* handle) { return static_cast<uint32_t>(as_program(handle)->expr.leaves.size()); }

extern "C" const char* mpJitLeafName(void* handle, uint32_t i) {
  JitProgram* p = as_program(handle);
  return i < p->expr.leaves.size() ? p->expr.leaves[i].c_str() : nullptr;
}

extern "C" void mpJitRelease(void* handle) {
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  JitProgram* p = as_program(handle);
  if (--p->refs > 0) return;
  for (auto it = g_jit_cache.begin(); it != g_jit_cache.end(); ++it)
    if (it->second == p) { g_jit_cache.erase(it); break; }
  if (p->module != nullptr) MP_CU_CHECK(driver()->moduleUnload(p->module));
  p->magic = 0;
  delete p;
}

static unsigned jit_grid(bool vec, len_t n, int pack, int unroll) {
  const size_t per_cta = vec ? static_cast<size_t>(JIT_THREADS) * unroll * pack : JIT_THREADS;
  size_t grid = (n + per_cta - 1) / per_cta;
  if (grid > (1u << 30)) grid = 1u << 30;
  return static_cast<unsigned>(grid < 1 ? 1 : grid);
}

// out[i] = f(leaves[0][i], leaves[1][i], ...), leaves in order of first appearance.
extern "C" void mpJitForward(void* handle, const void* const* leaves, void* out, len_t n, StreamContext ctx) {
  JitProgram* p = as_program(handle);
  if (n == 0) return;
  const int L = static_cast<int>(p->expr.leaves.size());
  bool vec = mp_aligned16(out);
  std::vector<const void*> lp(leaves, leaves + L);
  for (int l = 0; l < L; ++l) vec = vec && mp_aligned16(lp[l]);
  unsigned long long nn = n;
  std::vector<void*> args;
  for (int l = 0; l < L; ++l) args.push_back(&lp[l]);
  args.push_back(&out);
  args.push_back(&nn);
  const unsigned grid = jit_grid(vec, n, kTypes[p->dtype].pack, p->unroll);
  MP_CU_CHECK(driver()->launchKernel(vec ? p->fwd_vec : p->fwd_scalar, grid, 1, 1, JIT_THREADS, 1, 1, 0,
                                     reinterpret_cast<CUstream>(mp_stream(ctx)), args.data(), nullptr));
}

// g_leaves[l] = d out / d leaf_l * g_out + alpha * g_leaves[l]; g_out NULL means
// an upstream gradient of ones; a NULL entry of g_leaves skips that leaf.
extern "C" void mpJitReverse(void* handle, const void* const* leaves, const void* g_out, void* const* g_leaves, double alpha,
                             len_t n, StreamContext ctx) {
  JitProgram* p = as_program(handle);
  if (n == 0) return;
  const int L = static_cast<int>(p->expr.leaves.size());
  bool vec = mp_aligned16(g_out);
  std::vector<const void*> lp(leaves, leaves + L);
  std::vector<void*> gp(g_leaves, g_leaves + L);
  for (int l = 0; l < L; ++l) vec = vec && mp_aligned16(lp[l]) && mp_aligned16(gp[l]);
  unsigned long long nn = n;
  float alpha_f = static_cast<float>(alpha);
  double alpha_d = alpha;
  std::vector<void*> args;
  for (int l = 0; l < L; ++l) args.push_back(&lp[l]);
  args.push_back(&g_out);
  for (int l = 0; l < L; ++l) args.push_back(&gp[l]);
  args.push_back(p->dtype == 2 ? static_cast<void*>(&alpha_d) : static_cast<void*>(&alpha_f));
  args.push_back(&nn);
  const unsigned grid = jit_grid(vec, n, kTypes[p->dtype].pack, p->unroll);
  MP_CU_CHECK(driver()->launchKernel(vec ? p->rev_vec : p->rev_scalar, grid, 1, 1, JIT_THREADS, 1, 1, 0,
                                     reinterpret_cast<CUstream>(mp_stream(ctx)), args.data(), nullptr));
}
