// Implementation of the C++ host mirror (see metaphor.hpp).  Every device
// action goes through the extern "C" boundary of include/*.h.
#include "metaphor.hpp"

#include <cassert>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <set>
#include <string>

namespace mp {

// 3-entry launcher arrays indexed by the dtype key (file_gen.zig:298-328, root.zig:36-43)
#define MP_KERNELS(name) {launch_##name##_r16, launch_##name##_r32, launch_##name##_r64}
namespace kernels {
using Bin = void (*)(const void*, const void*, void*, len_t, StreamContext);
using Un = void (*)(const void*, void*, len_t, StreamContext);
using Sca = void (*)(const void*, double, void*, len_t, StreamContext);
using UnRev = void (*)(const void*, void*, const void*, len_t, StreamContext);
using Blend2 = void (*)(const void*, void*, double, len_t, len_t, StreamContext);
using Gemm = void (*)(const void*, const void*, const double, void*, const double, len_t, len_t, len_t, StreamContext);
static const Bin addition[3] = MP_KERNELS(addition), subtraction[3] = MP_KERNELS(subtraction),
                 hadamard[3] = MP_KERNELS(hadamard), hadamard_reverse[3] = MP_KERNELS(hadamard_reverse);
static const Un negate[3] = MP_KERNELS(negate), relu[3] = MP_KERNELS(relu), selu[3] = MP_KERNELS(selu), copy[3] = MP_KERNELS(copy),
                stepwise[3] = MP_KERNELS(stepwise);
static const Sca translate[3] = MP_KERNELS(translate), dilate[3] = MP_KERNELS(dilate), dilate_reverse[3] = MP_KERNELS(dilate_reverse);
static const UnRev relu_reverse[3] = MP_KERNELS(relu_reverse), selu_reverse[3] = MP_KERNELS(selu_reverse);
static const Blend2 reduce_ij_i[3] = MP_KERNELS(reduce_ij_i), reduce_ij_j[3] = MP_KERNELS(reduce_ij_j),
                    broadcast_i_ij[3] = MP_KERNELS(broadcast_i_ij), broadcast_j_ij[3] = MP_KERNELS(broadcast_j_ij),
                    permutate_ij_ji[3] = MP_KERNELS(permutate_ij_ji);
static const Gemm ip_ij_jk_ik[3] = MP_KERNELS(inner_product_ij_jk_ik), ip_ij_kj_ik[3] = MP_KERNELS(inner_product_ij_kj_ik),
                  ip_ji_jk_ik[3] = MP_KERNELS(inner_product_ji_jk_ik);
using GemmB = void (*)(const void*, const void*, const double, void*, const double, len_t, len_t, len_t, len_t, StreamContext);
static const GemmB ip_bij_bjk_bik[3] = MP_KERNELS(inner_product_bij_bjk_bik), ip_bij_bkj_bik[3] = MP_KERNELS(inner_product_bij_bkj_bik),
                   ip_bji_bjk_bik[3] = MP_KERNELS(inner_product_bji_bjk_bik);
static void (*const permutate[3])(const void*, void*, double, const len_t*, const len_t*, len_t, StreamContext) = MP_KERNELS(permutate);
static void (*const fill[3])(void*, double, len_t, StreamContext) = MP_KERNELS(fill);
static void (*const sequence[3])(void*, double, double, len_t, StreamContext) = MP_KERNELS(sequence);
static void (*const linear[3])(const void*, const void*, const void*, const double, void*, const double, len_t, len_t, len_t,
                               StreamContext) = MP_KERNELS(linear_ij_jk_ik);
static void (*const softmax[3])(const void*, void*, len_t, len_t, StreamContext) = MP_KERNELS(softmax_ij_j);
static void (*const softmax_reverse[3])(const void*, const void*, void*, double, len_t, len_t, StreamContext) = MP_KERNELS(softmax_ij_j_reverse);
static void (*const rmsnorm[3])(const void*, const void*, double, void*, void*, len_t, len_t, StreamContext) = MP_KERNELS(rmsnorm_ij_j);
static void (*const rmsnorm_reverse[3])(const void*, const void*, const void*, const void*, double, void*, void*, double, void*,
                                        len_t, len_t, StreamContext) = MP_KERNELS(rmsnorm_ij_j_reverse);
static void (*const sgd[3])(void*, const void*, double, double, double, len_t, StreamContext) = MP_KERNELS(sgd);
static void (*const momentum[3])(void*, const void*, void*, double, double, double, double, len_t, StreamContext) = MP_KERNELS(momentum);
static void (*const adam[3])(void*, const void*, void*, void*, double, double, double, double, double, len_t, len_t,
                             StreamContext) = MP_KERNELS(adam);
}  // namespace kernels

static inline int dkey(Tensor t) { return static_cast<int>(t.dtype()); }   // graph.zig:205-209

[[noreturn]] static void panic(const char* msg) {
  std::printf("metaphor: %s\n", msg);
  std::fflush(stdout);
  std::exit(EXIT_FAILURE);
}

// ------------------------------ device / stream -------------------------------
namespace device {
void init(unsigned n) { mpInitDevice(n); }
void sync() { mpDeviceSynchronize(); }
void check() { mpCheckLastError(); }
size_t total_memory(unsigned n) { return mpDeviceTotalMemory(n); }
}
namespace stream {
Stream init() { return Stream{mpInitStream()}; }
void deinit(Stream s) { mpDeinitStream(s.context); }
void sync(Stream s) { mpStreamSynchronize(s.context); }
}

// ------------------------------ allocator -------------------------------------
void* TensorAllocator::alloc(size_t bytes, StreamContext ctx) {
  auto it = free_.find(bytes);
  if (it != free_.end() && !it->second.empty()) {
    void* p = it->second.back();
    it->second.pop_back();
    return p;
  }
  void* p = mpMemAlloc(bytes, ctx);
  if (p == nullptr) panic("device allocation failed");
  return p;
}
void TensorAllocator::release(void* p, size_t bytes) { free_[bytes].push_back(p); }
void TensorAllocator::drain(StreamContext ctx) {
  for (auto& kv : free_)
    for (void* p : kv.second) mpMemFree(p, ctx);
  free_.clear();
}
size_t TensorAllocator::cached_blocks() const {
  size_t n = 0;
  for (const auto& kv : free_) n += kv.second.size();
  return n;
}

// ------------------------------ tensor handle ---------------------------------
void* Tensor::data_ptr() const { return ptr->block_of(cls).data[idx]; }
void* Tensor::grad_ptr() const { return ptr->block_of(cls).grad[idx]; }
const std::vector<size_t>& Tensor::sizes() const { return ptr->block_of(cls).sizes[idx]; }
size_t Tensor::len() const { return ptr->block_of(cls).len[idx]; }
Dtype Tensor::dtype() const { return ptr->block_of(cls).dtype[idx]; }
StreamContext Tensor::context() const { return ptr->stream.context; }
void Tensor::detach() const {
  assert(cls == Class::hid);
  ptr->node_block.attached[idx] = false;
}
void Tensor::free() const { ptr->free_tensor(*this); }

void Tensor::reverse(ReverseCleanup cleanup) const {
  if (grad_ptr() == nullptr) {
    // no loss was applied: the derivative with respect to self is 1 (graph.zig:112-117)
    enable_gradient(*this);
    kernels::fill[dkey(*this)](grad_ptr(), 1.0, len(), context());
  }
  if (cls != Class::hid) return;
  ptr->reverse(idx, cleanup);
}

static std::vector<double> to_host(const void* dptr, size_t n, Dtype dt, StreamContext ctx) {
  std::vector<double> out(n);
  if (n == 0 || dptr == nullptr) return out;
  std::vector<unsigned char> raw(n * dtype_size(dt));
  mpMemcpyDtoH(raw.data(), dptr, raw.size(), ctx);
  mpStreamSynchronize(ctx);   // the reference reads without waiting (utils.zig:182-218)
  for (size_t i = 0; i < n; ++i) {
    if (dt == Dtype::r32) { float f; std::memcpy(&f, raw.data() + 4 * i, 4); out[i] = f; }
    else if (dt == Dtype::r64) { double d; std::memcpy(&d, raw.data() + 8 * i, 8); out[i] = d; }
    else {
      uint16_t h; std::memcpy(&h, raw.data() + 2 * i, 2);
      const int s = h >> 15, e = (h >> 10) & 31, m = h & 1023;
      double v = e == 0 ? std::ldexp(static_cast<double>(m), -24)
                        : (e == 31 ? (m ? std::numeric_limits<double>::quiet_NaN() : std::numeric_limits<double>::infinity())
                                   : std::ldexp(static_cast<double>(m + 1024), e - 25));
      out[i] = s ? -v : v;
    }
  }
  return out;
}
std::vector<double> Tensor::native() const { return to_host(data_ptr(), len(), dtype(), context()); }
std::vector<double> Tensor::native_grad() const { return to_host(grad_ptr(), grad_ptr() ? len() : 0, dtype(), context()); }

// ------------------------------ graph ------------------------------------------
Graph* Graph::init(GraphConfig cfg) {
  Graph* g = new Graph();
  g->mode = cfg.mode;
  g->stream = cfg.stream;
  return g;
}

void Graph::deinit() {
  reset(ResetGroup::node, ResetComponent::all);
  reset(ResetGroup::leaf, ResetComponent::all);
  if (scratch_ != nullptr) mpMemFree(scratch_, stream.context);
  tensor_allocator.drain(stream.context);
  mpStreamSynchronize(stream.context);
  delete this;
}

Tensor Graph::tensor(const TensorConfig& cfg) {
  Block& b = block_of(cfg.cls);
  size_t n = 1;
  for (size_t s : cfg.sizes) n *= s;
  if (cfg.sizes.empty()) n = 0;
  b.data.push_back(n ? tensor_allocator.alloc(n * dtype_size(cfg.dtype), stream.context) : nullptr);
  b.grad.push_back(nullptr);
  b.len.push_back(n);
  b.sizes.push_back(cfg.sizes);
  b.dtype.push_back(cfg.dtype);
  b.cls.push_back(cfg.cls);
  if (cfg.cls == Class::hid) {
    b.deps.push_back(0);
    b.attached.push_back(true);
    b.has_op.push_back(false);
    b.op_reverse.push_back(nullptr);
    b.op_derive.push_back(nullptr);
    b.op_args.emplace_back();
  }
  return Tensor{this, cfg.cls, b.data.size() - 1};
}

void Graph::free_gradient(Tensor t) {
  Block& b = block_of(t.cls);
  if (b.grad[t.idx] != nullptr) {
    tensor_allocator.release(b.grad[t.idx], b.len[t.idx] * dtype_size(b.dtype[t.idx]));
    b.grad[t.idx] = nullptr;
  }
}

void Graph::free_tensor(Tensor t) {
  Block& b = block_of(t.cls);
  free_gradient(t);
  if (b.data[t.idx] != nullptr) {
    tensor_allocator.release(b.data[t.idx], b.len[t.idx] * dtype_size(b.dtype[t.idx]));
    b.data[t.idx] = nullptr;
  }
  b.len[t.idx] = 0;
}

static std::string weight_path(const std::string& dir, const std::string& prefix, size_t k) {
  return dir + "/" + prefix + "_" + std::to_string(k);
}
void Graph::save(const std::string& dir, const std::string& prefix) {
  std::vector<unsigned char> host;
  size_t k = 0;
  for (size_t i = 0; i < leaf_block.data.size(); ++i) {
    if (leaf_block.cls[i] != Class::wgt) continue;
    const size_t bytes = leaf_block.len[i] * dtype_size(leaf_block.dtype[i]);
    if (bytes == 0) panic("Graph.save: a weight has no data");
    host.resize(bytes);
    mpMemcpyDtoH(host.data(), leaf_block.data[i], bytes, stream.context);
    mpStreamSynchronize(stream.context);
    std::FILE* f = std::fopen(weight_path(dir, prefix, k).c_str(), "wb");
    if (f == nullptr || std::fwrite(host.data(), 1, bytes, f) != bytes) panic("Failed to save tensor data.");
    std::fclose(f);
    ++k;
  }
}
void Graph::load(const std::string& dir, const std::string& prefix) {
  std::vector<unsigned char> host;
  size_t k = 0;
  for (size_t i = 0; i < leaf_block.data.size(); ++i) {
    if (leaf_block.cls[i] != Class::wgt) continue;
    const size_t bytes = leaf_block.len[i] * dtype_size(leaf_block.dtype[i]);
    if (bytes == 0) panic("Graph.load: a weight has no data");
    host.resize(bytes + 1);
    std::FILE* f = std::fopen(weight_path(dir, prefix, k).c_str(), "rb");
    if (f == nullptr) panic("Failed to load tensor data.");
    const size_t got = std::fread(host.data(), 1, bytes + 1, f);   // one byte more: a longer file is also a mismatch
    std::fclose(f);
    if (got != bytes) panic("Failed to load tensor data (wrong byte count).");
    mpMemcpyHtoD(leaf_block.data[i], host.data(), bytes, stream.context);
    mpStreamSynchronize(stream.context);
    ++k;
  }
}

void Graph::reset(ResetGroup group, ResetComponent component) {
  Block& b = group == ResetGroup::node ? node_block : leaf_block;
  const Class c = group == ResetGroup::node ? Class::hid : Class::inp;
  if (component == ResetComponent::grd) {
    for (size_t i = 0; i < b.grad.size(); ++i) {
      free_gradient(Tensor{this, c, i});
      if (group == ResetGroup::node) b.deps[i] = 0;
    }
  } else {
    mpStreamSynchronize(stream.context);
    for (size_t i = 0; i < b.data.size(); ++i) free_tensor(Tensor{this, c, i});
    b = Block();
  }
}

void* Graph::scratch(size_t bytes) {
  if (bytes > scratch_bytes_) {
    if (scratch_ != nullptr) mpMemFree(scratch_, stream.context);
    scratch_ = mpMemAlloc(bytes, stream.context);
    scratch_bytes_ = bytes;
  }
  return scratch_;
}

void enable_gradient(Tensor t) {
  Graph* g = t.ptr;
  Graph::Block& b = g->block_of(t.cls);
  if (b.grad[t.idx] == nullptr && b.len[t.idx] > 0) {
    b.grad[t.idx] = g->tensor_allocator.alloc(b.len[t.idx] * dtype_size(b.dtype[t.idx]), g->stream.context);
    kernels::fill[dkey(t)](b.grad[t.idx], 0.0, b.len[t.idx], g->stream.context);   // gradients start at zero
  }
}

void attach_op(ReverseFn fn, Tensor out, const std::vector<OpDatum>& args, DeriveFn derive_fn) {
  assert(out.cls == Class::hid);
  Graph::Block& nb = out.ptr->node_block;
  nb.has_op[out.idx] = true;
  nb.op_reverse[out.idx] = fn;
  nb.op_derive[out.idx] = derive_fn;
  nb.op_args[out.idx] = args;
  for (size_t i = 0; i + 1 < args.size(); ++i) {   // the last argument is the output
    if (args[i].kind != OpDatum::tensor_k || args[i].tensor.cls != Class::hid) continue;
    nb.deps[args[i].tensor.idx] += 1;
  }
}

std::optional<OpDatum> derive(Tensor x, Tensor wrt) {
  if (x.cls != Class::hid) return x.same(wrt) ? std::optional<OpDatum>(OpDatum::of(1.0)) : std::nullopt;
  Graph::Block& nb = x.ptr->node_block;
  if (!nb.has_op[x.idx]) return std::nullopt;
  if (nb.op_derive[x.idx] == nullptr) panic("derive: an operator on the path has no element-wise derivative");
  return nb.op_derive[x.idx](nb.op_args[x.idx], wrt);
}

std::optional<Tensor> Tensor::derive(Tensor wrt) const {
  if (ptr->mode == Mode::eval) return std::nullopt;
  auto constant = [&](double value) {
    Tensor dx = wrt.ptr->tensor({Class::hid, dtype(), sizes()});
    algo::fill(dx, value);
    return dx;
  };
  if (same(wrt)) return constant(1.0);
  if (cls != Class::hid) return std::nullopt;
  const std::optional<OpDatum> d = mp::derive(*this, wrt);
  if (!d) return std::nullopt;
  if (d->kind == OpDatum::scalar_k) return constant(d->scalar);   // constant-valued tensor
  return d->tensor;
}

void Graph::reverse(size_t idx, ReverseCleanup cleanup) {
  assert(mode != Mode::eval);
  if (node_block.data.empty()) return;
  std::vector<size_t> node_stack{idx}, free_stack;
  while (!node_stack.empty()) {
    const size_t last = node_stack.back();
    node_stack.pop_back();
    if (!node_block.has_op[last]) continue;
    if (cleanup == ReverseCleanup::free) free_stack.push_back(last);
    const std::vector<OpDatum> args = node_block.op_args[last];
    node_block.op_reverse[last](args);
    for (const OpDatum& a : args) {
      if (a.kind != OpDatum::tensor_k) continue;
      if (a.tensor.cls != Class::hid || a.tensor.idx == last) continue;
      if (!node_block.attached[a.tensor.idx]) continue;
      if (--node_block.deps[a.tensor.idx] == 0) node_stack.push_back(a.tensor.idx);
    }
    node_block.has_op[last] = false;   // the dependency is consumed
    node_block.op_args[last].clear();
  }
  if (cleanup == ReverseCleanup::free) {
    mpStreamSynchronize(stream.context);
    for (size_t n : free_stack) free_tensor(Tensor{this, Class::hid, n});
  }
}

// ------------------------------ algo --------------------------------------------
namespace algo {
void fill(Tensor x, double value) { kernels::fill[dkey(x)](x.data_ptr(), value, x.len(), x.context()); }
void sequence(Tensor x, double init, double step) { kernels::sequence[dkey(x)](x.data_ptr(), init, step, x.len(), x.context()); }
void copy(Tensor src, Tensor dst) {
  assert(src.len() == dst.len() && src.dtype() == dst.dtype());
  kernels::copy[dkey(src)](src.data_ptr(), dst.data_ptr(), src.len(), src.context());
}
}

// ------------------------------ ops ----------------------------------------------
namespace ops {

static Tensor hidden_like(Graph* g, Tensor x) { return g->tensor({Class::hid, x.dtype(), x.sizes()}); }
static void check_same(Tensor x, Tensor y) {
  if (x.dtype() != y.dtype() || x.sizes() != y.sizes()) panic("operands differ in dtype or shape");
}

// forward-mode derivatives, defined after the ops they compose
static std::optional<OpDatum> add_derive(const std::vector<OpDatum>&, Tensor), sub_derive(const std::vector<OpDatum>&, Tensor),
    hadamard_derive(const std::vector<OpDatum>&, Tensor), negate_derive(const std::vector<OpDatum>&, Tensor),
    translate_derive(const std::vector<OpDatum>&, Tensor), dilate_derive(const std::vector<OpDatum>&, Tensor),
    relu_derive(const std::vector<OpDatum>&, Tensor), selu_derive(const std::vector<OpDatum>&, Tensor);

// --- add / sub / hadamard (addition.zig:27-82, subtraction.zig, hadamard.zig) ---
static void add_reverse(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[1].tensor, z = a[2].tensor;
  enable_gradient(x); enable_gradient(y);
  const int k = dkey(z);
  kernels::addition[k](z.grad_ptr(), x.grad_ptr(), x.grad_ptr(), x.len(), x.context());   // g_x = g_z + g_x
  kernels::addition[k](z.grad_ptr(), y.grad_ptr(), y.grad_ptr(), y.len(), y.context());
}
Tensor add(Tensor x, Tensor y) {
  check_same(x, y);
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::addition[dkey(z)](x.data_ptr(), y.data_ptr(), z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(add_reverse, z, {OpDatum::of(x), OpDatum::of(y), OpDatum::of(z)}, add_derive);
  return z;
}
static void sub_reverse(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[1].tensor, z = a[2].tensor;
  enable_gradient(x); enable_gradient(y);
  const int k = dkey(z);
  kernels::addition[k](z.grad_ptr(), x.grad_ptr(), x.grad_ptr(), x.len(), x.context());
  kernels::subtraction[k](y.grad_ptr(), z.grad_ptr(), y.grad_ptr(), y.len(), y.context());   // g_y = g_y - g_z
}
Tensor sub(Tensor x, Tensor y) {
  check_same(x, y);
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::subtraction[dkey(z)](x.data_ptr(), y.data_ptr(), z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(sub_reverse, z, {OpDatum::of(x), OpDatum::of(y), OpDatum::of(z)}, sub_derive);
  return z;
}
static void hadamard_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[1].tensor, z = a[2].tensor;
  enable_gradient(x); enable_gradient(y);
  const int k = dkey(z);
  kernels::hadamard_reverse[k](z.grad_ptr(), y.data_ptr(), x.grad_ptr(), x.len(), x.context());   // g_x += g_z*y
  kernels::hadamard_reverse[k](z.grad_ptr(), x.data_ptr(), y.grad_ptr(), y.len(), y.context());
}
Tensor hadamard(Tensor x, Tensor y) {
  check_same(x, y);
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::hadamard[dkey(z)](x.data_ptr(), y.data_ptr(), z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(hadamard_rev, z, {OpDatum::of(x), OpDatum::of(y), OpDatum::of(z)}, hadamard_derive);
  return z;
}

// --- unary / scalar ops (negate.zig, translate.zig, dilate.zig, relu.zig) ---
static void negate_reverse(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, z = a[1].tensor;
  enable_gradient(x);
  kernels::subtraction[dkey(z)](x.grad_ptr(), z.grad_ptr(), x.grad_ptr(), x.len(), x.context());
}
Tensor negate(Tensor x) {
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::negate[dkey(z)](x.data_ptr(), z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(negate_reverse, z, {OpDatum::of(x), OpDatum::of(z)}, negate_derive);
  return z;
}
static void translate_reverse(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, z = a[2].tensor;
  enable_gradient(x);
  kernels::addition[dkey(z)](z.grad_ptr(), x.grad_ptr(), x.grad_ptr(), x.len(), x.context());
}
Tensor translate(Tensor x, double value) {
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::translate[dkey(z)](x.data_ptr(), value, z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(translate_reverse, z, {OpDatum::of(x), OpDatum::of(value), OpDatum::of(z)}, translate_derive);
  return z;
}
static void dilate_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, z = a[2].tensor;
  enable_gradient(x);
  kernels::dilate_reverse[dkey(z)](z.grad_ptr(), a[1].scalar, x.grad_ptr(), x.len(), x.context());
}
Tensor dilate(Tensor x, double value) {
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::dilate[dkey(z)](x.data_ptr(), value, z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(dilate_rev, z, {OpDatum::of(x), OpDatum::of(value), OpDatum::of(z)}, dilate_derive);
  return z;
}
static void relu_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, z = a[1].tensor;
  enable_gradient(x);
  kernels::relu_reverse[dkey(z)](x.data_ptr(), x.grad_ptr(), z.grad_ptr(), x.len(), x.context());
}
Tensor relu(Tensor x) {
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::relu[dkey(z)](x.data_ptr(), z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(relu_rev, z, {OpDatum::of(x), OpDatum::of(z)}, relu_derive);
  return z;
}
static void selu_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, z = a[1].tensor;
  enable_gradient(x);
  kernels::selu_reverse[dkey(z)](x.data_ptr(), x.grad_ptr(), z.grad_ptr(), x.len(), x.context());
}
Tensor selu(Tensor x) {
  Graph* g = x.ptr;
  Tensor z = hidden_like(g, x);
  kernels::selu[dkey(z)](x.data_ptr(), z.data_ptr(), z.len(), z.context());
  if (g->mode == Mode::train) attach_op(selu_rev, z, {OpDatum::of(x), OpDatum::of(z)}, selu_derive);
  return z;
}

// --- forward-mode derivatives of the element-wise ops (the `derive` of addition.zig:84-116, subtraction.zig:85-124,
// hadamard.zig:85-160, negate.zig:55-61, translate.zig:60-62, dilate.zig:60-67, relu.zig:56-58).  The value algebra
// is the reference's: a derivative is nothing (no dependence), a scalar (constant) or a tensor; scalars 0 and 1 are
// folded away.  relu's derivative here applies the chain rule (the reference returns step(x) alone).
using Deriv = std::optional<OpDatum>;
static bool is_scalar(const Deriv& d) { return d && d->kind == OpDatum::scalar_k; }
static Deriv d_negate(Graph* g, const Deriv& d) {
  (void)g;
  if (!d) return d;
  if (is_scalar(d)) return OpDatum::of(-d->scalar);
  return OpDatum::of(negate(d->tensor));
}
static Deriv d_add(const Deriv& a, const Deriv& b) {
  if (!a) return b;
  if (!b) return a;
  if (is_scalar(a) && is_scalar(b)) return OpDatum::of(a->scalar + b->scalar);
  if (is_scalar(a)) return a->scalar == 0.0 ? b : Deriv(OpDatum::of(translate(b->tensor, a->scalar)));
  if (is_scalar(b)) return b->scalar == 0.0 ? a : Deriv(OpDatum::of(translate(a->tensor, b->scalar)));
  return OpDatum::of(add(a->tensor, b->tensor));
}
// d * t for a derivative d and a tensor factor t
static Deriv d_times(const Deriv& d, Tensor t) {
  if (!d) return d;
  if (is_scalar(d)) {
    if (d->scalar == 0.0) return std::nullopt;
    if (d->scalar == 1.0) return OpDatum::of(t);
    return OpDatum::of(dilate(t, d->scalar));
  }
  return OpDatum::of(hadamard(t, d->tensor));
}
static Deriv add_derive(const std::vector<OpDatum>& a, Tensor wrt) { return d_add(derive(a[0].tensor, wrt), derive(a[1].tensor, wrt)); }
static Deriv sub_derive(const std::vector<OpDatum>& a, Tensor wrt) {
  return d_add(derive(a[0].tensor, wrt), d_negate(wrt.ptr, derive(a[1].tensor, wrt)));
}
static Deriv hadamard_derive(const std::vector<OpDatum>& a, Tensor wrt) {
  Tensor x = a[0].tensor, y = a[1].tensor;
  if (x.same(wrt) && y.same(wrt)) return OpDatum::of(dilate(x, 2.0));   // power rule (hadamard.zig:87-90)
  return d_add(d_times(derive(x, wrt), y), d_times(derive(y, wrt), x));  // x'y + xy'
}
static Deriv negate_derive(const std::vector<OpDatum>& a, Tensor wrt) { return d_negate(wrt.ptr, derive(a[0].tensor, wrt)); }
static Deriv translate_derive(const std::vector<OpDatum>& a, Tensor wrt) { return derive(a[0].tensor, wrt); }
static Deriv dilate_derive(const std::vector<OpDatum>& a, Tensor wrt) {
  const Deriv d = derive(a[0].tensor, wrt);
  if (!d) return d;
  if (is_scalar(d)) return OpDatum::of(d->scalar * a[1].scalar);
  return OpDatum::of(dilate(d->tensor, a[1].scalar));
}
static Deriv relu_derive(const std::vector<OpDatum>& a, Tensor wrt) {
  Tensor x = a[0].tensor;
  const Deriv d = derive(x, wrt);
  if (!d) return d;
  Tensor step = hidden_like(x.ptr, x);
  kernels::stepwise[dkey(x)](x.data_ptr(), step.data_ptr(), x.len(), x.context());   // 1 where x >= 0 (stepwise.zig:21)
  return d_times(d, step);
}
static Deriv selu_derive(const std::vector<OpDatum>& a, Tensor wrt) {
  Tensor x = a[0].tensor;
  const Deriv d = derive(x, wrt);
  if (!d) return d;
  // selu'(x) through the reverse kernel: slope = 0 + 1 * selu'(x)
  Tensor slope = hidden_like(x.ptr, x), ones = hidden_like(x.ptr, x);
  algo::fill(slope, 0.0); algo::fill(ones, 1.0);
  kernels::selu_reverse[dkey(x)](x.data_ptr(), slope.data_ptr(), ones.data_ptr(), x.len(), x.context());
  return d_times(d, slope);
}

// --- reduce / broadcast (reduce.zig:98-182, broadcast.zig:96-183; grammar expression_parsing.zig:343-380) ---
// "ijk->ik" sums over the indices missing on the right; the broadcast "ik->ijk" is its transpose (NOTES.md:27-35).
// Any rank up to 6: trailing reduced indices are a row sum, leading ones a column sum of the flattened matrix
// (the reference's rank-2 kernels); any other pattern first moves the reduced indices to the end with the general
// permutation (through the stream's scratch buffer).
struct ReducePlan {
  std::vector<size_t> sizes, perm, moved_sizes, inverse, out_sizes;   // perm: kept indices in output order, then the reduced ones
  bool trailing = false, leading = false;
  size_t kept = 1, red = 1;
};
static ReducePlan plan_reduce(const std::string& expr, const std::vector<size_t>& sizes, const char* who) {
  const size_t arrow = expr.find("->");
  if (arrow == std::string::npos) panic("reduce / broadcast: expression has no \"->\"");
  const std::string lhs = expr.substr(0, arrow), rhs = expr.substr(arrow + 2);
  if (lhs.size() != sizes.size() || lhs.size() > 6 || lhs.empty()) { std::printf("%s: ", who); panic("the expression's rank differs from the tensor's"); }
  if (rhs.size() > lhs.size()) { std::printf("%s: ", who); panic("found extra indices in the expression"); }
  ReducePlan p;
  p.sizes = sizes;
  p.perm.assign(lhs.size(), 0);
  p.out_sizes.assign(rhs.size(), 0);
  size_t n_red = 0;
  for (size_t i = 0; i < lhs.size(); ++i) {
    if (lhs[i] < 'a' || lhs[i] > 'z' || lhs.find(lhs[i]) != i) panic("reduce / broadcast: indices must be distinct lower case characters");
    const size_t j = rhs.find(lhs[i]);
    if (j == std::string::npos) { p.perm[i] = rhs.size() + n_red++; p.red *= sizes[i]; }
    else { p.perm[i] = j; p.out_sizes[j] = sizes[i]; p.kept *= sizes[i]; }
  }
  for (size_t j = 0; j < rhs.size(); ++j)
    if (lhs.find(rhs[j]) == std::string::npos || rhs.find(rhs[j]) != j) panic("reduce / broadcast: the short side must be a subset of the long side");
  if (p.out_sizes.empty()) p.out_sizes = {1};   // full reduction
  p.trailing = true;
  for (size_t i = 0; i < lhs.size(); ++i) p.trailing = p.trailing && p.perm[i] == i;
  p.leading = !p.trailing;
  for (size_t i = 0; i < lhs.size(); ++i)   // reduced indices first, kept ones in order behind them
    p.leading = p.leading && p.perm[i] == (i < n_red ? rhs.size() + i : i - n_red);
  p.moved_sizes.assign(lhs.size(), 0);
  p.inverse.assign(lhs.size(), 0);
  for (size_t i = 0; i < lhs.size(); ++i) { p.moved_sizes[p.perm[i]] = sizes[i]; p.inverse[p.perm[i]] = i; }
  return p;
}
static void call_permutate(int key, const void* src, void* dst, double alpha, const std::vector<size_t>& sizes,
                           const std::vector<size_t>& perm, StreamContext ctx) {
  len_t sz[8], pm[8];
  for (size_t i = 0; i < sizes.size(); ++i) { sz[i] = sizes[i]; pm[i] = perm[i]; }
  kernels::permutate[key](src, dst, alpha, sz, pm, sizes.size(), ctx);
}
// small = sum over the reduced indices of big (+ alpha * small)
static void run_reduce(Graph* g, int key, size_t elem, const ReducePlan& p, const void* big, void* small, double alpha, StreamContext ctx) {
  if (p.trailing) { kernels::reduce_ij_i[key](big, small, alpha, p.kept, p.red, ctx); return; }
  if (p.leading) { kernels::reduce_ij_j[key](big, small, alpha, p.red, p.kept, ctx); return; }
  void* tmp = g->scratch(p.kept * p.red * elem);
  call_permutate(key, big, tmp, 0.0, p.sizes, p.perm, ctx);
  kernels::reduce_ij_i[key](tmp, small, alpha, p.kept, p.red, ctx);
}
// big = small repeated along the reduced indices (+ alpha * big)
static void run_broadcast(Graph* g, int key, size_t elem, const ReducePlan& p, const void* small, void* big, double alpha, StreamContext ctx) {
  if (p.trailing) { kernels::broadcast_i_ij[key](small, big, alpha, p.kept, p.red, ctx); return; }
  if (p.leading) { kernels::broadcast_j_ij[key](small, big, alpha, p.red, p.kept, ctx); return; }
  void* tmp = g->scratch(p.kept * p.red * elem);
  kernels::broadcast_i_ij[key](small, tmp, 0.0, p.kept, p.red, ctx);
  call_permutate(key, tmp, big, alpha, p.moved_sizes, p.inverse, ctx);
}
static void reduce_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[2].tensor;
  enable_gradient(x);
  const ReducePlan p = plan_reduce(a[1].expr, x.sizes(), "reduce");
  run_broadcast(x.ptr, dkey(y), dtype_size(y.dtype()), p, y.grad_ptr(), x.grad_ptr(), 1.0, x.context());
}
Tensor reduce(Tensor x, const std::string& expr) {
  Graph* g = x.ptr;
  const ReducePlan p = plan_reduce(expr, x.sizes(), "reduce");
  Tensor y = g->tensor({Class::hid, x.dtype(), p.out_sizes});
  run_reduce(g, dkey(y), dtype_size(y.dtype()), p, x.data_ptr(), y.data_ptr(), 0.0, y.context());
  if (g->mode == Mode::train) attach_op(reduce_rev, y, {OpDatum::of(x), OpDatum::of(expr), OpDatum::of(y)});
  return y;
}
// "i->ij": the plan is the one of the opposite reduction "ij->i" over the target's sizes
static std::string flipped(const std::string& expr) {
  const size_t arrow = expr.find("->");
  if (arrow == std::string::npos) panic("broadcast: expression has no \"->\"");
  return expr.substr(arrow + 2) + "->" + expr.substr(0, arrow);
}
static void broadcast_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[2].tensor;
  enable_gradient(x);
  const ReducePlan p = plan_reduce(flipped(a[1].expr), y.sizes(), "broadcast");
  run_reduce(x.ptr, dkey(y), dtype_size(y.dtype()), p, y.grad_ptr(), x.grad_ptr(), 1.0, x.context());
}
Tensor broadcast(Tensor x, const std::vector<size_t>& sizes, const std::string& expr) {
  Graph* g = x.ptr;
  const ReducePlan p = plan_reduce(flipped(expr), sizes, "broadcast");
  if (x.sizes() != p.out_sizes) panic("broadcast: the source's sizes differ from the target's sizes at its indices");
  Tensor y = g->tensor({Class::hid, x.dtype(), sizes});
  run_broadcast(g, dkey(y), dtype_size(y.dtype()), p, x.data_ptr(), y.data_ptr(), 0.0, y.context());
  if (g->mode == Mode::train) attach_op(broadcast_rev, y, {OpDatum::of(x), OpDatum::of(expr), OpDatum::of(y)});
  return y;
}

// --- permutate (permutate.zig:39-104; grammar expression_parsing.zig:205-255) ---
// "ijk->kij": both sides lower-case letters, each used once, the right side a permutation of the left.
// perm[i] = position of the i-th left letter on the right (`permutateSizes`).
std::vector<size_t> permutation_of(const std::string& expr) {
  const size_t arrow = expr.find("->");
  if (arrow == std::string::npos) panic("permutate: expression has no \"->\"");
  const std::string lhs = expr.substr(0, arrow), rhs = expr.substr(arrow + 2);
  if (lhs.empty() || lhs.size() != rhs.size()) panic("permutate: both sides must name the same indices");
  std::vector<size_t> perm(lhs.size());
  for (size_t i = 0; i < lhs.size(); ++i) {
    if (lhs[i] < 'a' || lhs[i] > 'z' || rhs[i] < 'a' || rhs[i] > 'z') panic("permutate: tensor indices must be lower case characters");
    if (lhs.find(lhs[i]) != i || rhs.find(rhs[i]) != i) panic("permutate: an index appears twice");
    const size_t j = rhs.find(lhs[i]);
    if (j == std::string::npos) panic("permutate: left and right operands must be permutations of each other");
    perm[i] = j;
  }
  return perm;
}
static void launch_permutate(Tensor src_t, const void* src, void* dst, double alpha, const std::vector<size_t>& sizes,
                             const std::vector<size_t>& perm) {
  len_t sz[8], pm[8];
  if (sizes.size() > 6) panic("permutate: rank above 6");
  for (size_t i = 0; i < sizes.size(); ++i) { sz[i] = sizes[i]; pm[i] = perm[i]; }
  kernels::permutate[dkey(src_t)](src, dst, alpha, sz, pm, sizes.size(), src_t.context());
}
// the gradient flows back through the inverse permutation (for "ij->ji" that is the permutation itself, the
// only case permutate.zig:62-72 handles), accumulated into x.grad
static void permutate_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[2].tensor;   // the output is the last argument (attach_op counts the others as dependencies)
  enable_gradient(x);
  const std::vector<size_t> perm = permutation_of(a[1].expr);
  if (perm.size() == 2 && perm[0] == 1) {
    const auto& s = y.sizes();
    kernels::permutate_ij_ji[dkey(y)](y.grad_ptr(), x.grad_ptr(), 1.0, s[0], s[1], x.context());
    return;
  }
  std::vector<size_t> inverse(perm.size());
  for (size_t i = 0; i < perm.size(); ++i) inverse[perm[i]] = i;
  launch_permutate(y, y.grad_ptr(), x.grad_ptr(), 1.0, y.sizes(), inverse);
}
// every output element is one input element: the element-wise derivative is the permuted derivative of the input
// (permutate.zig:71-73 panics here)
static std::optional<OpDatum> permutate_derive(const std::vector<OpDatum>& a, Tensor wrt) {
  const std::optional<OpDatum> d = derive(a[0].tensor, wrt);
  if (!d || d->kind == OpDatum::scalar_k) return d;
  return OpDatum::of(permutate(d->tensor, a[1].expr));
}
Tensor permutate(Tensor x, const std::string& expr) {
  const std::vector<size_t> perm = permutation_of(expr);
  const auto& s = x.sizes();
  if (perm.size() != s.size()) panic("permutate: the expression's rank differs from the tensor's");
  Graph* g = x.ptr;
  std::vector<size_t> out(s.size());
  for (size_t i = 0; i < s.size(); ++i) out[perm[i]] = s[i];
  Tensor y = g->tensor({Class::hid, x.dtype(), out});
  if (perm.size() == 2 && perm[0] == 1) kernels::permutate_ij_ji[dkey(y)](x.data_ptr(), y.data_ptr(), 0.0, s[0], s[1], y.context());
  else launch_permutate(x, x.data_ptr(), y.data_ptr(), 0.0, s, perm);
  if (g->mode == Mode::train) attach_op(permutate_rev, y, {OpDatum::of(x), OpDatum::of(expr), OpDatum::of(y)}, permutate_derive);
  return y;
}

// --- inner product (inner_product.zig:116-122 expression map, :163-419 variants and reverses) ---
// Logical shape of the contraction "lhs,rhs->out" as C[m,k] = op(A)[m,n] op(B)[n,k].
struct Contraction { len_t m, n, k; int kind; len_t batch; };   // kind: 0 = ij,jk  1 = ij,kj  2 = ji,jk;  batch 0 = rank-2 form
// A leading index shared by all three operands is a batch index ("bij,bjk->bik"); written as '_' it is optional
// ("_ij,_jk->_ik", NOTES.md:18): present for rank-3 operands, absent for rank-2 ones.
static Contraction parse_contraction(Tensor x, Tensor y, const std::string& expr, std::vector<size_t>& out_sizes) {
  const auto& xs = x.sizes(); const auto& ys = y.sizes();
  std::string e = expr;
  len_t batch = 0;
  size_t o = 0;   // offset of the matrix dimensions in the operands' sizes
  const size_t comma = e.find(','), arrow = e.find("->");
  if (comma != std::string::npos && arrow != std::string::npos && comma == 3 && arrow == 7 && e.size() == 12 && e[0] == e[4] &&
      e[0] == e[9] && e.find(e[0], 1) == 4) {
    const bool optional = e[0] == '_';
    e = e.substr(1, 2) + "," + e.substr(5, 2) + "->" + e.substr(10, 2);
    if (!(optional && xs.size() == 2 && ys.size() == 2)) {
      if (xs.size() != 3 || ys.size() != 3) panic("inner_product: a batched expression needs rank-3 operands");
      if (xs[0] != ys[0]) panic("inner_product: batch sizes differ");
      batch = xs[0];
      o = 1;
    }
  }
  Contraction c{};
  if (e == "ij,jk->ik") { c = {xs[o], xs[o + 1], ys[o + 1], 0, batch}; if (xs[o + 1] != ys[o]) panic("inner_product: inner sizes differ"); out_sizes = {xs[o], ys[o + 1]}; }
  else if (e == "ij,kj->ik") { c = {xs[o], xs[o + 1], ys[o], 1, batch}; if (xs[o + 1] != ys[o + 1]) panic("inner_product: inner sizes differ"); out_sizes = {xs[o], ys[o]}; }
  else if (e == "ji,jk->ik") { c = {xs[o + 1], xs[o], ys[o + 1], 2, batch}; if (xs[o] != ys[o]) panic("inner_product: inner sizes differ"); out_sizes = {xs[o + 1], ys[o + 1]}; }
  else if (o == 0 && e == "i,ij->j") { c = {1, xs[0], ys[1], 0, 0}; if (xs[0] != ys[0]) panic("inner_product: inner sizes differ"); out_sizes = {ys[1]}; }
  else if (o == 0 && e == "ij,j->i") { c = {xs[0], xs[1], 1, 0, 0}; if (xs[1] != ys[0]) panic("inner_product: inner sizes differ"); out_sizes = {xs[0]}; }
  else panic("inner_product: unknown expression");
  if (o == 1) out_sizes.insert(out_sizes.begin(), static_cast<size_t>(batch));
  return c;
}
static void gemm(int key, int kind, const void* a, const void* b, double alpha, void* c, double beta, len_t m, len_t n, len_t k,
                 StreamContext ctx, len_t batch = 0) {
  if (batch != 0) {
    if (kind == 0) kernels::ip_bij_bjk_bik[key](a, b, alpha, c, beta, batch, m, n, k, ctx);
    else if (kind == 1) kernels::ip_bij_bkj_bik[key](a, b, alpha, c, beta, batch, m, n, k, ctx);
    else kernels::ip_bji_bjk_bik[key](a, b, alpha, c, beta, batch, m, n, k, ctx);
    return;
  }
  if (kind == 0) kernels::ip_ij_jk_ik[key](a, b, alpha, c, beta, m, n, k, ctx);
  else if (kind == 1) kernels::ip_ij_kj_ik[key](a, b, alpha, c, beta, m, n, k, ctx);
  else kernels::ip_ji_jk_ik[key](a, b, alpha, c, beta, m, n, k, ctx);
}
// --- rank-N contractions (NOTES.md:3-5; grammar expression_parsing.zig:258-317) ---
// The indices fall into four groups: batch (both operands and the output), rows (first operand and output), columns
// (second operand and output) and summed (both operands only).  With every group flattened the contraction is
// C[batch][rows, columns] = A[batch][rows, summed] . B[batch][summed, columns]; an operand whose indices already lie
// as [batch, rows, summed] / [batch, summed, rows] (second operand: [batch, summed, columns] / [batch, columns,
// summed]) goes to the kernel of that form where it lies, any other order passes through the general permutation first.
struct SplitExpr { std::string xs, ys, os; };
static SplitExpr split_contraction(const std::string& expr) {
  const size_t comma = expr.find(','), arrow = expr.find("->");
  if (comma == std::string::npos || arrow == std::string::npos || comma > arrow) panic("inner_product: expression must read \"x,y->z\"");
  return {expr.substr(0, comma), expr.substr(comma + 1, arrow - comma - 1), expr.substr(arrow + 2)};
}
static void check_indices(const std::string& s, size_t rank) {
  if (s.size() != rank) panic("inner_product: the expression's rank differs from the tensor's");
  if (s.size() > 6) panic("inner_product: rank above 6");
  for (size_t i = 0; i < s.size(); ++i)
    if (s[i] < 'a' || s[i] > 'z' || s.find(s[i]) != i) panic("inner_product: indices must be distinct lower case characters");
}
static bool has(const std::string& s, char c) { return s.find(c) != std::string::npos; }
static std::vector<size_t> order_into(const std::string& from, const std::string& to) {   // perm[i] = position of from[i] in to
  std::vector<size_t> perm(from.size());
  for (size_t i = 0; i < from.size(); ++i) perm[i] = to.find(from[i]);
  return perm;
}
static ContractionPlan plan_contraction(const std::string& xs, const std::string& ys, const std::string& os,
                                        const std::vector<size_t>& xsz, const std::vector<size_t>& ysz, bool may_swap) {
  check_indices(xs, xsz.size()); check_indices(ys, ysz.size()); check_indices(os, os.size());
  size_t extent[26] = {};
  for (size_t i = 0; i < xs.size(); ++i) extent[xs[i] - 'a'] = xsz[i];
  for (size_t i = 0; i < ys.size(); ++i) {
    if (has(xs, ys[i]) && extent[ys[i] - 'a'] != ysz[i]) panic("inner_product: the operands' sizes differ at a shared index");
    extent[ys[i] - 'a'] = ysz[i];
  }
  std::string B, M, N, K;   // batch, rows, columns (in the output's order), summed (in the first operand's order)
  for (char c : os) {
    const bool in_x = has(xs, c), in_y = has(ys, c);
    if (in_x && in_y) B += c; else if (in_x) M += c; else if (in_y) N += c;
    else panic("inner_product: an output index is in neither operand");
  }
  for (char c : xs) if (!has(os, c)) { if (!has(ys, c)) panic("inner_product: an index of one operand only must be in the output"); K += c; }
  for (char c : ys) if (!has(os, c) && !has(xs, c)) panic("inner_product: an index of one operand only must be in the output");
  // "ik,ij->jk": the output lists the second operand's indices first: C^T = B^T A^T, the same contraction with the operands exchanged
  if (may_swap && !M.empty() && !N.empty() && os != B + M + N && os == B + N + M) {
    ContractionPlan p = plan_contraction(ys, xs, os, ysz, xsz, false);
    p.swap = true;
    return p;
  }
  ContractionPlan p;
  auto volume = [&](const std::string& s) { size_t v = 1; for (char c : s) v *= extent[c - 'a']; return v; };
  p.batch = B.empty() ? 0 : volume(B);
  p.m = volume(M); p.n = volume(K); p.k = volume(N);
  const std::string x_rows = B + M + K, x_cols = B + K + M, y_rows = B + K + N, y_cols = B + N + K;
  const bool x_a = xs == x_rows, x_t = xs == x_cols, y_a = ys == y_rows, y_t = ys == y_cols;
  // kinds the kernels take: (rows, rows) = 0, (rows, cols) = 1, (cols, rows) = 2
  if (x_a && y_a) p.kind = 0;
  else if (x_a && y_t) p.kind = 1;
  else if (x_t && y_a) p.kind = 2;
  else if (x_a || x_t) { p.kind = x_a ? 0 : 2; p.y_perm = order_into(ys, y_rows); }
  else if (y_a || y_t) { p.kind = y_a ? 0 : 1; p.x_perm = order_into(xs, x_rows); }
  else { p.kind = 0; p.x_perm = order_into(xs, x_rows); p.y_perm = order_into(ys, y_rows); }
  const std::string z_lies = B + M + N;
  if (os != z_lies) {
    p.z_perm = order_into(z_lies, os);
    for (char c : z_lies) p.z_sizes.push_back(extent[c - 'a']);
  }
  for (char c : os) p.out_sizes.push_back(extent[c - 'a']);
  if (p.out_sizes.empty()) p.out_sizes = {1};   // full contraction
  return p;
}
ContractionPlan contraction_plan(const std::string& expr, const std::vector<size_t>& x_sizes, const std::vector<size_t>& y_sizes) {
  const SplitExpr e = split_contraction(expr);
  return plan_contraction(e.xs, e.ys, e.os, x_sizes, y_sizes, true);
}
// z[os] = scale * sum x[xs] y[ys] + beta * z; the permuted copies live in the stream's scratch buffer
static void run_contraction(Graph* g, int key, size_t elem, StreamContext ctx, const void* x, const std::vector<size_t>& xsz,
                            const std::string& xs, const void* y, const std::vector<size_t>& ysz, const std::string& ys, double scale,
                            void* z, const std::string& os, double beta) {
  const ContractionPlan p = plan_contraction(xs, ys, os, xsz, ysz, true);
  if (p.swap) { std::swap(x, y); }
  const std::vector<size_t>& asz = p.swap ? ysz : xsz;
  const std::vector<size_t>& bsz = p.swap ? xsz : ysz;
  auto bytes_of = [&](const std::vector<size_t>& sz) { size_t v = elem; for (size_t e : sz) v *= e; return (v + 255) & ~size_t(255); };
  const size_t xb = p.x_perm.empty() ? 0 : bytes_of(asz), yb = p.y_perm.empty() ? 0 : bytes_of(bsz),
               zb = p.z_perm.empty() ? 0 : bytes_of(p.z_sizes);
  unsigned char* tmp = (xb + yb + zb) != 0 ? static_cast<unsigned char*>(g->scratch(xb + yb + zb)) : nullptr;
  if (xb != 0) { call_permutate(key, x, tmp, 0.0, asz, p.x_perm, ctx); x = tmp; }
  if (yb != 0) { call_permutate(key, y, tmp + xb, 0.0, bsz, p.y_perm, ctx); y = tmp + xb; }
  void* c = zb != 0 ? static_cast<void*>(tmp + xb + yb) : z;
  gemm(key, p.kind, x, y, scale, c, zb != 0 ? 0.0 : beta, p.m, p.n, p.k, ctx, p.batch);
  if (zb != 0) call_permutate(key, c, z, beta, p.z_sizes, p.z_perm, ctx);
}
// Z = X.Y over the summed indices: dX is the contraction of dZ with Y over the indices X lacks ("os,ys->xs"), dY that
// of X with dZ ("xs,os->ys"); both accumulate
static void contraction_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[1].tensor, z = a[4].tensor;
  const SplitExpr e = split_contraction(a[3].expr);
  enable_gradient(x); enable_gradient(y);
  const std::vector<size_t> zsz = e.os.empty() ? std::vector<size_t>{} : z.sizes();
  const int key = dkey(z);
  const size_t elem = dtype_size(z.dtype());
  run_contraction(z.ptr, key, elem, z.context(), z.grad_ptr(), zsz, e.os, y.data_ptr(), y.sizes(), e.ys, a[2].scalar, x.grad_ptr(), e.xs, 1.0);
  run_contraction(z.ptr, key, elem, z.context(), x.data_ptr(), x.sizes(), e.xs, z.grad_ptr(), zsz, e.os, a[2].scalar, y.grad_ptr(), e.ys, 1.0);
}
// the expressions the reference spells out (inner_product.zig:116-122) and the batched forms keep their direct path
static bool named_contraction(const std::string& e) {
  static const char* const forms[] = {"ij,jk->ik", "ij,kj->ik", "ji,jk->ik", "i,ij->j", "ij,j->i"};
  for (const char* f : forms) if (e == f) return true;
  if (e.size() == 12 && e[3] == ',' && e[7] == '-' && e[8] == '>' && e[0] == e[4] && e[0] == e[9] && e.find(e[0], 1) == 4) {
    const std::string inner = e.substr(1, 2) + "," + e.substr(5, 2) + "->" + e.substr(10, 2);
    for (int i = 0; i < 3; ++i) if (inner == forms[i]) return true;
  }
  return false;
}
static void inner_product_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[1].tensor, z = a[4].tensor;
  const double scale = a[2].scalar;
  std::vector<size_t> tmp;
  const Contraction c = parse_contraction(x, y, a[3].expr, tmp);
  enable_gradient(x); enable_gradient(y);
  const int key = dkey(z);
  StreamContext ctx = z.context();
  const void* G = z.grad_ptr();
  // Z = op(X) op(Y):  dX and dY as native transposed-operand contractions, accumulated (beta = 1)
  if (c.kind == 0) {          // Z = X Y: dX = G Y^T (ij,kj), dY = X^T G (ji,jk)
    gemm(key, 1, G, y.data_ptr(), scale, x.grad_ptr(), 1.0, c.m, c.k, c.n, ctx, c.batch);
    gemm(key, 2, x.data_ptr(), G, scale, y.grad_ptr(), 1.0, c.n, c.m, c.k, ctx, c.batch);
  } else if (c.kind == 1) {   // Z = X Y^T: dX = G Y (ij,jk), dY = G^T X (ji,jk)
    gemm(key, 0, G, y.data_ptr(), scale, x.grad_ptr(), 1.0, c.m, c.k, c.n, ctx, c.batch);
    gemm(key, 2, G, x.data_ptr(), scale, y.grad_ptr(), 1.0, c.k, c.m, c.n, ctx, c.batch);
  } else {                    // Z = X^T Y: dX = Y G^T (ij,kj), dY = X G (ij,jk)
    gemm(key, 1, y.data_ptr(), G, scale, x.grad_ptr(), 1.0, c.n, c.k, c.m, ctx, c.batch);
    gemm(key, 0, x.data_ptr(), G, scale, y.grad_ptr(), 1.0, c.n, c.m, c.k, ctx, c.batch);
  }
}
Tensor inner_product_scaled(Tensor x, Tensor y, double scale, const std::string& expr) {
  if (x.dtype() != y.dtype()) panic("inner_product: dtypes differ");
  Graph* g = x.ptr;
  if (!named_contraction(expr)) {
    const SplitExpr e = split_contraction(expr);
    const ContractionPlan p = plan_contraction(e.xs, e.ys, e.os, x.sizes(), y.sizes(), true);
    Tensor z = g->tensor({Class::hid, x.dtype(), p.out_sizes});
    run_contraction(g, dkey(z), dtype_size(z.dtype()), z.context(), x.data_ptr(), x.sizes(), e.xs, y.data_ptr(), y.sizes(), e.ys, scale,
                    z.data_ptr(), e.os, 0.0);
    if (g->mode == Mode::train)
      attach_op(contraction_rev, z, {OpDatum::of(x), OpDatum::of(y), OpDatum::of(scale), OpDatum::of(expr), OpDatum::of(z)});
    return z;
  }
  std::vector<size_t> out_sizes;
  const Contraction c = parse_contraction(x, y, expr, out_sizes);
  Tensor z = g->tensor({Class::hid, x.dtype(), out_sizes});
  gemm(dkey(z), c.kind, x.data_ptr(), y.data_ptr(), scale, z.data_ptr(), 0.0, c.m, c.n, c.k, z.context(), c.batch);
  if (g->mode == Mode::train)
    attach_op(inner_product_rev, z, {OpDatum::of(x), OpDatum::of(y), OpDatum::of(scale), OpDatum::of(expr), OpDatum::of(z)});
  return z;
}
Tensor inner_product(Tensor x, Tensor y, const std::string& expr) { return inner_product_scaled(x, y, 1.0, expr); }

// --- linear: y = x.A + b, bias added in the GEMM epilogue (README.md:81,97) ---
static void linear_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, A = a[1].tensor, b = a[2].tensor, z = a[4].tensor;
  std::vector<size_t> tmp;
  const Contraction c = parse_contraction(x, A, a[3].expr, tmp);
  enable_gradient(x); enable_gradient(A); enable_gradient(b);
  const int key = dkey(z);
  StreamContext ctx = z.context();
  if (a[3].expr == "ij,j->i") {
    // y = M v + b with M = x [m,n], v = A [n]: dM = G v^T, dv = M^T G, db = G (one bias entry per output row)
    gemm(key, 1, z.grad_ptr(), A.data_ptr(), 1.0, x.grad_ptr(), 1.0, c.m, c.k, c.n, ctx);
    gemm(key, 2, x.data_ptr(), z.grad_ptr(), 1.0, A.grad_ptr(), 1.0, c.n, c.m, c.k, ctx);
    kernels::addition[key](z.grad_ptr(), b.grad_ptr(), b.grad_ptr(), c.m, ctx);
    return;
  }
  gemm(key, 1, z.grad_ptr(), A.data_ptr(), 1.0, x.grad_ptr(), 1.0, c.m, c.k, c.n, ctx);   // dx = G A^T
  gemm(key, 2, x.data_ptr(), z.grad_ptr(), 1.0, A.grad_ptr(), 1.0, c.n, c.m, c.k, ctx);   // dA = x^T G
  kernels::reduce_ij_j[key](z.grad_ptr(), b.grad_ptr(), 1.0, c.m, c.k, ctx);              // db = sum_i G
}
// "ij,jk->ik" and "i,ij->j": y = x.A + b with b along the output columns.  "ij,j->i" (README.md:81, called as
// linear(A, x, b, ...)): y = A.x + b with one bias entry per output row, so the first operand is the matrix.
Tensor linear(Tensor x, Tensor A, Tensor b, const std::string& expr) {
  if (expr != "ij,jk->ik" && expr != "i,ij->j" && expr != "ij,j->i")
    panic("linear: expression must be \"ij,jk->ik\", \"i,ij->j\" or \"ij,j->i\"");
  Graph* g = x.ptr;
  std::vector<size_t> out_sizes;
  const Contraction c = parse_contraction(x, A, expr, out_sizes);
  const bool mat_vec = expr == "ij,j->i";
  if (b.len() != (mat_vec ? c.m : c.k)) panic("linear: bias length differs from the output length");
  Tensor z = g->tensor({Class::hid, x.dtype(), out_sizes});
  if (mat_vec) {
    gemm(dkey(z), 0, x.data_ptr(), A.data_ptr(), 1.0, z.data_ptr(), 0.0, c.m, c.n, c.k, z.context());
    kernels::addition[dkey(z)](z.data_ptr(), b.data_ptr(), z.data_ptr(), c.m, z.context());
  } else {
    kernels::linear[dkey(z)](x.data_ptr(), A.data_ptr(), b.data_ptr(), 1.0, z.data_ptr(), 0.0, c.m, c.n, c.k, z.context());
  }
  if (g->mode == Mode::train)
    attach_op(linear_rev, z, {OpDatum::of(x), OpDatum::of(A), OpDatum::of(b), OpDatum::of(expr), OpDatum::of(z)});
  return z;
}

// --- row-wise softmax / RMSNorm ("ij|j", expression_parsing.zig:319-340) ---
static void softmax_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, y = a[1].tensor;
  enable_gradient(x);
  const auto& s = y.sizes();
  kernels::softmax_reverse[dkey(y)](y.data_ptr(), y.grad_ptr(), x.grad_ptr(), 1.0, s[0], s[1], y.context());
}
Tensor softmax(Tensor x) {
  if (x.sizes().size() != 2) panic("softmax needs a rank-2 tensor");
  Graph* g = x.ptr;
  Tensor y = hidden_like(g, x);
  kernels::softmax[dkey(y)](x.data_ptr(), y.data_ptr(), x.sizes()[0], x.sizes()[1], y.context());
  if (g->mode == Mode::train) attach_op(softmax_rev, y, {OpDatum::of(x), OpDatum::of(y)});
  return y;
}
static void rmsnorm_rev(const std::vector<OpDatum>& a) {
  Tensor x = a[0].tensor, gain = a[1].tensor, y = a[3].tensor;
  enable_gradient(x); enable_gradient(gain);
  const auto& s = x.sizes();
  Graph* g = x.ptr;
  void* scratch = g->scratch(mpRmsnormReverseScratchBytes(s[0], s[1], y.context()));
  kernels::rmsnorm_reverse[dkey(y)](x.data_ptr(), gain.data_ptr(), nullptr, y.grad_ptr(), a[2].scalar, x.grad_ptr(),
                                    gain.grad_ptr(), 1.0, scratch, s[0], s[1], y.context());
}
Tensor rmsnorm(Tensor x, Tensor gain, double eps) {
  if (x.sizes().size() != 2 || gain.len() != x.sizes()[1]) panic("rmsnorm: x must be [m,n] and gain [n]");
  Graph* g = x.ptr;
  Tensor y = hidden_like(g, x);
  kernels::rmsnorm[dkey(y)](x.data_ptr(), gain.data_ptr(), eps, y.data_ptr(), nullptr, x.sizes()[0], x.sizes()[1], y.context());
  if (g->mode == Mode::train) attach_op(rmsnorm_rev, y, {OpDatum::of(x), OpDatum::of(gain), OpDatum::of(eps), OpDatum::of(y)});
  return y;
}

}  // namespace ops

// ------------------------------ optimizers ------------------------------------------
namespace optm {
ClipRange::ClipRange() : lower(-std::numeric_limits<double>::infinity()), upper(std::numeric_limits<double>::infinity()) {}

// Every weight leaf that has a gradient: w -= rate * clip(g) (optimizer.zig:140-179).
void SGD::update(Graph* graph) {
  Graph::Block& b = graph->leaf_block;
  for (size_t i = 0; i < b.data.size(); ++i) {
    if (b.cls[i] != Class::wgt || b.grad[i] == nullptr || b.len[i] == 0) continue;
    kernels::sgd[static_cast<int>(b.dtype[i])](b.data[i], b.grad[i], rate, clip.lower, clip.upper, b.len[i], graph->stream.context);
  }
  mpStreamSynchronize(graph->stream.context);   // the reference synchronises each active stream once
}

void Momentum::update(Graph* graph) {
  if (!(alpha > 0.0 && alpha < 1.0)) panic("Momentum: alpha must lie in (0, 1)");
  Graph::Block& b = graph->leaf_block;
  for (size_t i = 0; i < b.data.size(); ++i) {
    if (b.cls[i] != Class::wgt || b.grad[i] == nullptr || b.len[i] == 0) continue;
    const int key = static_cast<int>(b.dtype[i]);
    auto k = std::make_pair(graph, i);
    auto it = state.find(k);
    if (it == state.end()) {   // optimizer.zig:249-256: allocated and zero-filled on first use
      void* m = mpMemAlloc(b.len[i] * dtype_size(b.dtype[i]), graph->stream.context);
      kernels::fill[key](m, 0.0, b.len[i], graph->stream.context);
      it = state.emplace(k, m).first;
    }
    kernels::momentum[key](b.data[i], b.grad[i], it->second, rate, alpha, clip.lower, clip.upper, b.len[i], graph->stream.context);
  }
  mpStreamSynchronize(graph->stream.context);
}
void Momentum::deinit(Stream stream) {   // optimizer.zig:211-218
  for (auto& kv : state) mpMemFree(kv.second, stream.context);
  state.clear();
}

void Adam::update(Graph* graph) {
  Graph::Block& b = graph->leaf_block;
  ++step;
  for (size_t i = 0; i < b.data.size(); ++i) {
    if (b.cls[i] != Class::wgt || b.grad[i] == nullptr || b.len[i] == 0) continue;
    const int key = static_cast<int>(b.dtype[i]);
    auto k = std::make_pair(graph, i);
    auto it = state.find(k);
    if (it == state.end()) {   // zero-filled on first use, like the reference's Momentum map (optimizer.zig:249-256)
      const size_t bytes = b.len[i] * dtype_size(b.dtype[i]);
      void* m = mpMemAlloc(bytes, graph->stream.context);
      void* v = mpMemAlloc(bytes, graph->stream.context);
      kernels::fill[key](m, 0.0, b.len[i], graph->stream.context);
      kernels::fill[key](v, 0.0, b.len[i], graph->stream.context);
      it = state.emplace(k, std::make_pair(m, v)).first;
    }
    kernels::adam[key](b.data[i], b.grad[i], it->second.first, it->second.second, rate, beta1, beta2, eps, grad_scale, step,
                       b.len[i], graph->stream.context);
  }
  mpStreamSynchronize(graph->stream.context);
}
}  // namespace optm

}  // namespace mp

// README feed-forward block (README.md:90-104) timed through this layer: y = selu(linear(x, A, b)) on
// x[32,256], A[256,256], b[256] in r32, then reverse(.free) of the sum loss and one SGD step (rate 1e-2).
// out[0] = host microseconds per forward (stream-synchronised, as the .free walk is), out[1] = per forward +
// reverse + update, out[2], out[3] = kernel launches per forward / per step.  Returns 0 on success.
extern "C" int mpHostFeedForwardBench(int iters, double* out) {
  using namespace mp;
  if (iters <= 0 || out == nullptr) return 1;
  const size_t m = 32, n = 256, k = 256;
  Stream st = stream::init();
  Graph* G = Graph::init({st, Mode::train});
  Tensor x = G->tensor({Class::inp, Dtype::r32, {m, n}});
  Tensor A = G->tensor({Class::wgt, Dtype::r32, {n, k}});
  Tensor b = G->tensor({Class::wgt, Dtype::r32, {k}});
  // deterministic values with the scale of the configuration (x ~ unit scale, A ~ 1/16, b = 0)
  algo::sequence(x, -1.0, 2.0 / static_cast<double>(m * n));
  algo::sequence(A, -1.0 / 16.0, 2.0 / 16.0 / static_cast<double>(n * k));
  algo::fill(b, 0.0);
  optm::SGD sgd{1e-2, optm::ClipRange()};
  auto step = [&](bool train) {
    Tensor lin = ops::linear(x, A, b, "ij,jk->ik");
    Tensor y = ops::selu(lin);
    if (train) {
      G->reset(ResetGroup::leaf, ResetComponent::grd);
      y.reverse(ReverseCleanup::free);
      sgd.update(G);
    } else {
      stream::sync(st);
      y.free(); lin.free();
    }
  };
  for (int i = 0; i < 20; ++i) step(true);
  stream::sync(st);
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < iters; ++i) step(false);
  const auto t1 = std::chrono::steady_clock::now();
  for (int i = 0; i < iters; ++i) step(true);
  stream::sync(st);
  const auto t2 = std::chrono::steady_clock::now();
  out[0] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
  out[1] = std::chrono::duration<double, std::micro>(t2 - t1).count() / iters;
  out[2] = 2.0;    // linear (bias in the contraction's epilogue), selu
  out[3] = 13.0;   // + 3 gradient fills, seed fill, selu reverse, 2 contractions, column sum (2 kernels), 2 SGD updates
  G->deinit();
  stream::deinit(st);
  return 0;
}
