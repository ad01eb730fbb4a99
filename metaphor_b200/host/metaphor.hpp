// C++ mirror of the reference's Zig host layer (src/metaphor.zig facade,
// src/core/graph.zig, src/core/tensor_allocator.zig, src/ops/*.zig,
// src/algo/mem.zig, src/optm/optimizer.zig) over the extern "C" device layer of
// include/*.h.  No Zig toolchain exists where this library is built and tested,
// so this layer keeps the reference's names, argument meaning and behaviour in
// C++: the same kernel call sequences, the same reverse walk over dependency
// counters with .keep / .free clean-up and detach(), the same exact-size tensor
// cache.  One deliberate difference: a gradient buffer is zero-filled when it is
// created (the reference allocates it without initialising it, graph.zig:710-722,
// and then accumulates into it).
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <optional>
#include <string>
#include <vector>

#include "../../include/mp_device_utils.h"
#include "../../include/mp_kernels.h"

namespace mp {

enum class Dtype : int { r16 = 0, r32 = 1, r64 = 2 };   // scalar.zig:35-40, = dispatch key
enum class Class { inp, wgt, hid };                     // graph.zig TensorClass
enum class Mode { train, eval };
enum class ReverseCleanup { keep, free };               // graph.zig:254
enum class ResetGroup { node, leaf };
enum class ResetComponent { all, grd };

inline size_t dtype_size(Dtype d) { return d == Dtype::r16 ? 2 : (d == Dtype::r32 ? 4 : 8); }

struct Stream { StreamContext context; };

namespace device {          // metaphor.zig:13-18
void init(unsigned device_number);
void sync();
void check();
size_t total_memory(unsigned device_number);
}
namespace stream {          // metaphor.zig:20-25
Stream init();
void deinit(Stream s);
void sync(Stream s);
}

class Graph;

// Handle into a graph (graph.zig:34-183): leaves (inp, wgt) and computed nodes
// (hid) live in separate blocks, idx indexes the block of `cls`.
struct Tensor {
  Graph* ptr = nullptr;
  Class cls = Class::inp;
  size_t idx = 0;

  void* data_ptr() const;
  void* grad_ptr() const;                 // nullptr until a gradient exists
  bool has_grad() const { return grad_ptr() != nullptr; }
  const std::vector<size_t>& sizes() const;
  size_t len() const;                     // 0 after the tensor was freed
  Dtype dtype() const;
  StreamContext context() const;
  void reverse(ReverseCleanup cleanup) const;   // graph.zig:111-121
  void detach() const;                          // graph.zig:103-105
  void free() const;
  // Forward-mode derivative d self / d wrt of an element-wise expression, as a new tensor of self's shape
  // (graph.zig:123-148); nullopt when self does not depend on wrt or the graph is in eval mode.
  std::optional<Tensor> derive(Tensor wrt) const;
  bool same(Tensor o) const { return ptr == o.ptr && cls == o.cls && idx == o.idx; }
  std::vector<double> native() const;           // values copied to the host (widened to double)
  std::vector<double> native_grad() const;
};

struct TensorConfig { Class cls; Dtype dtype; std::vector<size_t> sizes; };
struct GraphConfig { Stream stream; Mode mode = Mode::train; };

// Exact-size cache over stream-ordered allocation (tensor_allocator.zig:95-141).
class TensorAllocator {
 public:
  void* alloc(size_t bytes, StreamContext ctx);
  void release(void* p, size_t bytes);          // back into the cache
  void drain(StreamContext ctx);                // mpMemFree everything cached
  size_t cached_blocks() const;
 private:
  std::map<size_t, std::vector<void*>> free_;
};

struct OpDatum {            // graph.zig:776-886 (tensor or scalar or expression operand)
  enum Kind { tensor_k, scalar_k, expr_k } kind = tensor_k;
  Tensor tensor;
  double scalar = 0.0;
  std::string expr;
  static OpDatum of(Tensor t) { OpDatum d; d.kind = tensor_k; d.tensor = t; return d; }
  static OpDatum of(double s) { OpDatum d; d.kind = scalar_k; d.scalar = s; return d; }
  static OpDatum of(const std::string& e) { OpDatum d; d.kind = expr_k; d.expr = e; return d; }
};
using ReverseFn = void (*)(const std::vector<OpDatum>& args);
// Element-wise derivative of an op's output w.r.t. `wrt`: a scalar (the same value everywhere), a tensor, or
// nullopt = no dependence (the `?OpDatum` of graph.zig:802-807).
using DeriveFn = std::optional<OpDatum> (*)(const std::vector<OpDatum>& args, Tensor wrt);

class Graph {
 public:
  static Graph* init(GraphConfig cfg);          // graph.zig:331-348
  void deinit();                                // graph.zig:350-369
  Tensor tensor(const TensorConfig& cfg);       // graph.zig:500-520
  void reset(ResetGroup group, ResetComponent component);   // graph.zig:371-414
  // Weights as raw bytes, one file "<dir>/<prefix>_<k>" per weight, k counting the weights in leaf order
  // (graph.zig:633-703, tensor_file.zig:36-40,56-86).  load panics when a file's size differs from the tensor's.
  void save(const std::string& dir, const std::string& prefix);
  void load(const std::string& dir, const std::string& prefix);
  Mode mode;
  Stream stream;

  // internal interface used by ops (attach_op / enable_gradient / reverse walk)
  struct Block {
    std::vector<void*> data, grad;
    std::vector<size_t> len;
    std::vector<std::vector<size_t>> sizes;
    std::vector<Dtype> dtype;
    std::vector<Class> cls;
    // node block only
    std::vector<int> deps;
    std::vector<bool> attached, has_op;
    std::vector<ReverseFn> op_reverse;
    std::vector<DeriveFn> op_derive;
    std::vector<std::vector<OpDatum>> op_args;
  };
  Block leaf_block, node_block;
  TensorAllocator tensor_allocator;
  Block& block_of(Class c) { return c == Class::hid ? node_block : leaf_block; }
  void reverse(size_t idx, ReverseCleanup cleanup);          // graph.zig:552-631
  void free_tensor(Tensor t);
  void free_gradient(Tensor t);
  void* scratch(size_t bytes);                                // utils.zig:20-36 grow-only per-stream scratch
 private:
  void* scratch_ = nullptr;
  size_t scratch_bytes_ = 0;
};

void enable_gradient(Tensor t);                               // graph.zig:710-722 (+ zero fill)
void attach_op(ReverseFn fn, Tensor out, const std::vector<OpDatum>& args, DeriveFn derive = nullptr);   // graph.zig:733-757
std::optional<OpDatum> derive(Tensor x, Tensor wrt);          // graph.zig:762-771: what op.derive functions call

namespace algo {            // src/algo/mem.zig:24-39
void fill(Tensor x, double value);
void sequence(Tensor x, double init, double step);
void copy(Tensor src, Tensor dst);
}
namespace mem = algo;       // README spelling

namespace ops {             // metaphor.zig:44-56 plus the ops the README names
Tensor add(Tensor x, Tensor y);
Tensor sub(Tensor x, Tensor y);
Tensor hadamard(Tensor x, Tensor y);
Tensor negate(Tensor x);
Tensor translate(Tensor x, double value);
Tensor dilate(Tensor x, double value);
Tensor relu(Tensor x);
Tensor selu(Tensor x);
Tensor reduce(Tensor x, const std::string& expr);                       // "ij->i", "ij->j", and any rank <= 6: "ijk->ik", "ijk->j", ...
Tensor broadcast(Tensor x, const std::vector<size_t>& sizes, const std::string& expr);   // "i->ij", "j->ij", "ik->ijk", ...
Tensor inner_product(Tensor x, Tensor y, const std::string& expr);      // "ij,jk->ik", "ij,kj->ik", "ji,jk->ik", "i,ij->j", "ij,j->i";
                                                                        // batched "bij,bjk->bik" (and the kj / ji forms), "_ij,_jk->_ik" = optional batch
Tensor inner_product_scaled(Tensor x, Tensor y, double scale, const std::string& expr);
inline Tensor innerProduct(Tensor x, Tensor y, const std::string& e) { return inner_product(x, y, e); }
// Any other expression is a rank-N contraction (NOTES.md:3-5; grammar expression_parsing.zig:258-317): operands of rank
// <= 6 with distinct lower-case indices in any order, e.g. "abc,cd->abd", "ikj,lk->lij", "bhqd,bhkd->bhqk".  An index of
// both operands that is missing on the right is summed; one of both operands and the output is a batch index; every
// other index must be in the output.  It runs as one (batched) GEMM, with general permutations only around the
// operands whose index order no kernel takes directly; its reverse is two such contractions.
struct ContractionPlan {
  bool swap = false;                       // the GEMM takes the operands in the opposite order; x_* below then describe the caller's second operand
  int kind = 0;                            // 0 = "ij,jk->ik", 1 = "ij,kj->ik", 2 = "ji,jk->ik" after the permutations below
  size_t batch = 0, m = 1, n = 1, k = 1;   // batch 0 = the rank-2 kernel; C[m,k] = A[m,n] B[n,k] in the reference's letters
  std::vector<size_t> x_perm, y_perm;      // empty = the operand is used where it lies; else perm[i] = new position of its i-th index
  std::vector<size_t> z_sizes, z_perm;     // z_perm empty = the GEMM writes the output itself; else its [batch.., m.., k..] result (z_sizes) is permuted into the output
  std::vector<size_t> out_sizes;
};
ContractionPlan contraction_plan(const std::string& expr, const std::vector<size_t>& x_sizes, const std::vector<size_t>& y_sizes);
Tensor linear(Tensor x, Tensor A, Tensor b, const std::string& expr);   // "ij,jk->ik", "i,ij->j"; "ij,j->i" = matrix first: linear(A, x, b, ...)
Tensor permutate(Tensor x, const std::string& expr);                    // any permutation up to rank 6: "ij->ji", "ijk->kij", ...
std::vector<size_t> permutation_of(const std::string& expr);            // perm[i] = position of the i-th left index on the right
Tensor softmax(Tensor x);                                               // over the last axis ("ij|j")
Tensor rmsnorm(Tensor x, Tensor gain, double eps);
}

namespace optm {            // src/optm/optimizer.zig:126-180 (SGD); Adam is named in NOTES.md:11
struct ClipRange { double lower, upper; ClipRange(); ClipRange(double lo, double hi) : lower(lo), upper(hi) {} };
struct SGD {
  double rate;
  ClipRange clip;
  void update(Graph* graph);
};
struct Momentum {           // optimizer.zig:182-275: m = alpha*m + clip(g); w -= rate*m; state per (graph, weight), zero on first use
  double rate, alpha = 0.90;
  ClipRange clip;
  std::map<std::pair<Graph*, size_t>, void*> state;
  void update(Graph* graph);
  void deinit(Stream stream);
};
struct Adam {
  double rate, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, grad_scale = 1.0;
  size_t step = 0;
  std::map<std::pair<Graph*, size_t>, std::pair<void*, void*>> state;   // per (graph, weight): m, v
  void update(Graph* graph);
};
}

}  // namespace mp
