// Scenario tests of the C++ host mirror, replaying the reference's example
// programs (src/examples/subgraphs.zig, src/examples/experimental.zig) and the
// README feed-forward block (README.md:90-104) on the GPU, with numeric checks
// against the CPU oracle (liboracle.so; test infrastructure).
// Usage: host_scenarios [timing-iterations [directory for weight files]]; exit code 0 = all checks passed.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <optional>
#include <random>
#include <string>
#include <vector>

#include "../../metaphor_b200/host/metaphor.hpp"

extern "C" {
void orc_inner_product_f32(const float*, const float*, const float*, double, float*, double, size_t, size_t, size_t, int, int);
void orc_selu_f32(const float*, float*, size_t);
void orc_selu_reverse_f32(const float*, float*, const float*, size_t);
void orc_reduce_ij_j_f32(const float*, float*, double, size_t, size_t);
void orc_sgd_f32(float*, const float*, double, double, double, size_t);
void orc_softmax_ij_j_f32(const float*, float*, size_t, size_t);
void orc_softmax_ij_j_reverse_f32(const float*, const float*, float*, double, size_t, size_t);
void orc_rmsnorm_ij_j_f32(const float*, const float*, double, float*, float*, size_t, size_t);
void orc_rmsnorm_ij_j_reverse_f32(const float*, const float*, const float*, double, float*, float*, double, size_t, size_t);
void orc_momentum_f32(float*, const float*, float*, double, double, double, double, size_t);
void orc_permutate_f32(const float*, float*, double, const size_t*, const size_t*, size_t);
}

static int failures = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) { std::printf("CHECK failed: %s (line %d)\n", #cond, __LINE__); ++failures; } \
  } while (0)

static double rel_err(const std::vector<double>& got, const std::vector<float>& ref) {
  double mx = 1e-30, err = 0;
  if (got.size() != ref.size()) return 1e9;
  for (size_t i = 0; i < ref.size(); ++i) { mx = std::fmax(mx, std::fabs(ref[i])); err = std::fmax(err, std::fabs(got[i] - ref[i])); }
  return err / mx;
}
static void upload(mp::Tensor t, const std::vector<float>& v) {
  mpMemcpyHtoD(t.data_ptr(), v.data(), v.size() * 4, t.context());
  mpStreamSynchronize(t.context());
}
static std::vector<float> normal(size_t n, unsigned seed, float scale) {
  std::mt19937 gen(seed);
  std::normal_distribution<float> d(0.f, scale);
  std::vector<float> v(n);
  for (auto& x : v) x = d(gen);
  return v;
}

// src/examples/subgraphs.zig:6-150
static void scenario_subgraphs(mp::Stream stream) {
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  const size_t M = 32;
  mp::Tensor x = G->tensor({mp::Class::inp, mp::Dtype::r32, {M}});
  mp::Tensor w1 = G->tensor({mp::Class::wgt, mp::Dtype::r32, {M}});
  mp::Tensor w2 = G->tensor({mp::Class::wgt, mp::Dtype::r32, {M}});
  mp::algo::fill(x, 1.0); mp::algo::fill(w1, 1.0); mp::algo::fill(w2, 1.0);
  mp::Tensor z1 = mp::ops::add(x, w1);
  mp::Tensor z2 = mp::ops::relu(z1);
  mp::Tensor z3 = mp::ops::add(z2, w2);
  mp::Tensor z4 = mp::ops::relu(z3);
  for (double v : z4.native()) CHECK(v == 3.0);
  z2.detach();
  z4.reverse(mp::ReverseCleanup::free);
  CHECK(z4.len() == 0); CHECK(z3.len() == 0);
  CHECK(!z4.has_grad()); CHECK(!z3.has_grad());
  CHECK(z2.len() != 0); CHECK(w2.len() != 0);
  CHECK(z2.has_grad()); CHECK(w2.has_grad());
  CHECK(z1.len() != 0); CHECK(w1.len() != 0);
  CHECK(!z1.has_grad()); CHECK(!w1.has_grad());
  for (double v : w2.native_grad()) CHECK(v == 1.0);
  for (double v : z2.native_grad()) CHECK(v == 1.0);
  CHECK(G->tensor_allocator.cached_blocks() >= 2);   // freed nodes went back to the exact-size cache
  z2.reverse(mp::ReverseCleanup::keep);
  CHECK(x.len() != 0); CHECK(z1.len() != 0); CHECK(w1.len() != 0);
  CHECK(z1.has_grad()); CHECK(w1.has_grad());
  for (double v : w1.native_grad()) CHECK(v == 1.0);
  G->reset(mp::ResetGroup::node, mp::ResetComponent::all);
  G->reset(mp::ResetGroup::leaf, mp::ResetComponent::grd);
  CHECK(!w1.has_grad()); CHECK(w1.len() == M);
  mp::device::check();
  G->deinit();
}

// src/examples/experimental.zig:19-71 (values derivable by hand)
static void scenario_experimental(mp::Stream stream) {
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  mp::Tensor x = G->tensor({mp::Class::wgt, mp::Dtype::r32, {3, 2}});
  mp::Tensor y = G->tensor({mp::Class::wgt, mp::Dtype::r32, {2, 2}});
  mp::algo::sequence(x, 1.0, 1.0); mp::algo::sequence(y, 1.0, 1.0);
  mp::Tensor z = mp::ops::inner_product(x, y, "ij,jk->ik");
  CHECK((z.native() == std::vector<double>{7, 10, 15, 22, 23, 34}));
  mp::Tensor a = mp::ops::reduce(y, "ij->i");
  mp::Tensor b = mp::ops::broadcast(a, x.sizes(), "j->ij");
  CHECK((b.native() == std::vector<double>{3, 7, 3, 7, 3, 7}));
  mp::Tensor c = mp::ops::reduce(x, "ij->j");
  mp::Tensor d = mp::ops::broadcast(c, y.sizes(), "i->ij");
  CHECK((d.native() == std::vector<double>{9, 9, 12, 12}));
  z.reverse(mp::ReverseCleanup::keep);
  CHECK((x.native_grad() == std::vector<double>{3, 7, 3, 7, 3, 7}));
  CHECK((y.native_grad() == std::vector<double>{9, 9, 12, 12}));
  mp::Tensor t = mp::ops::permutate(x, "ij->ji");
  CHECK((t.native() == std::vector<double>{1, 3, 5, 2, 4, 6}));
  G->deinit();
}

// README feed-forward block: y = selu(linear(x, A, b)); y.reverse(.free); one SGD step.
static void scenario_feed_forward(mp::Stream stream, int timing_iters) {
  const size_t m = 32, n = 256, k = 256;
  const double lr = 1e-2;
  std::vector<float> hx = normal(m * n, 0, 1.f), hA = normal(n * k, 1, 1.f / 16.f), hb(k, 0.f);
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  mp::Tensor x = G->tensor({mp::Class::inp, mp::Dtype::r32, {m, n}});
  mp::Tensor A = G->tensor({mp::Class::wgt, mp::Dtype::r32, {n, k}});
  mp::Tensor b = G->tensor({mp::Class::wgt, mp::Dtype::r32, {k}});
  upload(x, hx); upload(A, hA); upload(b, hb);
  mp::Tensor lin = mp::ops::linear(x, A, b, "ij,jk->ik");
  mp::Tensor y = mp::ops::selu(lin);
  // oracle: forward
  std::vector<float> rl(m * k), ry(m * k);
  orc_inner_product_f32(hx.data(), hA.data(), hb.data(), 1.0, rl.data(), 0.0, m, n, k, 0, 0);
  orc_selu_f32(rl.data(), ry.data(), m * k);
  CHECK(rel_err(y.native(), ry) <= 1e-4);
  y.reverse(mp::ReverseCleanup::free);
  CHECK(y.len() == 0); CHECK(lin.len() == 0);
  // oracle: reverse of the sum loss (seed 1), gradients start at zero
  std::vector<float> seed(m * k, 1.f), gl(m * k, 0.f), gx(m * n, 0.f), gA(n * k, 0.f), gb(k, 0.f);
  orc_selu_reverse_f32(rl.data(), gl.data(), seed.data(), m * k);
  orc_inner_product_f32(gl.data(), hA.data(), nullptr, 1.0, gx.data(), 1.0, m, k, n, 0, 1);   // dx = G A^T
  orc_inner_product_f32(hx.data(), gl.data(), nullptr, 1.0, gA.data(), 1.0, n, m, k, 1, 0);   // dA = x^T G
  orc_reduce_ij_j_f32(gl.data(), gb.data(), 1.0, m, k);
  CHECK(rel_err(x.native_grad(), gx) <= 1e-4);
  CHECK(rel_err(A.native_grad(), gA) <= 1e-4);
  CHECK(rel_err(b.native_grad(), gb) <= 1e-4);
  mp::optm::SGD sgd{lr, mp::optm::ClipRange()};
  sgd.update(G);
  const double inf = INFINITY;
  orc_sgd_f32(hA.data(), gA.data(), lr, -inf, inf, n * k);
  orc_sgd_f32(hb.data(), gb.data(), lr, -inf, inf, k);
  CHECK(rel_err(A.native(), hA) <= 1e-5);
  CHECK(rel_err(b.native(), hb) <= 1e-4);
  // timing of the whole step through the host layer (launch-latency bound: 12.6 MFLOP, 0.6 MB)
  if (timing_iters > 0) {
    auto step = [&](bool train) {
      mp::Tensor l2 = mp::ops::linear(x, A, b, "ij,jk->ik");
      mp::Tensor y2 = mp::ops::selu(l2);
      if (train) {
        G->reset(mp::ResetGroup::leaf, mp::ResetComponent::grd);
        y2.reverse(mp::ReverseCleanup::free);
        sgd.update(G);
      } else {
        mp::stream::sync(stream);
        y2.free(); l2.free();
      }
    };
    for (int i = 0; i < 20; ++i) step(true);
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < timing_iters; ++i) step(false);
    auto t1 = std::chrono::steady_clock::now();
    for (int i = 0; i < timing_iters; ++i) step(true);
    auto t2 = std::chrono::steady_clock::now();
    const double fwd_us = std::chrono::duration<double, std::micro>(t1 - t0).count() / timing_iters;
    const double all_us = std::chrono::duration<double, std::micro>(t2 - t1).count() / timing_iters;
    std::printf("FEED_FORWARD_TIMING {\"forward_us\": %.2f, \"forward_reverse_sgd_us\": %.2f, \"forward_launches\": 2, "
                "\"step_launches\": 13, \"iters\": %d}\n", fwd_us, all_us, timing_iters);
  }
  G->deinit();
}

// README.md:78-81: y = A.x ("ij,j->i") and y = A.x + b through linear(A, x, b, "ij,j->i"), forward and reverse.
static void scenario_matrix_vector(mp::Stream stream) {
  const size_t m = 48, n = 200;
  std::vector<float> hA = normal(m * n, 11, 0.1f), hx = normal(n, 12, 1.f), hb = normal(m, 13, 1.f);
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  mp::Tensor A = G->tensor({mp::Class::wgt, mp::Dtype::r32, {m, n}});
  mp::Tensor x = G->tensor({mp::Class::inp, mp::Dtype::r32, {n}});
  mp::Tensor b = G->tensor({mp::Class::wgt, mp::Dtype::r32, {m}});
  upload(A, hA); upload(x, hx); upload(b, hb);
  mp::Tensor y0 = mp::ops::innerProduct(A, x, "ij,j->i");
  mp::Tensor y = mp::ops::linear(A, x, b, "ij,j->i");
  std::vector<float> r0(m), r1(m);
  orc_inner_product_f32(hA.data(), hx.data(), nullptr, 1.0, r0.data(), 0.0, m, n, 1, 0, 0);
  for (size_t i = 0; i < m; ++i) r1[i] = r0[i] + hb[i];
  CHECK(y0.sizes() == std::vector<size_t>{m});
  CHECK(rel_err(y0.native(), r0) <= 1e-4);
  CHECK(rel_err(y.native(), r1) <= 1e-4);
  y.reverse(mp::ReverseCleanup::keep);
  // sum loss: G = 1, dA = 1 x^T, dx = A^T 1, db = 1
  std::vector<float> gA(m * n), gx(n, 0.f), gb(m, 1.f);
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) { gA[i * n + j] = hx[j]; gx[j] += hA[i * n + j]; }
  CHECK(rel_err(A.native_grad(), gA) <= 1e-4);
  CHECK(rel_err(x.native_grad(), gx) <= 1e-4);
  CHECK(rel_err(b.native_grad(), gb) <= 1e-5);
  G->deinit();
}

static void scenario_row_ops(mp::Stream stream) {
  const size_t m = 48, n = 1024;
  std::vector<float> hx = normal(m * n, 5, 1.f), hgain = normal(n, 6, 0.02f);
  for (auto& g : hgain) g += 1.f;
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  mp::Tensor x = G->tensor({mp::Class::wgt, mp::Dtype::r32, {m, n}});
  mp::Tensor gain = G->tensor({mp::Class::wgt, mp::Dtype::r32, {n}});
  upload(x, hx); upload(gain, hgain);
  mp::Tensor y = mp::ops::softmax(mp::ops::rmsnorm(x, gain, 1e-6));
  std::vector<float> rn(m * n), rstd(m), ry(m * n);
  orc_rmsnorm_ij_j_f32(hx.data(), hgain.data(), 1e-6, rn.data(), rstd.data(), m, n);
  orc_softmax_ij_j_f32(rn.data(), ry.data(), m, n);
  CHECK(rel_err(y.native(), ry) <= 1e-4);
  y.reverse(mp::ReverseCleanup::keep);
  std::vector<float> ones(m * n, 1.f), gn(m * n, 0.f), gx(m * n, 0.f), gg(n, 0.f);
  orc_softmax_ij_j_reverse_f32(ry.data(), ones.data(), gn.data(), 0.0, m, n);
  orc_rmsnorm_ij_j_reverse_f32(hx.data(), hgain.data(), gn.data(), 1e-6, gx.data(), gg.data(), 0.0, m, n);
  // gradient of sum(softmax) is zero up to rounding: compare on the scale of the activations
  const std::vector<double> got = x.native_grad();
  double err = 0;
  for (size_t i = 0; i < got.size(); ++i) err = std::fmax(err, std::fabs(got[i] - gx[i]));
  CHECK(err <= 1e-6);
  G->deinit();
}

// Rank-3 operators of the reference's roadmap (NOTES.md:3-5 general permutation, NOTES.md:18 "_ij,_jk->_ik")
static void scenario_rank3(mp::Stream stream) {
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  // y = permute(x, "ijk->kij"), loss = sum(y o w): x.grad is w carried back through the inverse permutation
  const size_t sizes[3] = {2, 3, 4};
  mp::Tensor x = G->tensor({mp::Class::wgt, mp::Dtype::r32, {2, 3, 4}});
  mp::Tensor w = G->tensor({mp::Class::wgt, mp::Dtype::r32, {4, 2, 3}});
  mp::algo::sequence(x, 1.0, 1.0); mp::algo::sequence(w, 0.5, 0.25);
  CHECK((mp::ops::permutation_of("ijk->kij") == std::vector<size_t>{1, 2, 0}));
  mp::Tensor y = mp::ops::permutate(x, "ijk->kij");
  CHECK((y.sizes() == std::vector<size_t>{4, 2, 3}));
  std::vector<float> hx(24), hw(24), ref(24), gref(24, 0.f);
  for (int i = 0; i < 24; ++i) { hx[i] = 1.f + i; hw[i] = 0.5f + 0.25f * i; }
  const size_t perm[3] = {1, 2, 0}, out_sizes[3] = {4, 2, 3}, inverse[3] = {2, 0, 1};
  orc_permutate_f32(hx.data(), ref.data(), 0.0, sizes, perm, 3);
  CHECK(rel_err(y.native(), ref) == 0.0);
  mp::Tensor z = mp::ops::hadamard(y, w);
  z.reverse(mp::ReverseCleanup::keep);
  orc_permutate_f32(hw.data(), gref.data(), 1.0, out_sizes, inverse, 3);   // accumulated into a zeroed gradient
  CHECK(rel_err(x.native_grad(), gref) == 0.0);

  // batched contraction and its reverse, every entry against the rank-2 oracle
  const size_t nb = 3, m = 5, n = 7, k = 4;
  std::vector<float> ha = normal(nb * m * n, 21, 1.f), hb = normal(nb * n * k, 22, 0.4f);
  mp::Tensor a = G->tensor({mp::Class::wgt, mp::Dtype::r32, {nb, m, n}});
  mp::Tensor b = G->tensor({mp::Class::wgt, mp::Dtype::r32, {nb, n, k}});
  upload(a, ha); upload(b, hb);
  mp::Tensor c = mp::ops::inner_product(a, b, "bij,bjk->bik");
  CHECK((c.sizes() == std::vector<size_t>{nb, m, k}));
  std::vector<float> rc(nb * m * k), ga(nb * m * n, 0.f), gb(nb * n * k, 0.f), ones(m * k, 1.f);
  for (size_t q = 0; q < nb; ++q) {
    orc_inner_product_f32(&ha[q * m * n], &hb[q * n * k], nullptr, 1.0, &rc[q * m * k], 0.0, m, n, k, 0, 0);
    orc_inner_product_f32(ones.data(), &hb[q * n * k], nullptr, 1.0, &ga[q * m * n], 1.0, m, k, n, 0, 1);   // dA = G B^T
    orc_inner_product_f32(&ha[q * m * n], ones.data(), nullptr, 1.0, &gb[q * n * k], 1.0, n, m, k, 1, 0);   // dB = A^T G
  }
  CHECK(rel_err(c.native(), rc) <= 1e-4);
  c.reverse(mp::ReverseCleanup::keep);
  CHECK(rel_err(a.native_grad(), ga) <= 1e-4);
  CHECK(rel_err(b.native_grad(), gb) <= 1e-4);
  // the optional batch index: rank-3 operands take the batched kernel, rank-2 operands the plain one
  mp::Tensor c3 = mp::ops::inner_product(a, b, "_ij,_jk->_ik");
  CHECK(rel_err(c3.native(), rc) <= 1e-4);
  mp::Tensor x2 = G->tensor({mp::Class::inp, mp::Dtype::r32, {3, 2}});
  mp::Tensor y2 = G->tensor({mp::Class::inp, mp::Dtype::r32, {2, 2}});
  mp::algo::sequence(x2, 1.0, 1.0); mp::algo::sequence(y2, 1.0, 1.0);
  CHECK((mp::ops::inner_product(x2, y2, "_ij,_jk->_ik").native() == std::vector<double>{7, 10, 15, 22, 23, 34}));
  mp::device::check();
  G->deinit();
}

// Rank-N contractions (NOTES.md:3-5; grammar expression_parsing.zig:258-317): forward and both gradients against
// the contraction summed straight from its expression
static std::vector<float> contraction_direct(const std::string& xs, const std::string& ys, const std::string& os,
                                             const std::vector<float>& x, const std::vector<float>& y, const size_t* extent) {
  std::string letters;
  for (char c : xs + ys + os) if (letters.find(c) == std::string::npos) letters += c;
  std::vector<size_t> idx(letters.size(), 0);
  auto offset = [&](const std::string& s) {
    size_t off = 0;
    for (char c : s) off = off * extent[c - 'a'] + idx[letters.find(c)];
    return off;
  };
  size_t zlen = 1;
  for (char c : os) zlen *= extent[c - 'a'];
  std::vector<double> z(zlen, 0.0);
  for (;;) {
    z[offset(os)] += static_cast<double>(x[offset(xs)]) * y[offset(ys)];
    size_t i = letters.size();
    while (i-- > 0) { if (++idx[i] < extent[letters[i] - 'a']) break; idx[i] = 0; }
    if (i == static_cast<size_t>(-1)) break;
  }
  return std::vector<float>(z.begin(), z.end());
}
static void scenario_rank_n_contractions(mp::Stream stream) {
  size_t extent[26] = {};
  extent['a' - 'a'] = 3; extent['b' - 'a'] = 8; extent['c' - 'a'] = 32; extent['d' - 'a'] = 24; extent['h' - 'a'] = 2;
  extent['i' - 'a'] = 8; extent['j' - 'a'] = 16; extent['k' - 'a'] = 12; extent['l' - 'a'] = 20; extent['q' - 'a'] = 16;
  const char* cases[][3] = {{"abc", "cd", "abd"},  {"ikj", "lk", "lij"},      {"bhqd", "bhkd", "bhqk"}, {"abc", "cd", "adb"},
                            {"ij", "jk", "ki"},    {"acb", "dc", "dab"},      {"bqhd", "bkhd", "bhqk"}, {"i", "j", "ij"},
                            {"ab", "ab", ""}};
  unsigned seed = 300;
  for (const auto& c : cases) {
    const std::string xs = c[0], ys = c[1], os = c[2], expr = xs + "," + ys + "->" + os;
    mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
    std::vector<size_t> xsz, ysz, osz;
    for (char ch : xs) xsz.push_back(extent[ch - 'a']);
    for (char ch : ys) ysz.push_back(extent[ch - 'a']);
    for (char ch : os) osz.push_back(extent[ch - 'a']);
    if (osz.empty()) osz = {1};
    mp::Tensor x = G->tensor({mp::Class::wgt, mp::Dtype::r32, xsz});
    mp::Tensor y = G->tensor({mp::Class::wgt, mp::Dtype::r32, ysz});
    mp::Tensor w = G->tensor({mp::Class::inp, mp::Dtype::r32, osz});
    const std::vector<float> hx = normal(x.len(), seed++, 1.f), hy = normal(y.len(), seed++, 0.5f), hw = normal(w.len(), seed++, 1.f);
    upload(x, hx); upload(y, hy); upload(w, hw);
    mp::Tensor z = mp::ops::inner_product(x, y, expr);
    CHECK(z.sizes() == osz);
    const double ez = rel_err(z.native(), contraction_direct(xs, ys, os, hx, hy, extent));
    mp::Tensor loss = mp::ops::hadamard(z, w);
    loss.reverse(mp::ReverseCleanup::keep);
    const double ex = rel_err(x.native_grad(), contraction_direct(os, ys, xs, hw, hy, extent));
    const double ey = rel_err(y.native_grad(), contraction_direct(xs, os, ys, hx, hw, extent));
    if (!(ez <= 1e-4 && ex <= 1e-4 && ey <= 1e-4)) std::printf("contraction %s: errors %.3g %.3g %.3g\n", expr.c_str(), ez, ex, ey);
    CHECK(ez <= 1e-4); CHECK(ex <= 1e-4); CHECK(ey <= 1e-4);
    mp::device::check();
    G->deinit();
  }
}

// Momentum steps (optimizer.zig:182-275) and weight files (graph.zig:633-703): train two steps, save, perturb,
// load, and compare with the oracle's two steps
static void scenario_momentum_and_weight_files(mp::Stream stream, const char* dir) {
  const size_t m = 6, n = 10;
  std::vector<float> hw = normal(m * n, 31, 1.f), hx = normal(m * n, 32, 1.f), mom(m * n, 0.f);
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  mp::Tensor x = G->tensor({mp::Class::inp, mp::Dtype::r32, {m, n}});
  mp::Tensor w = G->tensor({mp::Class::wgt, mp::Dtype::r32, {m, n}});
  mp::Tensor bias = G->tensor({mp::Class::wgt, mp::Dtype::r64, {n}});   // a second weight of another dtype: file index 1
  upload(x, hx); upload(w, hw); mp::algo::sequence(bias, 0.0, 0.5);
  mp::optm::Momentum opt{0.1, 0.9, mp::optm::ClipRange(-0.5, 0.5), {}};
  for (int step = 0; step < 2; ++step) {
    mp::Tensor z = mp::ops::hadamard(x, w);       // d(sum z)/dw = x
    z.reverse(mp::ReverseCleanup::free);
    opt.update(G);
    orc_momentum_f32(hw.data(), hx.data(), mom.data(), 0.1, 0.9, -0.5, 0.5, m * n);
    G->reset(mp::ResetGroup::leaf, mp::ResetComponent::grd);
    G->reset(mp::ResetGroup::node, mp::ResetComponent::all);
  }
  CHECK(rel_err(w.native(), hw) <= 1e-6);
  G->save(dir, "scenario");
  const std::vector<double> saved = w.native(), saved_bias = bias.native();
  mp::algo::fill(w, -7.0); mp::algo::fill(bias, 3.0);
  G->load(dir, "scenario");
  CHECK(w.native() == saved);
  CHECK(bias.native() == saved_bias);
  std::FILE* f = std::fopen((std::string(dir) + "/scenario_0").c_str(), "rb");
  CHECK(f != nullptr);
  if (f) { std::fseek(f, 0, SEEK_END); CHECK(std::ftell(f) == static_cast<long>(m * n * 4)); std::fclose(f); }
  f = std::fopen((std::string(dir) + "/scenario_1").c_str(), "rb");
  CHECK(f != nullptr);
  if (f) { std::fseek(f, 0, SEEK_END); CHECK(std::ftell(f) == static_cast<long>(n * 8)); std::fclose(f); }
  opt.deinit(stream);
  mp::device::check();
  G->deinit();
}

// Forward-mode `derive` (graph.zig:123-148, the per-op derive functions): hand-derivable values, and agreement with
// the reverse pass (for an element-wise f, reverse with a seed of ones leaves f'(x) in x.grad)
static void scenario_derive(mp::Stream stream) {
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  mp::Tensor x = G->tensor({mp::Class::wgt, mp::Dtype::r32, {6}});
  mp::Tensor y = G->tensor({mp::Class::inp, mp::Dtype::r32, {6}});
  mp::algo::sequence(x, -2.5, 1.0);    // -2.5 -1.5 -0.5 0.5 1.5 2.5
  mp::algo::sequence(y, 1.0, 1.0);     // 1 .. 6
  // f = x*x + 3x - relu(x):  f' = 2x + 3 - step(x)
  mp::Tensor f = mp::ops::sub(mp::ops::add(mp::ops::hadamard(x, x), mp::ops::dilate(x, 3.0)), mp::ops::relu(x));
  std::optional<mp::Tensor> df = f.derive(x);
  CHECK(df.has_value());
  if (df) CHECK((df->native() == std::vector<double>{-2, 0, 2, 3, 5, 7}));
  f.reverse(mp::ReverseCleanup::keep);
  if (df) CHECK(df->native() == x.native_grad());
  // constants: d(x + y)/dx = 1 everywhere, d(-(x + 4))/dx = -1, no dependence -> nothing
  std::optional<mp::Tensor> d1 = mp::ops::add(x, y).derive(x);
  CHECK(d1 && d1->native() == std::vector<double>(6, 1.0));
  std::optional<mp::Tensor> d2 = mp::ops::negate(mp::ops::translate(x, 4.0)).derive(x);
  CHECK(d2 && d2->native() == std::vector<double>(6, -1.0));
  CHECK(!mp::ops::dilate(y, 2.0).derive(x).has_value());
  CHECK(x.derive(x) && x.derive(x)->native() == std::vector<double>(6, 1.0));
  // chain rule through relu and a product with a constant tensor: d(relu(2x) * y)/dx = 2 step(2x) y
  std::optional<mp::Tensor> d3 = mp::ops::hadamard(mp::ops::relu(mp::ops::dilate(x, 2.0)), y).derive(x);
  CHECK(d3 && d3->native() == (std::vector<double>{0, 0, 0, 8, 10, 12}));
  // selu'(x) = lambda (x > 0), lambda alpha e^x otherwise
  std::optional<mp::Tensor> d4 = mp::ops::selu(x).derive(x);
  CHECK(d4.has_value());
  if (d4) {
    const double lam = 1.0507009873554805, al = 1.6732632423543772;
    const std::vector<double> got = d4->native();
    const double xs[6] = {-2.5, -1.5, -0.5, 0.5, 1.5, 2.5};
    for (int i = 0; i < 6; ++i) CHECK(std::fabs(got[i] - (xs[i] > 0 ? lam : lam * al * std::exp(xs[i]))) <= 1e-6);
  }
  // through a permutation: d permute(x2*x2)/dx2 = permute(2 x2)
  mp::Tensor x2 = G->tensor({mp::Class::wgt, mp::Dtype::r32, {2, 3}});
  mp::algo::sequence(x2, 1.0, 1.0);    // [[1 2 3] [4 5 6]]
  std::optional<mp::Tensor> d5 = mp::ops::permutate(mp::ops::hadamard(x2, x2), "ij->ji").derive(x2);
  CHECK(d5 && d5->sizes() == (std::vector<size_t>{3, 2}) && d5->native() == (std::vector<double>{2, 8, 4, 10, 6, 12}));
  // eval mode: no derivative
  mp::Graph* E = mp::Graph::init({stream, mp::Mode::eval});
  mp::Tensor xe = E->tensor({mp::Class::wgt, mp::Dtype::r32, {4}});
  mp::algo::fill(xe, 1.0);
  CHECK(!mp::ops::dilate(xe, 2.0).derive(xe).has_value());
  mp::device::check();
  E->deinit();
  G->deinit();
}

// Rank-3 reduce / broadcast (NOTES.md:27-35): "ijk->ik" sums over j, its reverse broadcasts the gradient back
static void scenario_rank3_reduce(mp::Stream stream) {
  mp::Graph* G = mp::Graph::init({stream, mp::Mode::train});
  const size_t I = 2, J = 3, K = 4;
  mp::Tensor x = G->tensor({mp::Class::wgt, mp::Dtype::r32, {I, J, K}});
  mp::algo::sequence(x, 1.0, 1.0);     // x[i,j,k] = 1 + (i*J + j)*K + k
  auto at = [&](size_t i, size_t j, size_t k) { return 1.0 + (i * J + j) * K + k; };
  struct Case { const char* expr; std::vector<size_t> out; };
  const Case cases[] = {{"ijk->ij", {I, J}}, {"ijk->jk", {J, K}}, {"ijk->ik", {I, K}}, {"ijk->j", {J}}, {"ijk->ki", {K, I}},
                        {"ijk->k", {K}}, {"ijk->i", {I}}};
  for (const Case& c : cases) {
    mp::Tensor y = mp::ops::reduce(x, c.expr);
    CHECK(y.sizes() == c.out);
    const std::string rhs = std::string(c.expr).substr(5);
    std::vector<double> want(y.len(), 0.0);
    for (size_t i = 0; i < I; ++i) for (size_t j = 0; j < J; ++j) for (size_t k = 0; k < K; ++k) {
      size_t o = 0;
      for (char ch : rhs) o = o * (ch == 'i' ? I : ch == 'j' ? J : K) + (ch == 'i' ? i : ch == 'j' ? j : k);
      want[o] += at(i, j, k);
    }
    CHECK(y.native() == want);
  }
  // reverse of "ijk->ik" weighted by w[i,k]: x.grad[i,j,k] = w[i,k]
  mp::Tensor w = G->tensor({mp::Class::inp, mp::Dtype::r32, {I, K}});
  mp::algo::sequence(w, 0.5, 0.5);
  mp::Tensor z = mp::ops::hadamard(mp::ops::reduce(x, "ijk->ik"), w);
  z.reverse(mp::ReverseCleanup::keep);
  std::vector<double> gwant(I * J * K);
  for (size_t i = 0; i < I; ++i) for (size_t j = 0; j < J; ++j) for (size_t k = 0; k < K; ++k) gwant[(i * J + j) * K + k] = 0.5 + 0.5 * (i * K + k);
  CHECK(x.native_grad() == gwant);
  // broadcast "ik->ijk" equals that gradient pattern; its reverse sums over j
  mp::Tensor v = G->tensor({mp::Class::wgt, mp::Dtype::r32, {I, K}});
  mp::algo::sequence(v, 0.5, 0.5);
  mp::Tensor b = mp::ops::broadcast(v, {I, J, K}, "ik->ijk");
  CHECK(b.native() == gwant);
  mp::Tensor b2 = mp::ops::broadcast(v, {K, J, I}, "ik->kji");   // target order differs from the source order
  std::vector<double> want2(I * J * K);
  for (size_t k = 0; k < K; ++k) for (size_t j = 0; j < J; ++j) for (size_t i = 0; i < I; ++i) want2[(k * J + j) * I + i] = 0.5 + 0.5 * (i * K + k);
  CHECK(b2.native() == want2);
  b.reverse(mp::ReverseCleanup::keep);
  CHECK(v.native_grad() == std::vector<double>(I * K, static_cast<double>(J)));
  mp::device::check();
  G->deinit();
}

int main(int argc, char** argv) {
  const int timing_iters = argc > 1 ? std::atoi(argv[1]) : 0;
  mp::device::init(0);
  std::printf("device memory: %zu bytes\n", mp::device::total_memory(0));
  mp::Stream s = mp::stream::init();
  scenario_subgraphs(s);
  scenario_experimental(s);
  scenario_feed_forward(s, timing_iters);
  scenario_matrix_vector(s);
  scenario_row_ops(s);
  scenario_rank3(s);
  scenario_derive(s);
  scenario_rank3_reduce(s);
  scenario_rank_n_contractions(s);
  scenario_momentum_and_weight_files(s, argc > 2 ? argv[2] : "/tmp");
  mp::stream::deinit(s);
  std::printf(failures == 0 ? "ALL SCENARIOS PASSED\n" : "%d CHECKS FAILED\n", failures);
  return failures == 0 ? 0 : 1;
}
