// CPU check of the host mirror's rank-N contraction planner (mp::ops::contraction_plan): every plan is carried out
// here with plain loops (permutations, one batched matrix product of the planned form, the output permutation) and
// compared with the contraction summed straight from its expression.  The reverse of "x,y->z" runs the expressions
// "z,y->x" and "x,z->y", so those are planned and checked for every case as well.  No device call is made.
// Usage: contraction_plans; exit code 0 = all checks passed.
#include <cmath>
#include <cstdio>
#include <map>
#include <random>
#include <string>
#include <vector>

#include "../../metaphor_b200/host/metaphor.hpp"

static int failures = 0;

static size_t volume(const std::vector<size_t>& s) { size_t v = 1; for (size_t e : s) v *= e; return v; }

// dst[.. perm ..] = src: perm[i] = position of the source's i-th index in the destination
static std::vector<double> permuted(const std::vector<double>& src, const std::vector<size_t>& sizes, const std::vector<size_t>& perm) {
  const size_t r = sizes.size();
  std::vector<size_t> dsz(r), dstride(r), idx(r, 0);
  for (size_t i = 0; i < r; ++i) dsz[perm[i]] = sizes[i];
  size_t s = 1;
  for (size_t i = r; i-- > 0;) { dstride[i] = s; s *= dsz[i]; }
  std::vector<double> dst(src.size());
  for (size_t lin = 0; lin < src.size(); ++lin) {
    size_t off = 0;
    for (size_t i = 0; i < r; ++i) off += idx[i] * dstride[perm[i]];
    dst[off] = src[lin];
    for (size_t i = r; i-- > 0;) { if (++idx[i] < sizes[i]) break; idx[i] = 0; }
  }
  return dst;
}

// the contraction summed from its expression, index by index
static std::vector<double> direct(const std::string& xs, const std::string& ys, const std::string& os, const std::vector<double>& x,
                                  const std::vector<double>& y, const std::map<char, size_t>& extent) {
  std::string letters;
  for (char c : xs + ys + os) if (letters.find(c) == std::string::npos) letters += c;
  std::vector<size_t> idx(letters.size(), 0);
  auto offset = [&](const std::string& s) {
    size_t off = 0;
    for (char c : s) off = off * extent.at(c) + idx[letters.find(c)];
    return off;
  };
  size_t zlen = 1;
  for (char c : os) zlen *= extent.at(c);
  std::vector<double> z(zlen, 0.0);
  for (;;) {
    z[offset(os)] += x[offset(xs)] * y[offset(ys)];
    size_t i = letters.size();
    while (i-- > 0) { if (++idx[i] < extent.at(letters[i])) break; idx[i] = 0; }
    if (i == static_cast<size_t>(-1)) break;
  }
  return z;
}

static void check_case(const std::string& xs, const std::string& ys, const std::string& os, const std::map<char, size_t>& extent, unsigned seed) {
  std::vector<size_t> xsz, ysz;
  for (char c : xs) xsz.push_back(extent.at(c));
  for (char c : ys) ysz.push_back(extent.at(c));
  std::mt19937 gen(seed);
  std::uniform_real_distribution<double> d(-1.0, 1.0);
  std::vector<double> x(volume(xsz)), y(volume(ysz));
  for (auto& v : x) v = d(gen);
  for (auto& v : y) v = d(gen);
  const std::string expr = xs + "," + ys + "->" + os;
  const mp::ops::ContractionPlan p = mp::ops::contraction_plan(expr, xsz, ysz);
  const std::vector<double>* a = p.swap ? &y : &x;
  const std::vector<double>* b = p.swap ? &x : &y;
  const std::vector<size_t>& asz = p.swap ? ysz : xsz;
  const std::vector<size_t>& bsz = p.swap ? xsz : ysz;
  std::vector<double> at, bt;
  if (!p.x_perm.empty()) { at = permuted(*a, asz, p.x_perm); a = &at; }
  if (!p.y_perm.empty()) { bt = permuted(*b, bsz, p.y_perm); b = &bt; }
  const size_t nb = p.batch == 0 ? 1 : p.batch, M = p.m, N = p.n, K = p.k;
  bool ok = a->size() == nb * M * N && b->size() == nb * N * K;
  std::vector<double> c(nb * M * K, 0.0);
  if (ok)
    for (size_t q = 0; q < nb; ++q)
      for (size_t i = 0; i < M; ++i)
        for (size_t k = 0; k < K; ++k) {
          double acc = 0.0;
          for (size_t j = 0; j < N; ++j) {
            const double av = p.kind == 2 ? (*a)[(q * N + j) * M + i] : (*a)[(q * M + i) * N + j];
            const double bv = p.kind == 1 ? (*b)[(q * K + k) * N + j] : (*b)[(q * N + j) * K + k];
            acc += av * bv;
          }
          c[(q * M + i) * K + k] = acc;
        }
  if (ok && !p.z_perm.empty()) { ok = volume(p.z_sizes) == c.size(); if (ok) c = permuted(c, p.z_sizes, p.z_perm); }
  const std::vector<double> ref = direct(xs, ys, os, x, y, extent);
  std::vector<size_t> osz;
  for (char ch : os) osz.push_back(extent.at(ch));
  if (osz.empty()) osz = {1};
  ok = ok && p.out_sizes == osz && c.size() == ref.size();
  double err = 0.0;
  if (ok) for (size_t i = 0; i < ref.size(); ++i) err = std::fmax(err, std::fabs(c[i] - ref[i]));
  if (!ok || err > 1e-12) {
    std::printf("FAILED %s (swap %d kind %d batch %zu m %zu n %zu k %zu, error %.3g)\n", expr.c_str(), int(p.swap), p.kind, p.batch, p.m,
                p.n, p.k, err);
    ++failures;
  }
}

struct Expect { const char* expr; bool swap; int kind; bool x_moved, y_moved, z_moved; };

int main() {
  const std::map<char, size_t> extent = {{'a', 3}, {'b', 2}, {'c', 5}, {'d', 4}, {'e', 2}, {'f', 3}, {'i', 4}, {'j', 6}, {'k', 5},
                                         {'l', 3}, {'h', 2}, {'q', 3}, {'p', 2}};
  const char* cases[][3] = {
      {"ij", "jk", "ik"},         {"ij", "kj", "ik"},       {"ji", "jk", "ik"},        {"ji", "kj", "ik"},     {"ij", "jk", "ki"},
      {"abc", "cd", "abd"},       {"abc", "dc", "abd"},     {"cab", "cd", "abd"},      {"acb", "cd", "abd"},   {"abc", "cd", "dab"},
      {"abc", "cd", "adb"},       {"ikj", "lk", "lij"},     {"bij", "bjk", "bik"},     {"bij", "bkj", "bik"},  {"ibj", "bjk", "bik"},
      {"bhqd", "bhkd", "bhqk"},   {"bhqk", "bhkd", "bhqd"}, {"bqhd", "bkhd", "bhqk"},  {"abcd", "cdef", "abef"}, {"abcd", "dcef", "abef"},
      {"i", "ij", "j"},           {"ij", "j", "i"},         {"i", "j", "ij"},          {"i", "i", ""},          {"bi", "bi", "b"},
      {"abcdef", "fedc", "ab"},   {"ab", "bcdefi", "acdefi"}, {"pij", "pjk", "ipk"},   {"aij", "ajk", "kai"},
  };
  unsigned seed = 1;
  for (const auto& c : cases) {
    const std::string xs = c[0], ys = c[1], os = c[2];
    check_case(xs, ys, os, extent, seed++);
    check_case(os, ys, xs, extent, seed++);   // gradient of the first operand
    check_case(xs, os, ys, extent, seed++);   // gradient of the second operand
  }
  // which operands move: orders a kernel takes directly stay where they lie
  const Expect expects[] = {
      {"ij,jk->ik", false, 0, false, false, false},   {"ij,kj->ik", false, 1, false, false, false},
      {"ji,jk->ik", false, 2, false, false, false},   {"ji,kj->ik", false, 2, false, true, false},
      {"ij,jk->ki", true, 2, false, true, false},     {"abc,cd->abd", false, 0, false, false, false},
      {"abc,dc->abd", false, 1, false, false, false}, {"cab,cd->abd", false, 2, false, false, false},
      {"acb,cd->abd", false, 0, true, false, false},  {"abc,cd->adb", false, 0, false, false, true},
      {"bhqd,bhkd->bhqk", false, 1, false, false, false}, {"bhqk,bhkd->bhqd", false, 0, false, false, false},
      {"abcd,cdef->abef", false, 0, false, false, false},
  };
  for (const Expect& e : expects) {
    const std::string expr = e.expr;
    const size_t comma = expr.find(','), arrow = expr.find("->");
    std::vector<size_t> xsz, ysz;
    for (char ch : expr.substr(0, comma)) xsz.push_back(extent.at(ch));
    for (char ch : expr.substr(comma + 1, arrow - comma - 1)) ysz.push_back(extent.at(ch));
    const mp::ops::ContractionPlan p = mp::ops::contraction_plan(expr, xsz, ysz);
    if (p.swap != e.swap || p.kind != e.kind || !p.x_perm.empty() != e.x_moved || !p.y_perm.empty() != e.y_moved ||
        !p.z_perm.empty() != e.z_moved) {
      std::printf("UNEXPECTED PLAN %s: swap %d kind %d moved %d %d %d\n", e.expr, int(p.swap), p.kind, int(!p.x_perm.empty()),
                  int(!p.y_perm.empty()), int(!p.z_perm.empty()));
      ++failures;
    }
  }
  if (failures == 0) std::printf("ALL PLANS PASSED\n");
  return failures == 0 ? 0 : 1;
}
