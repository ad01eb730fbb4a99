// Row-wise softmax and RMSNorm over the last axis of a row-major [m, n]
// matrix, forward and reverse.  HBM-bound: each row is read from global memory
// exactly once with 128-bit loads, lives in registers while its statistics are
// reduced (warp shuffles, plus one shared-memory hop when a row spans several
// warps), and is written once.  A row is owned by GROUP threads: one warp for
// short rows (four rows per CTA) or the whole CTA; CTAs walk the rows
// grid-stride so that per-column state (gain, gain-gradient partials) is
// loaded or accumulated once per CTA, not once per row.
//
// The reference has no kernel for these ops; the op naming follows its "ij|j"
// transform grammar (src/ops/expression_parsing.zig:319-340).
#include "mp_common.cuh"

#include <cfloat>

namespace {

template <int GROUP>
struct RowCfg {
  static constexpr int THREADS = GROUP < 128 ? 128 : GROUP;
  static constexpr int ROWS = THREADS / GROUP;  // rows in flight per CTA
};

__device__ __forceinline__ float mp_neg_inf(float) { return -INFINITY; }
__device__ __forceinline__ double mp_neg_inf(double) { return -INFINITY; }
__device__ __forceinline__ float mp_exp_diff(float x, float mx) {
  return exp2f((x - mx) * 1.4426950408889634f);
}
__device__ __forceinline__ double mp_exp_diff(double x, double mx) { return exp(x - mx); }
__device__ __forceinline__ float mp_rsqrt(float x) { return 1.0f / sqrtf(x); }
__device__ __forceinline__ double mp_rsqrt(double x) { return 1.0 / sqrt(x); }

template <typename Op, int GROUP, typename A>
__device__ __forceinline__ A group_reduce(A v, A* smem, A identity) {
  if constexpr (GROUP == 32) return warp_reduce<Op>(v);
  else return cta_reduce<Op, GROUP>(v, smem, identity);
}

// Two sums at once (one barrier pair instead of two).
template <int GROUP, typename A>
__device__ __forceinline__ void group_sum2(A& a, A& b, A* smem) {
  a = warp_reduce<SumOp>(a);
  b = warp_reduce<SumOp>(b);
  if constexpr (GROUP > 32) {
    constexpr int WARPS = GROUP / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { smem[warp] = a; smem[32 + warp] = b; }
    __syncthreads();
    A ra = lane < WARPS ? smem[lane] : A(0);
    A rb = lane < WARPS ? smem[32 + lane] : A(0);
    a = warp_reduce<SumOp>(ra);
    b = warp_reduce<SumOp>(rb);
    __syncthreads();
  }
}

// ------------------------------- softmax ----------------------------------
template <typename T, int GROUP, int PPT>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) softmax_fwd_kernel(const T* x, T* y,
                                                                            size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int ROWS = RowCfg<GROUP>::ROWS;
  __shared__ A red[64];
  const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
  const size_t nv = n / PN;
  for (size_t row = static_cast<size_t>(blockIdx.x) * ROWS + g; row < m; row += static_cast<size_t>(gridDim.x) * ROWS) {
    const T* xr = x + row * n;
    T* yr = y + row * n;
    Pack<T> p[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) p[u] = ld_pack_stream(xr, v);
    }
    A e[PPT][PN];
    A mx = mp_neg_inf(A(0));
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
#pragma unroll
      for (int k = 0; k < PN; ++k) {
        e[u][k] = mp_up(p[u].v[k]);
        if (v < nv) mx = MaxOp::apply(mx, e[u][k]);
      }
    }
    mx = group_reduce<MaxOp, GROUP>(mx, red, mp_neg_inf(A(0)));
    A sum = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
#pragma unroll
      for (int k = 0; k < PN; ++k) {
        e[u][k] = mp_exp_diff(e[u][k], mx);
        if (v < nv) sum += e[u][k];
      }
    }
    sum = group_reduce<SumOp, GROUP>(sum, red, A(0));
    const A inv = A(1) / sum;
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
        Pack<T> o;
#pragma unroll
        for (int k = 0; k < PN; ++k) o.v[k] = mp_down<T>(e[u][k] * inv);
        st_pack_stream(yr, v, o);
      }
    }
  }
}

// gx = y o (gy - <gy, y>) + alpha*gx
template <typename T, int GROUP, int PPT, bool BLEND>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) softmax_rev_kernel(const T* y, const T* gy,
                                                                            T* gx, typename Acc<T>::type alpha, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int ROWS = RowCfg<GROUP>::ROWS;
  __shared__ A red[64];
  const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
  const size_t nv = n / PN;
  for (size_t row = static_cast<size_t>(blockIdx.x) * ROWS + g; row < m; row += static_cast<size_t>(gridDim.x) * ROWS) {
    const T* yr = y + row * n;
    const T* gr = gy + row * n;
    T* xr = gx + row * n;
    Pack<T> py[PPT], pg[PPT], po[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
        py[u] = ld_pack_stream(yr, v);
        pg[u] = ld_pack_stream(gr, v);
        if constexpr (BLEND) po[u] = ld_pack_stream(xr, v);
      }
    }
    A dot = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
#pragma unroll
        for (int k = 0; k < PN; ++k) dot += mp_up(py[u].v[k]) * mp_up(pg[u].v[k]);
      }
    }
    dot = group_reduce<SumOp, GROUP>(dot, red, A(0));
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
        Pack<T> o;
#pragma unroll
        for (int k = 0; k < PN; ++k) {
          A r = mp_up(py[u].v[k]) * (mp_up(pg[u].v[k]) - dot);
          if constexpr (BLEND) r += alpha * mp_up(po[u].v[k]);
          o.v[k] = mp_down<T>(r);
        }
        st_pack_stream(xr, v, o);
      }
    }
  }
}

// ------------------------------- RMSNorm ----------------------------------
template <typename T, int GROUP, int PPT>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gain,
                                                                            typename Acc<T>::type eps, T* y,
                                                                            typename Acc<T>::type* __restrict__ rstd_out,
                                                                            size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int ROWS = RowCfg<GROUP>::ROWS;
  __shared__ A red[64];
  const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
  const size_t nv = n / PN;
  Pack<T> pgain[PPT];
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const size_t v = t + static_cast<size_t>(u) * GROUP;
    if (v < nv) pgain[u] = ld_pack(gain, v);
  }
  const A inv_n = A(1) / static_cast<A>(n);
  for (size_t row = static_cast<size_t>(blockIdx.x) * ROWS + g; row < m; row += static_cast<size_t>(gridDim.x) * ROWS) {
    const T* xr = x + row * n;
    T* yr = y + row * n;
    Pack<T> p[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) p[u] = ld_pack_stream(xr, v);
    }
    A ss = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
#pragma unroll
        for (int k = 0; k < PN; ++k) { const A a = mp_up(p[u].v[k]); ss += a * a; }
      }
    }
    ss = group_reduce<SumOp, GROUP>(ss, red, A(0));
    const A rstd = mp_rsqrt(ss * inv_n + eps);
    if (rstd_out != nullptr && t == 0) rstd_out[row] = rstd;
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
        Pack<T> o;
#pragma unroll
        for (int k = 0; k < PN; ++k) o.v[k] = mp_down<T>(mp_up(p[u].v[k]) * rstd * mp_up(pgain[u].v[k]));
        st_pack_stream(yr, v, o);
      }
    }
  }
}

// gx = rstd*(gy o gain) - x*rstd^3*mean_j(gy o gain o x) + alpha*gx, and the
// CTA's partial of ggain_j = sum_i gy_ij*x_ij*rstd_i into partial[slot][n],
// slot = blockIdx.x*ROWS + row-group.  Both row sums are independent of each
// other, so they share one reduction.
template <typename T, int GROUP, int PPT, bool BLEND>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) rmsnorm_rev_kernel(
    const T* x, const T* __restrict__ gain, const typename Acc<T>::type* __restrict__ rstd_in,
    const T* gy, typename Acc<T>::type eps, T* gx, typename Acc<T>::type alpha,
    typename Acc<T>::type* __restrict__ partial, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int ROWS = RowCfg<GROUP>::ROWS;
  __shared__ A red[64];
  const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
  const size_t nv = n / PN;
  Pack<T> pgain[PPT];
  A acc[PPT][PN];
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const size_t v = t + static_cast<size_t>(u) * GROUP;
    if (v < nv) pgain[u] = ld_pack(gain, v);
#pragma unroll
    for (int k = 0; k < PN; ++k) acc[u][k] = A(0);
  }
  const A inv_n = A(1) / static_cast<A>(n);
  for (size_t row = static_cast<size_t>(blockIdx.x) * ROWS + g; row < m; row += static_cast<size_t>(gridDim.x) * ROWS) {
    const T* xr = x + row * n;
    const T* gr = gy + row * n;
    T* or_ = gx + row * n;
    Pack<T> px[PPT], pg[PPT], po[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
        px[u] = ld_pack_stream(xr, v);
        pg[u] = ld_pack_stream(gr, v);
        if constexpr (BLEND) po[u] = ld_pack_stream(or_, v);
      }
    }
    A ss = A(0), dot = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
#pragma unroll
        for (int k = 0; k < PN; ++k) {
          const A a = mp_up(px[u].v[k]);
          ss += a * a;
          dot += mp_up(pg[u].v[k]) * mp_up(pgain[u].v[k]) * a;
        }
      }
    }
    group_sum2<GROUP>(ss, dot, red);
    const A rstd = rstd_in != nullptr ? rstd_in[row] : mp_rsqrt(ss * inv_n + eps);
    const A coef = rstd * rstd * rstd * dot * inv_n;
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      const size_t v = t + static_cast<size_t>(u) * GROUP;
      if (v < nv) {
        Pack<T> o;
#pragma unroll
        for (int k = 0; k < PN; ++k) {
          const A a = mp_up(px[u].v[k]);
          const A gk = mp_up(pg[u].v[k]);
          A r = rstd * gk * mp_up(pgain[u].v[k]) - a * coef;
          if constexpr (BLEND) r += alpha * mp_up(po[u].v[k]);
          o.v[k] = mp_down<T>(r);
          acc[u][k] += gk * a * rstd;
        }
        st_pack_stream(or_, v, o);
      }
    }
  }
  A* pr = partial + (static_cast<size_t>(blockIdx.x) * ROWS + g) * n;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const size_t v = t + static_cast<size_t>(u) * GROUP;
    if (v < nv) {
#pragma unroll
      for (int k = 0; k < PN; ++k) pr[v * PN + k] = acc[u][k];
    }
  }
}

// ggain[j] = sum_p partial[p][j] + alpha*ggain[j].  CTA = 32 columns x 8 slices.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_fold_kernel(const typename Acc<T>::type* __restrict__ partial, T* ggain,
                                                           typename Acc<T>::type alpha, bool blend, size_t n, size_t slots) {
  using A = typename Acc<T>::type;
  __shared__ A sm[8][33];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const size_t col = static_cast<size_t>(blockIdx.x) * 32 + lane;
  A s = A(0);
  if (col < n) {
    for (size_t p = slice; p < slots; p += 8) s += partial[p * n + col];
  }
  sm[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && col < n) {
    A r = A(0);
#pragma unroll
    for (int w = 0; w < 8; ++w) r += sm[w][lane];
    ggain[col] = mp_down<T>(blend ? r + alpha * mp_up(ggain[col]) : r);
  }
}

// --------------------- generic fallback (any n, any alignment) ------------
// One CTA per row, scalar coalesced accesses, the row is re-read from L2 for
// each pass.  Used when n is not a multiple of the pack width, a pointer is
// not 16-byte aligned, or the row does not fit the register-resident kernels.
constexpr int GEN_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) softmax_fwd_generic(const T* x, T* y, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  __shared__ A red[64];
  for (size_t row = blockIdx.x; row < m; row += gridDim.x) {
    const T* xr = x + row * n; T* yr = y + row * n;
    A mx = mp_neg_inf(A(0));
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) mx = MaxOp::apply(mx, mp_up(xr[j]));
    mx = cta_reduce<MaxOp, GEN_THREADS>(mx, red, mp_neg_inf(A(0)));
    A sum = A(0);
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) sum += mp_exp_diff(mp_up(xr[j]), mx);
    sum = cta_reduce<SumOp, GEN_THREADS>(sum, red, A(0));
    const A inv = A(1) / sum;
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) yr[j] = mp_down<T>(mp_exp_diff(mp_up(xr[j]), mx) * inv);
  }
}

template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) softmax_rev_generic(const T* y, const T* gy, T* gx, typename Acc<T>::type alpha,
                                                                   bool blend, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  __shared__ A red[64];
  for (size_t row = blockIdx.x; row < m; row += gridDim.x) {
    const T* yr = y + row * n; const T* gr = gy + row * n; T* xr = gx + row * n;
    A dot = A(0);
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) dot += mp_up(yr[j]) * mp_up(gr[j]);
    dot = cta_reduce<SumOp, GEN_THREADS>(dot, red, A(0));
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) {
      A r = mp_up(yr[j]) * (mp_up(gr[j]) - dot);
      if (blend) r += alpha * mp_up(xr[j]);
      xr[j] = mp_down<T>(r);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) rmsnorm_fwd_generic(const T* x, const T* gain, typename Acc<T>::type eps, T* y,
                                                                   typename Acc<T>::type* rstd_out, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  __shared__ A red[64];
  const A inv_n = A(1) / static_cast<A>(n);
  for (size_t row = blockIdx.x; row < m; row += gridDim.x) {
    const T* xr = x + row * n; T* yr = y + row * n;
    A ss = A(0);
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) { const A a = mp_up(xr[j]); ss += a * a; }
    ss = cta_reduce<SumOp, GEN_THREADS>(ss, red, A(0));
    const A rstd = mp_rsqrt(ss * inv_n + eps);
    if (rstd_out != nullptr && threadIdx.x == 0) rstd_out[row] = rstd;
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) yr[j] = mp_down<T>(mp_up(xr[j]) * rstd * mp_up(gain[j]));
  }
}

// Partials of ggain: CTA b accumulates its rows into partial[b][n] (read-modify-
// write of its own private row of the scratch, zeroed first by the same CTA).
template <typename T>
__global__ void __launch_bounds__(GEN_THREADS) rmsnorm_rev_generic(const T* x, const T* gain, const typename Acc<T>::type* rstd_in,
                                                                   const T* gy, typename Acc<T>::type eps, T* gx,
                                                                   typename Acc<T>::type alpha, bool blend,
                                                                   typename Acc<T>::type* partial, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  __shared__ A red[64];
  const A inv_n = A(1) / static_cast<A>(n);
  A* pr = partial + static_cast<size_t>(blockIdx.x) * n;
  for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) pr[j] = A(0);
  for (size_t row = blockIdx.x; row < m; row += gridDim.x) {
    const T* xr = x + row * n; const T* gr = gy + row * n; T* or_ = gx + row * n;
    A ss = A(0), dot = A(0);
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) {
      const A a = mp_up(xr[j]);
      ss += a * a;
      dot += mp_up(gr[j]) * mp_up(gain[j]) * a;
    }
    group_sum2<GEN_THREADS>(ss, dot, red);
    const A rstd = rstd_in != nullptr ? rstd_in[row] : mp_rsqrt(ss * inv_n + eps);
    const A coef = rstd * rstd * rstd * dot * inv_n;
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) {
      const A a = mp_up(xr[j]);
      const A gk = mp_up(gr[j]);
      A r = rstd * gk * mp_up(gain[j]) - a * coef;
      if (blend) r += alpha * mp_up(or_[j]);
      or_[j] = mp_down<T>(r);
      pr[j] += gk * a * rstd;  // column j is owned by this thread for every row
    }
  }
}

// ------------------------------ planning ----------------------------------
struct RowPlan {
  bool generic;
  int group, ppt, threads, rows;
};

template <typename T>
RowPlan plan_rows(size_t n, bool aligned) {
  constexpr int PN = Pack<T>::N;
  RowPlan p{true, GEN_THREADS, 0, GEN_THREADS, 1};
  if (!aligned || n % PN != 0 || n == 0) return p;
  const size_t nv = n / PN;
  int group;
  if (nv <= 32 * 4) group = 32;
  else if (nv <= 128 * 4) group = 128;
  else if (nv <= 256 * 4) group = 256;
  else if (nv <= 512 * 4) group = 512;
  else return p;
  const size_t need = (nv + group - 1) / group;
  p.generic = false;
  p.group = group;
  p.ppt = need <= 1 ? 1 : (need <= 2 ? 2 : 4);
  if (group >= 256) p.ppt = 4;
  if (group == 128 && p.ppt == 1) p.ppt = 2;
  p.threads = group < 128 ? 128 : group;
  p.rows = p.threads / group;
  return p;
}

// CTAs per SM that keep roughly 2048 (streaming kernels) or 1024 (register-
// heavy reverse kernels) threads resident.
inline size_t row_grid(const RowPlan& p, size_t m, int sm_count, int threads_per_sm) {
  size_t per_sm = static_cast<size_t>(threads_per_sm / p.threads);
  if (per_sm < 1) per_sm = 1;
  size_t grid = (m + p.rows - 1) / p.rows;
  const size_t cap = static_cast<size_t>(sm_count) * per_sm;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return grid;
}

#define MP_ROW_DISPATCH(PLAN, CALL)                                         \
  do {                                                                      \
    if ((PLAN).group == 32 && (PLAN).ppt == 1) { CALL(32, 1); }             \
    else if ((PLAN).group == 32 && (PLAN).ppt == 2) { CALL(32, 2); }        \
    else if ((PLAN).group == 32) { CALL(32, 4); }                           \
    else if ((PLAN).group == 128 && (PLAN).ppt == 2) { CALL(128, 2); }      \
    else if ((PLAN).group == 128) { CALL(128, 4); }                         \
    else if ((PLAN).group == 256) { CALL(256, 4); }                         \
    else { CALL(512, 4); }                                                  \
  } while (0)

constexpr int REV_THREADS_PER_SM = 1024;

}  // namespace

template <typename T>
static void softmax_ij_j_impl(const void* src_, void* dst_, len_t m, len_t n, StreamContext ctx) {
  if (m == 0 || n == 0) return;
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  const RowPlan p = plan_rows<T>(n, mp_aligned16(src) && mp_aligned16(dst));
  cudaStream_t st = mp_stream(ctx);
  const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), 2048));
  if (p.generic) {
    softmax_fwd_generic<T><<<grid, GEN_THREADS, 0, st>>>(src, dst, m, n);
  } else {
#define CALL(G, P) softmax_fwd_kernel<T, G, P><<<grid, RowCfg<G>::THREADS, 0, st>>>(src, dst, m, n)
    MP_ROW_DISPATCH(p, CALL);
#undef CALL
  }
  MP_LAUNCH_CHECK();
}

template <typename T>
static void softmax_ij_j_reverse_impl(const void* y_, const void* gy_, void* gx_, double alpha, len_t m, len_t n,
                                      StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (m == 0 || n == 0) return;
  const T* y = static_cast<const T*>(y_);
  const T* gy = static_cast<const T*>(gy_);
  T* gx = static_cast<T*>(gx_);
  const RowPlan p = plan_rows<T>(n, mp_aligned16(y) && mp_aligned16(gy) && mp_aligned16(gx));
  cudaStream_t st = mp_stream(ctx);
  const A a = static_cast<A>(alpha);
  const bool blend = alpha != 0.0;
  const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), 2048));
  if (p.generic) {
    softmax_rev_generic<T><<<grid, GEN_THREADS, 0, st>>>(y, gy, gx, a, blend, m, n);
  } else if (blend) {
#define CALL(G, P) softmax_rev_kernel<T, G, P, true><<<grid, RowCfg<G>::THREADS, 0, st>>>(y, gy, gx, a, m, n)
    MP_ROW_DISPATCH(p, CALL);
#undef CALL
  } else {
#define CALL(G, P) softmax_rev_kernel<T, G, P, false><<<grid, RowCfg<G>::THREADS, 0, st>>>(y, gy, gx, a, m, n)
    MP_ROW_DISPATCH(p, CALL);
#undef CALL
  }
  MP_LAUNCH_CHECK();
}

template <typename T>
static void rmsnorm_ij_j_impl(const void* x_, const void* gain_, double eps, void* y_, void* rstd_, len_t m, len_t n,
                              StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (m == 0 || n == 0) return;
  const T* x = static_cast<const T*>(x_);
  const T* gain = static_cast<const T*>(gain_);
  T* y = static_cast<T*>(y_);
  A* rstd = static_cast<A*>(rstd_);
  const RowPlan p = plan_rows<T>(n, mp_aligned16(x) && mp_aligned16(gain) && mp_aligned16(y));
  cudaStream_t st = mp_stream(ctx);
  const A e = static_cast<A>(eps);
  const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), 2048));
  if (p.generic) {
    rmsnorm_fwd_generic<T><<<grid, GEN_THREADS, 0, st>>>(x, gain, e, y, rstd, m, n);
  } else {
#define CALL(G, P) rmsnorm_fwd_kernel<T, G, P><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, e, y, rstd, m, n)
    MP_ROW_DISPATCH(p, CALL);
#undef CALL
  }
  MP_LAUNCH_CHECK();
}

// Number of partial rows the reverse kernel writes for this shape and device.
// The plan only looks at n and at whether the pointers are aligned; the
// scratch is sized for the larger of the two possible plans.
template <typename T>
static size_t rmsnorm_rev_slots(size_t m, size_t n, int sm_count, bool aligned) {
  const RowPlan p = plan_rows<T>(n, aligned);
  return row_grid(p, m, sm_count, REV_THREADS_PER_SM) * p.rows;
}

template <typename T>
static void rmsnorm_ij_j_reverse_impl(const void* x_, const void* gain_, const void* rstd_, const void* gy_, double eps,
                                      void* gx_, void* ggain_, double alpha, void* scratch, len_t m, len_t n,
                                      StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (n == 0) return;
  const T* x = static_cast<const T*>(x_);
  const T* gain = static_cast<const T*>(gain_);
  const A* rstd = static_cast<const A*>(rstd_);
  const T* gy = static_cast<const T*>(gy_);
  T* gx = static_cast<T*>(gx_);
  T* ggain = static_cast<T*>(ggain_);
  A* partial = static_cast<A*>(scratch);
  cudaStream_t st = mp_stream(ctx);
  const A a = static_cast<A>(alpha);
  const A e = static_cast<A>(eps);
  const bool blend = alpha != 0.0;
  size_t slots = 0;
  if (m > 0) {
    if (scratch == nullptr) MP_FATAL("rmsnorm_ij_j_reverse: scratch must not be NULL");
    const bool aligned = mp_aligned16(x) && mp_aligned16(gain) && mp_aligned16(gy) && mp_aligned16(gx);
    const RowPlan p = plan_rows<T>(n, aligned);
    const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), REV_THREADS_PER_SM));
    slots = static_cast<size_t>(grid) * p.rows;
    if (p.generic) {
      rmsnorm_rev_generic<T><<<grid, GEN_THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, blend, partial, m, n);
    } else if (blend) {
#define CALL(G, P) rmsnorm_rev_kernel<T, G, P, true><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m, n)
      MP_ROW_DISPATCH(p, CALL);
#undef CALL
    } else {
#define CALL(G, P) rmsnorm_rev_kernel<T, G, P, false><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m, n)
      MP_ROW_DISPATCH(p, CALL);
#undef CALL
    }
    MP_LAUNCH_CHECK();
  }
  rmsnorm_fold_kernel<T><<<static_cast<unsigned>((n + 31) / 32), 256, 0, st>>>(partial, ggain, a, blend, n, slots);
  MP_LAUNCH_CHECK();
}

extern "C" len_t mpRmsnormReverseScratchBytes(len_t m, len_t n, StreamContext ctx) {
  const int sms = mp_sm_count(ctx);
  // Upper bound over dtypes and over the aligned / generic plans.
  size_t slots = 1;
  const size_t cand[] = {
      rmsnorm_rev_slots<__half>(m, n, sms, true), rmsnorm_rev_slots<__half>(m, n, sms, false),
      rmsnorm_rev_slots<float>(m, n, sms, true),  rmsnorm_rev_slots<float>(m, n, sms, false),
      rmsnorm_rev_slots<double>(m, n, sms, true), rmsnorm_rev_slots<double>(m, n, sms, false)};
  for (size_t c : cand) if (c > slots) slots = c;
  return static_cast<len_t>(slots * n * sizeof(double));
}

MP_STAMP3(softmax_ij_j, (const void* src, void* dst, len_t m, len_t n, StreamContext ctx), (src, dst, m, n, ctx))
MP_STAMP3(softmax_ij_j_reverse, (const void* y, const void* gy, void* gx, double alpha, len_t m, len_t n, StreamContext ctx), (y, gy, gx, alpha, m, n, ctx))
MP_STAMP3(rmsnorm_ij_j, (const void* x, const void* gain, double eps, void* y, void* rstd, len_t m, len_t n, StreamContext ctx), (x, gain, eps, y, rstd, m, n, ctx))
MP_STAMP3(rmsnorm_ij_j_reverse, (const void* x, const void* gain, const void* rstd, const void* gy, double eps, void* gx, void* ggain, double alpha, void* scratch, len_t m, len_t n, StreamContext ctx), (x, gain, rstd, gy, eps, gx, ggain, alpha, scratch, m, n, ctx))
