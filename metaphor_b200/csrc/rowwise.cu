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
#include "mp_async.cuh"

#include <cfloat>
#include <mutex>

namespace {

template <int GROUP>
struct RowCfg {
  static constexpr int THREADS = GROUP < 128 ? 128 : GROUP;
  static constexpr int ROWS = THREADS / GROUP;  // rows in flight per CTA
};

__device__ __forceinline__ float mp_neg_inf(float) { return -INFINITY; }
__device__ __forceinline__ double mp_neg_inf(double) { return -INFINITY; }
// exp(x - mx) with the row maximum pre-scaled once per row: fp32 uses one FFMA
// and one ex2.approx (rel. error 2^-22, inputs <= 0, results below 2^-126 flush
// to zero); fp64 uses exp().
__device__ __forceinline__ float mp_exp_prescale(float mx) { return mx * 1.4426950408889634f; }
__device__ __forceinline__ double mp_exp_prescale(double mx) { return mx; }
__device__ __forceinline__ float mp_exp_diff(float x, float mx_scaled) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmaf(x, 1.4426950408889634f, -mx_scaled)));
  return y;
}
__device__ __forceinline__ double mp_exp_diff(double x, double mx) { return exp(x - mx); }
// MUFU.RSQ, relative error about 2^-22: far inside the 1e-4 budget of a row reduction
__device__ __forceinline__ float mp_rsqrt(float x) { return rsqrtf(x); }
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
    a = warp_reduce_width<SumOp, WARPS>(smem[lane & (WARPS - 1)]);
    b = warp_reduce_width<SumOp, WARPS>(smem[32 + (lane & (WARPS - 1))]);
    __syncthreads();
  }
}

// Thread t of a row group owns packs t, t+GROUP, ... (PPT of them).  FULL: the
// row has exactly GROUP*PPT packs, so no pack needs a bounds guard.
#define MP_PACK_VALID(u) (FULL || (t + static_cast<size_t>(u) * GROUP) < nv)
#define MP_PACK_INDEX(u) (t + static_cast<size_t>(u) * GROUP)

// ------------------------------- softmax ----------------------------------
template <typename T, int GROUP, int PPT, bool FULL>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) softmax_fwd_kernel(const T* x, T* y, size_t m, size_t n) {
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
    for (int u = 0; u < PPT; ++u)
      if (MP_PACK_VALID(u)) p[u] = ld_pack_stream(xr, MP_PACK_INDEX(u));
    A e[PPT][PN];
    A mx = mp_neg_inf(A(0));
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        unpack<T>(p[u], e[u]);
#pragma unroll
        for (int k = 0; k < PN; ++k) mx = MaxOp::apply(mx, e[u][k]);
      }
    }
    mx = group_reduce<MaxOp, GROUP>(mx, red, mp_neg_inf(A(0)));
    const A mxs = mp_exp_prescale(mx);
    A sum = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
#pragma unroll
        for (int k = 0; k < PN; ++k) {
          e[u][k] = mp_exp_diff(e[u][k], mxs);
          sum += e[u][k];
        }
      }
    }
    sum = group_reduce<SumOp, GROUP>(sum, red, A(0));
    const A inv = A(1) / sum;
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
#pragma unroll
        for (int k = 0; k < PN; ++k) e[u][k] *= inv;
        st_pack_stream(yr, MP_PACK_INDEX(u), pack<T>(e[u]));
      }
    }
  }
}

// gx = y o (gy - <gy, y>) + alpha*gx
template <typename T, int GROUP, int PPT, bool FULL, bool BLEND>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) softmax_rev_kernel(const T* y, const T* gy, T* gx,
                                                                            typename Acc<T>::type alpha, size_t m, size_t n) {
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
      if (MP_PACK_VALID(u)) {
        py[u] = ld_pack_stream(yr, MP_PACK_INDEX(u));
        pg[u] = ld_pack_stream(gr, MP_PACK_INDEX(u));
        if constexpr (BLEND) po[u] = ld_pack_stream(xr, MP_PACK_INDEX(u));
      }
    }
    A fy[PPT][PN], fg[PPT][PN];
    A dot = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        unpack<T>(py[u], fy[u]);
        unpack<T>(pg[u], fg[u]);
#pragma unroll
        for (int k = 0; k < PN; ++k) dot += fy[u][k] * fg[u][k];
      }
    }
    dot = group_reduce<SumOp, GROUP>(dot, red, A(0));
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        A fo[PN];
        if constexpr (BLEND) unpack<T>(po[u], fo);
#pragma unroll
        for (int k = 0; k < PN; ++k) {
          A r = fy[u][k] * (fg[u][k] - dot);
          if constexpr (BLEND) r += alpha * fo[k];
          fy[u][k] = r;
        }
        st_pack_stream(xr, MP_PACK_INDEX(u), pack<T>(fy[u]));
      }
    }
  }
}

// ------------------------------- RMSNorm ----------------------------------
template <typename T, int GROUP, int PPT, bool FULL>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) rmsnorm_fwd_kernel(const T* x, const T* __restrict__ gain,
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
  for (int u = 0; u < PPT; ++u)
    if (MP_PACK_VALID(u)) pgain[u] = ld_pack(gain, MP_PACK_INDEX(u));
  const A inv_n = A(1) / static_cast<A>(n);
  for (size_t row = static_cast<size_t>(blockIdx.x) * ROWS + g; row < m; row += static_cast<size_t>(gridDim.x) * ROWS) {
    const T* xr = x + row * n;
    T* yr = y + row * n;
    Pack<T> p[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u)
      if (MP_PACK_VALID(u)) p[u] = ld_pack_stream(xr, MP_PACK_INDEX(u));
    A f[PPT][PN];
    A ss = A(0);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        unpack<T>(p[u], f[u]);
#pragma unroll
        for (int k = 0; k < PN; ++k) ss += f[u][k] * f[u][k];
      }
    }
    ss = group_reduce<SumOp, GROUP>(ss, red, A(0));
    const A rstd = mp_rsqrt(ss * inv_n + eps);
    if (rstd_out != nullptr && t == 0) rstd_out[row] = rstd;
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        A fgain[PN];
        unpack<T>(pgain[u], fgain);
#pragma unroll
        for (int k = 0; k < PN; ++k) f[u][k] = f[u][k] * rstd * fgain[k];
        st_pack_stream(yr, MP_PACK_INDEX(u), pack<T>(f[u]));
      }
    }
  }
}

// One row of the RMSNorm reverse, shared by the register and the staged kernel:
// px/pg hold this thread's packs of x and gy, acc its gain-gradient partials.
//   gx = rstd*(gy o gain) - x*rstd^3*mean_j(gy o gain o x) + alpha*gx
template <typename T, int GROUP, int PPT, bool FULL, bool BLEND>
__device__ __forceinline__ void rmsnorm_rev_row(const Pack<T>* px, const Pack<T>* pg, const Pack<T>* pgain,
                                                typename Acc<T>::type (*acc)[Pack<T>::N], const typename Acc<T>::type* rstd_in,
                                                typename Acc<T>::type eps, typename Acc<T>::type inv_n,
                                                typename Acc<T>::type alpha, T* out_row, size_t row, int t, size_t nv,
                                                typename Acc<T>::type* red) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  if constexpr (std::is_same<T, __half>::value) {
    // r16: gx = rstd * (gy o gain) - coef * x (+ alpha * gx) is linear in the row's coef, which is
    // only known after the row sum.  The first pass leaves rstd * gy o gain as packed halves and the second is one or
    // two packed multiply-adds per pair of elements on the raw x packs: ten instructions per element instead of
    // nineteen, which is what kept the r16 kernel below the copy bandwidth.  (alpha must be exact in r16: 0, 1, ...)
    if (!BLEND || __half2float(__float2half_rn(alpha)) == alpha) {
      float rstd;
      float dot = 0.f, unused = 0.f;
      if (rstd_in != nullptr) {
        rstd = rstd_in[row];
      } else {   // one more reduction round for the row's own sum of squares
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < PPT; ++u) {
          if (MP_PACK_VALID(u)) {
            const __half2* hx = reinterpret_cast<const __half2*>(&px[u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 fx = __half22float2(hx[q]);
              ss += fx.x * fx.x + fx.y * fx.y;
            }
          }
        }
        group_sum2<GROUP>(ss, unused, red);
        rstd = mp_rsqrt(ss * inv_n + eps);
      }
      __half2 pa[PPT][4];
#pragma unroll
      for (int u = 0; u < PPT; ++u) {
        if (MP_PACK_VALID(u)) {
          const __half2* hx = reinterpret_cast<const __half2*>(&px[u]);
          const __half2* hg = reinterpret_cast<const __half2*>(&pg[u]);
          const __half2* hn = reinterpret_cast<const __half2*>(&pgain[u]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 fx = __half22float2(hx[q]), fg = __half22float2(hg[q]), fn = __half22float2(hn[q]);
            const float ux = fg.x * fn.x, uy = fg.y * fn.y;
            dot += ux * fx.x + uy * fx.y;
            acc[u][2 * q] += fg.x * fx.x * rstd;
            acc[u][2 * q + 1] += fg.y * fx.y * rstd;
            pa[u][q] = __floats2half2_rn(ux * rstd, uy * rstd);
          }
        }
      }
      group_sum2<GROUP>(unused, dot, red);
      const __half2 nc = __float2half2_rn(-rstd * rstd * rstd * dot * inv_n);
      const __half2 al2 = __float2half2_rn(alpha);
#pragma unroll
      for (int u = 0; u < PPT; ++u) {
        if (MP_PACK_VALID(u)) {
          const __half2* hx = reinterpret_cast<const __half2*>(&px[u]);
          Pack<T> po, out;
          if constexpr (BLEND) po = ld_pack_stream(out_row, MP_PACK_INDEX(u));
          __half2* ho = reinterpret_cast<__half2*>(&out);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            __half2 r = __hfma2(nc, hx[q], pa[u][q]);
            if constexpr (BLEND) r = __hfma2(al2, reinterpret_cast<const __half2*>(&po)[q], r);
            ho[q] = r;
          }
          st_pack_stream(out_row, MP_PACK_INDEX(u), out);
        }
      }
      return;
    }
  }
  A fx[PPT][PN], fu[PPT][PN], ft[PPT][PN];  // x, gy*gain, gy*x
  A ss = A(0), dot = A(0);
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    if (MP_PACK_VALID(u)) {
      A fg[PN], fgain[PN];
      unpack<T>(px[u], fx[u]);
      unpack<T>(pg[u], fg);
      unpack<T>(pgain[u], fgain);
#pragma unroll
      for (int k = 0; k < PN; ++k) {
        ss += fx[u][k] * fx[u][k];
        fu[u][k] = fg[k] * fgain[k];
        ft[u][k] = fg[k] * fx[u][k];
        dot += fu[u][k] * fx[u][k];
      }
    }
  }
  group_sum2<GROUP>(ss, dot, red);
  const A rstd = rstd_in != nullptr ? rstd_in[row] : mp_rsqrt(ss * inv_n + eps);
  const A coef = rstd * rstd * rstd * dot * inv_n;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    if (MP_PACK_VALID(u)) {
      A fo[PN];
      if constexpr (BLEND) {
        const Pack<T> po = ld_pack_stream(out_row, MP_PACK_INDEX(u));
        unpack<T>(po, fo);
      }
#pragma unroll
      for (int k = 0; k < PN; ++k) {
        A r = rstd * fu[u][k] - fx[u][k] * coef;
        if constexpr (BLEND) r += alpha * fo[k];
        acc[u][k] += ft[u][k] * rstd;
        fu[u][k] = r;
      }
      st_pack_stream(out_row, MP_PACK_INDEX(u), pack<T>(fu[u]));
    }
  }
}

// Register variant: a CTA owns rows_per_cta consecutive row groups and writes
// its gain-gradient partial to partial[blockIdx.x*ROWS + group][n].
template <typename T, int GROUP, int PPT, bool FULL, bool BLEND>
__global__ void __launch_bounds__(RowCfg<GROUP>::THREADS) rmsnorm_rev_kernel(
    const T* x, const T* __restrict__ gain, const typename Acc<T>::type* __restrict__ rstd_in, const T* gy,
    typename Acc<T>::type eps, T* gx, typename Acc<T>::type alpha, typename Acc<T>::type* __restrict__ partial, size_t m,
    size_t n, size_t rows_per_cta) {
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
    if (MP_PACK_VALID(u)) pgain[u] = ld_pack(gain, MP_PACK_INDEX(u));
#pragma unroll
    for (int k = 0; k < PN; ++k) acc[u][k] = A(0);
  }
  const A inv_n = A(1) / static_cast<A>(n);
  // The next row's packs are requested before the current row is reduced: a narrow row is a few hundred bytes per
  // thread group, and with one row in flight per group the kernel waits on memory latency, not bandwidth.
  Pack<T> px[PPT], pg[PPT], nx[PPT], ng[PPT];
  const size_t row0 = static_cast<size_t>(blockIdx.x) * rows_per_cta * ROWS + g;
  if (row0 < m) {
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        px[u] = ld_pack_stream(x + row0 * n, MP_PACK_INDEX(u));
        pg[u] = ld_pack_stream(gy + row0 * n, MP_PACK_INDEX(u));
      }
    }
  }
  for (size_t i = 0; i < rows_per_cta; ++i) {
    const size_t row = (static_cast<size_t>(blockIdx.x) * rows_per_cta + i) * ROWS + g;
    if (row >= m) break;
    const size_t next = row + ROWS;
    if (i + 1 < rows_per_cta && next < m) {
#pragma unroll
      for (int u = 0; u < PPT; ++u) {
        if (MP_PACK_VALID(u)) {
          nx[u] = ld_pack_stream(x + next * n, MP_PACK_INDEX(u));
          ng[u] = ld_pack_stream(gy + next * n, MP_PACK_INDEX(u));
        }
      }
    }
    rmsnorm_rev_row<T, GROUP, PPT, FULL, BLEND>(px, pg, pgain, acc, rstd_in, eps, inv_n, alpha, gx + row * n, row, t, nv, red);
#pragma unroll
    for (int u = 0; u < PPT; ++u) { px[u] = nx[u]; pg[u] = ng[u]; }
  }
  A* pr = partial + (static_cast<size_t>(blockIdx.x) * ROWS + g) * n;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    if (MP_PACK_VALID(u)) {
#pragma unroll
      for (int k = 0; k < PN; ++k) pr[MP_PACK_INDEX(u) * PN + k] = acc[u][k];
    }
  }
}

// Warp-per-row variant for narrow rows (n = 32 * NP packs, NP <= 8): a row lives in one warp's registers, the two
// row sums are warp shuffles (no CTA barrier per row), the next row's packs are requested before the current row is
// reduced, and the gain-gradient sums stay in registers over all rows of the warp.  The four warps of a CTA meet in
// shared memory once, so the call leaves gridDim.x partial rows (at most three per SM) instead of one per row group.
constexpr int WROW_THREADS = 128;

template <typename P>
__device__ __forceinline__ void pack_fence(P& v) {
  static_assert(sizeof(P) == 16, "16-byte packs");
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) asm volatile("" : "+r"(w[i]));
}

template <typename T, int NP, bool BLEND>
__global__ void __launch_bounds__(WROW_THREADS, 3) rmsnorm_rev_warp_kernel(
    const T* x, const T* __restrict__ gain, const typename Acc<T>::type* __restrict__ rstd_in, const T* gy,
    typename Acc<T>::type eps, T* gx, typename Acc<T>::type alpha, typename Acc<T>::type* __restrict__ partial, size_t m) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr size_t n = static_cast<size_t>(NP) * 32 * PN;
  __shared__ A cols[NP * 32 * PN];
  for (int i = threadIdx.x; i < NP * 32 * PN; i += WROW_THREADS) cols[i] = A(0);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Pack<T> pgain[NP];
  A acc[NP][PN];
#pragma unroll
  for (int u = 0; u < NP; ++u) {
    pgain[u] = ld_pack(gain, u * 32 + lane);
#pragma unroll
    for (int k = 0; k < PN; ++k) acc[u][k] = A(0);
  }
  const A inv_n = A(1) / static_cast<A>(n);
  const size_t stride = static_cast<size_t>(gridDim.x) * (WROW_THREADS / 32);
  size_t row = static_cast<size_t>(blockIdx.x) * (WROW_THREADS / 32) + warp;
  Pack<T> px[NP], pg[NP], nx[NP], ng[NP];
  if (row < m) {
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      px[u] = ld_pack_stream(x + row * n, u * 32 + lane);
      pg[u] = ld_pack_stream(gy + row * n, u * 32 + lane);
    }
  }
  for (; row < m; row += stride) {
    const size_t next = row + stride;
    if (next < m) {
#pragma unroll
      for (int u = 0; u < NP; ++u) {
        nx[u] = ld_pack_stream(x + next * n, u * 32 + lane);
        ng[u] = ld_pack_stream(gy + next * n, u * 32 + lane);
      }
    }
    Pack<T> po[BLEND ? NP : 1];
    if constexpr (BLEND) {
#pragma unroll
      for (int u = 0; u < NP; ++u) po[u] = ld_pack_stream(gx + row * n, u * 32 + lane);
    }
    A ss = A(0), dot = A(0);
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      A fx[PN], fg[PN], fgain[PN];
      unpack<T>(px[u], fx);
      unpack<T>(pg[u], fg);
      unpack<T>(pgain[u], fgain);
#pragma unroll
      for (int k = 0; k < PN; ++k) {
        ss += fx[k] * fx[k];
        dot += fg[k] * fgain[k] * fx[k];
      }
    }
    ss = warp_reduce<SumOp>(ss);
    dot = warp_reduce<SumOp>(dot);
    const A rstd = rstd_in != nullptr ? rstd_in[row] : mp_rsqrt(ss * inv_n + eps);
    const A coef = rstd * rstd * rstd * dot * inv_n;
    // the packs are decoded again below: without the fence the compiler keeps the first pass's converted values
    // alive (r16: four registers per pack become eight) and spills
#pragma unroll
    for (int u = 0; u < NP; ++u) { pack_fence(px[u]); pack_fence(pg[u]); pack_fence(pgain[u]); }
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      A fx[PN], fg[PN], fgain[PN], fo[PN], r[PN];
      unpack<T>(px[u], fx);
      unpack<T>(pg[u], fg);
      unpack<T>(pgain[u], fgain);
      if constexpr (BLEND) unpack<T>(po[u], fo);
#pragma unroll
      for (int k = 0; k < PN; ++k) {
        r[k] = rstd * fg[k] * fgain[k] - fx[k] * coef;
        if constexpr (BLEND) r[k] += alpha * fo[k];
        acc[u][k] += fg[k] * fx[k] * rstd;
      }
      st_pack_stream(gx + row * n, u * 32 + lane, pack<T>(r));
    }
#pragma unroll
    for (int u = 0; u < NP; ++u) { px[u] = nx[u]; pg[u] = ng[u]; }
  }
#pragma unroll
  for (int u = 0; u < NP; ++u) {
#pragma unroll
    for (int k = 0; k < PN; ++k) atomicAdd(cols + (u * 32 + lane) * PN + k, acc[u][k]);
  }
  __syncthreads();
  A* pr = partial + static_cast<size_t>(blockIdx.x) * n;
  for (int i = threadIdx.x; i < NP * 32 * PN; i += WROW_THREADS) pr[i] = cols[i];
}

// r16 rows with rstd supplied: gx = rstd * gxh - coef * x (+ alpha * gx) is linear in the row's coef, which is only
// known after the row sum, so the first pass leaves gxh = gy o gain as packed halves beside the raw x packs and the
// second pass is two or three packed multiply-adds per pair of elements; no value is decoded twice and nothing is
// prefetched into a second register set (at most 128 registers: sixteen warps per SM, and one partial row of gain
// gradients per 256-thread CTA, two per SM, so one small fold finishes the call).
constexpr int WROWH_THREADS = 256;

template <int NP, bool BLEND>
__global__ void __launch_bounds__(WROWH_THREADS, 2) rmsnorm_rev_warp_h_kernel(const __half* x, const __half* __restrict__ gain,
                                                                         const float* __restrict__ rstd_in, const __half* gy, __half* gx,
                                                                         float alpha, float* __restrict__ partial, size_t m) {
  constexpr size_t n = static_cast<size_t>(NP) * 256;
  __shared__ float cols[NP * 256];
  for (int i = threadIdx.x; i < NP * 256; i += WROWH_THREADS) cols[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float acc[NP][8];
#pragma unroll
  for (int u = 0; u < NP; ++u) {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
  }
  const float inv_n = 1.f / static_cast<float>(n);
  const __half2 al2 = __float2half2_rn(alpha);
  const size_t stride = static_cast<size_t>(gridDim.x) * (WROWH_THREADS / 32);
  for (size_t row = static_cast<size_t>(blockIdx.x) * (WROWH_THREADS / 32) + warp; row < m; row += stride) {
    uint4 px[NP], pg[NP], po[BLEND ? NP : 1];
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      px[u] = __ldcs(reinterpret_cast<const uint4*>(x + row * n) + u * 32 + lane);
      pg[u] = __ldcs(reinterpret_cast<const uint4*>(gy + row * n) + u * 32 + lane);
      if constexpr (BLEND) po[u] = __ldcs(reinterpret_cast<const uint4*>(gx + row * n) + u * 32 + lane);
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      const uint4 pn = __ldg(reinterpret_cast<const uint4*>(gain) + u * 32 + lane);
      const __half2* hx = reinterpret_cast<const __half2*>(&px[u]);
      __half2* hg = reinterpret_cast<__half2*>(&pg[u]);
      const __half2* hn = reinterpret_cast<const __half2*>(&pn);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fx = __half22float2(hx[q]), fg = __half22float2(hg[q]), fn = __half22float2(hn[q]);
        const float ux = fg.x * fn.x, uy = fg.y * fn.y;
        dot += ux * fx.x + uy * fx.y;
        acc[u][2 * q] += fg.x * fx.x * rstd;
        acc[u][2 * q + 1] += fg.y * fx.y * rstd;
        hg[q] = __floats2half2_rn(ux * rstd, uy * rstd);   // rstd * gxh replaces gy in place
      }
    }
    dot = warp_reduce<SumOp>(dot);
    const __half2 nc = __float2half2_rn(-rstd * rstd * rstd * dot * inv_n);
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      const __half2* hx = reinterpret_cast<const __half2*>(&px[u]);
      const __half2* hg = reinterpret_cast<const __half2*>(&pg[u]);
      uint4 o;
      __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __half2 r = __hfma2(nc, hx[q], hg[q]);
        if constexpr (BLEND) r = __hfma2(al2, reinterpret_cast<const __half2*>(&po[u])[q], r);
        ho[q] = r;
      }
      __stcs(reinterpret_cast<uint4*>(gx + row * n) + u * 32 + lane, o);
    }
  }
#pragma unroll
  for (int u = 0; u < NP; ++u) {
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(cols + (u * 32 + lane) * 8 + k, acc[u][k]);
  }
  __syncthreads();
  float* pr = partial + static_cast<size_t>(blockIdx.x) * n;
  for (int i = threadIdx.x; i < NP * 256; i += WROWH_THREADS) pr[i] = cols[i];
}

// Shared-memory staged variant of the RMSNorm reverse kernel: the rows of x and
// gy that a CTA will need are fetched ahead of time by 1-D bulk async copies
// (TMA unit) into a ring of `stages` buffers, each guarded by an mbarrier, so
// the bytes in flight are bounded by shared memory instead of by registers.
// All 256 threads wait for a stage, copy their slice into registers, and meet
// in the reduction barrier; after that barrier nobody reads the stage any more
// and thread 0 refills it with the row `stages` ahead.  Waits are bounded
// (mp_async.cuh); a timeout sets the status word and ends the CTA's loop.
constexpr int STG_THREADS = 256;

// CTAs per SM the staged kernel is compiled for: up to 2 packs per thread and
// stream fit 3 CTAs (<= 85 registers), wider rows 2.
template <typename T, int PPT> struct StgOcc { static constexpr int value = (PPT <= 2 && sizeof(T) < 8) ? 3 : 2; };

template <typename T, int PPT, bool FULL, bool BLEND>
__global__ void __launch_bounds__(STG_THREADS, StgOcc<T, PPT>::value) rmsnorm_rev_staged_kernel(
    const T* x, const T* __restrict__ gain, const typename Acc<T>::type* __restrict__ rstd_in, const T* gy,
    typename Acc<T>::type eps, T* gx, typename Acc<T>::type alpha, typename Acc<T>::type* __restrict__ partial,
    size_t m, size_t n, size_t rows_per_cta, int stages, uint32_t* status) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int GROUP = STG_THREADS;
  extern __shared__ __align__(128) unsigned char stg_smem[];
  __shared__ A red[64];
  uint64_t* full = reinterpret_cast<uint64_t*>(stg_smem);  // one barrier per stage (<= 16)
  unsigned char* data = stg_smem + 128;
  const int t = threadIdx.x;
  const size_t nv = n / PN;
  const uint32_t row_bytes = static_cast<uint32_t>(n * sizeof(T));
  const size_t stage_bytes = 2 * static_cast<size_t>(row_bytes);
  const size_t r0 = static_cast<size_t>(blockIdx.x) * rows_per_cta;
  const size_t count = (m - r0) < rows_per_cta ? (m - r0) : rows_per_cta;

  if (t == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(full + s, 1);
    mbar_fence_init();
  }
  __syncthreads();
  auto issue = [&](size_t i, int s) {  // row r0 + i into stage s (= i mod stages)
    unsigned char* dst = data + s * stage_bytes;
    mbar_arrive_expect_tx(full + s, 2 * row_bytes);
    bulk_load_1d(dst, x + (r0 + i) * n, row_bytes, full + s);
    bulk_load_1d(dst + row_bytes, gy + (r0 + i) * n, row_bytes, full + s);
  };
  if (t == 0) {
    for (size_t i = 0; i < count && i < static_cast<size_t>(stages); ++i) issue(i, static_cast<int>(i));
  }

  Pack<T> pgain[PPT];
  A acc[PPT][PN];
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    if (MP_PACK_VALID(u)) pgain[u] = ld_pack(gain, MP_PACK_INDEX(u));
#pragma unroll
    for (int k = 0; k < PN; ++k) acc[u][k] = A(0);
  }
  const A inv_n = A(1) / static_cast<A>(n);
  int s = 0;            // stage of row i
  uint32_t parity = 0;  // phase of that stage's barrier
  for (size_t i = 0; i < count; ++i) {
    if (!mbar_wait(full + s, parity, status)) break;  // every thread waits on the same phase
    const size_t row = r0 + i;
    const unsigned char* sx = data + s * stage_bytes;
    const unsigned char* sg = sx + row_bytes;
    Pack<T> px[PPT], pg[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
      if (MP_PACK_VALID(u)) {
        px[u] = *reinterpret_cast<const Pack<T>*>(sx + MP_PACK_INDEX(u) * 16);
        pg[u] = *reinterpret_cast<const Pack<T>*>(sg + MP_PACK_INDEX(u) * 16);
      }
    }
    // The first barrier inside the row function's reduction also tells thread 0
    // that every thread has copied stage s to registers; the refill is issued
    // right after the row is finished.
    rmsnorm_rev_row<T, GROUP, PPT, FULL, BLEND>(px, pg, pgain, acc, rstd_in, eps, inv_n, alpha, gx + row * n, row, t, nv, red);
    if (t == 0 && i + stages < count) issue(i + stages, s);
    if (++s == stages) { s = 0; parity ^= 1u; }
  }
  A* pr = partial + static_cast<size_t>(blockIdx.x) * n;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    if (MP_PACK_VALID(u)) {
#pragma unroll
      for (int k = 0; k < PN; ++k) pr[MP_PACK_INDEX(u) * PN + k] = acc[u][k];
    }
  }
}

// ggain[j] = sum_p partial[p][j] + alpha*ggain[j].  CTA = 32 columns x blockDim.x / 32 slices (8 or 32: a few hundred
// partial rows are a chain of ~40 dependent additions per thread with 8 slices, ~10 with 32).
template <typename T>
__global__ void __launch_bounds__(1024) rmsnorm_fold_kernel(const typename Acc<T>::type* __restrict__ partial, T* ggain,
                                                            typename Acc<T>::type alpha, bool blend, size_t n, size_t slots) {
  using A = typename Acc<T>::type;
  __shared__ A sm[32][33];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5, slices = blockDim.x >> 5;
  const size_t col = static_cast<size_t>(blockIdx.x) * 32 + lane;
  A s = A(0);
  if (col < n) {
    for (size_t p = slice; p < slots; p += slices) s += partial[p * n + col];
  }
  sm[slice][lane] = s;
  __syncthreads();
  if (slice == 0 && col < n) {
    A r = A(0);
    for (int w = 0; w < slices; ++w) r += sm[w][lane];
    ggain[col] = mp_down<T>(blend ? r + alpha * mp_up(ggain[col]) : r);
  }
}
inline unsigned rmsnorm_fold_threads(size_t slots) { return slots > 64 ? 1024u : 256u; }

// First stage of a two-stage fold for many partial rows: CTA (column block c,
// split f) sums the partial rows f, f+F, f+2F, ... of 32*W columns (W = values
// per 16-byte load) into partial2[f][:].  Eight warps stride the rows with four
// independent 16-byte loads in flight each; the warps meet in shared memory.
// The second stage is rmsnorm_fold_kernel over the F rows of partial2.
constexpr int FOLD_SPLITS = 16;

template <typename A>
__global__ void __launch_bounds__(256) rmsnorm_fold_stage1_kernel(const A* __restrict__ partial, A* __restrict__ partial2,
                                                                  size_t n, size_t slots) {
  constexpr int W = 16 / sizeof(A);
  __shared__ A sm[8][32 * W + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t c = (static_cast<size_t>(blockIdx.x) * 32 + lane) * W;
  const size_t F = gridDim.y, f = blockIdx.y;
  A acc[W];
#pragma unroll
  for (int e = 0; e < W; ++e) acc[e] = A(0);
  if (c < n) {
    // rows f + F*(warp + 8*j)
    size_t r = f + F * warp;
    const size_t step = F * 8;
    for (; r + 3 * step < slots; r += 4 * step) {
      Pack<A> q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = ld_pack(partial, ((r + u * step) * n + c) / W);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] += q[u].v[e];
    }
    for (; r < slots; r += step) {
      const Pack<A> q = ld_pack(partial, (r * n + c) / W);
#pragma unroll
      for (int e = 0; e < W; ++e) acc[e] += q.v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < W; ++e) sm[warp][lane * W + e] = acc[e];
  __syncthreads();
  for (int j = threadIdx.x; j < 32 * W; j += 256) {
    const size_t col = static_cast<size_t>(blockIdx.x) * 32 * W + j;
    if (col < n) {
      A t = A(0);
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sm[w][j];
      partial2[f * n + col] = t;
    }
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
    const A mxs = mp_exp_prescale(mx);
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) sum += mp_exp_diff(mp_up(xr[j]), mxs);
    sum = cta_reduce<SumOp, GEN_THREADS>(sum, red, A(0));
    const A inv = A(1) / sum;
    for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) yr[j] = mp_down<T>(mp_exp_diff(mp_up(xr[j]), mxs) * inv);
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
                                                                   typename Acc<T>::type* partial, size_t m, size_t n,
                                                                   size_t rows_per_cta) {
  using A = typename Acc<T>::type;
  __shared__ A red[64];
  const A inv_n = A(1) / static_cast<A>(n);
  A* pr = partial + static_cast<size_t>(blockIdx.x) * n;
  for (size_t j = threadIdx.x; j < n; j += GEN_THREADS) pr[j] = A(0);
  for (size_t i = 0; i < rows_per_cta; ++i) {
    const size_t row = static_cast<size_t>(blockIdx.x) * rows_per_cta + i;
    if (row >= m) break;
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
  bool full;
};

// Up to 4 packs per thread.  Measured on B200 at n = 4096: for r16 rows, 128
// threads x 4 packs beat 256 threads x 2 packs (fewer barrier participants,
// more independent loads per thread).
template <typename T>
RowPlan plan_rows(size_t n, bool aligned) {
  constexpr int PN = Pack<T>::N;
  constexpr int P = 4;
  RowPlan p{true, GEN_THREADS, 0, GEN_THREADS, 1, false};
  if (!aligned || n % PN != 0 || n == 0) return p;
  const size_t nv = n / PN;
  int group;
  if (nv <= 32 * P) group = 32;
  else if (nv <= 128 * P) group = 128;
  else if (nv <= 256 * P) group = 256;
  else if (nv <= 512 * P) group = 512;
  else if (nv <= 1024 * P) group = 1024;
  else return p;
  const size_t need = (nv + group - 1) / group;
  p.generic = false;
  p.group = group;
  p.ppt = need <= 1 ? 1 : (need <= 2 ? 2 : 4);
  p.threads = group < 128 ? 128 : group;
  p.rows = p.threads / group;
  p.full = nv == static_cast<size_t>(p.group) * p.ppt;
  return p;
}

// Plan of the RMSNorm reverse (register variant).  One warp per row with four packs per lane keeps 32 r16 values
// of x, gy, their products and the gain-gradient sums per lane: 226 registers, two CTAs per SM.  Rows of 65..128
// r16 packs therefore take 128 threads with one pack each (about 50 registers; a quarter of the partial rows).
// (The forward keeps one warp per row at that width: 14.5 against 17.0 us on [16384, 768].)
template <typename T>
RowPlan plan_rows_rev(size_t n, bool aligned) {
  RowPlan p = plan_rows<T>(n, aligned);
  if (!p.generic && sizeof(T) == 2 && p.group == 32 && p.ppt == 4 && getenv("MP_RMS_REV_WARP_ROWS") == nullptr) {
    p.group = 128;
    p.ppt = 1;
    p.threads = 128;
    p.rows = 1;
    p.full = n / Pack<T>::N == 128;
  }
  return p;
}

// Streaming row kernels launch one CTA per row group (measured faster on B200
// than persistent CTAs looping in lock-step).  `threads_per_sm` != 0 asks for a
// persistent grid instead (kernels that carry per-CTA state across rows).
inline size_t row_grid(const RowPlan& p, size_t m, int sm_count, int threads_per_sm) {
  size_t grid = (m + p.rows - 1) / p.rows;
  if (threads_per_sm != 0) {
    size_t per_sm = static_cast<size_t>(threads_per_sm / p.threads);
    if (per_sm < 1) per_sm = 1;
    const size_t cap = static_cast<size_t>(sm_count) * per_sm;
    if (grid > cap) grid = cap;
  }
  if (grid > (1u << 30)) grid = 1u << 30;
  if (grid < 1) grid = 1;
  return grid;
}

// (group, packs per thread) pairs plan_rows can produce.
#define MP_ROW_DISPATCH_G(PLAN, CALL, F, G)                                   \
  do {                                                                        \
    if ((PLAN).ppt == 1) { CALL(G, 1, F); }                                   \
    else if ((PLAN).ppt == 2) { CALL(G, 2, F); }                              \
    else { CALL(G, 4, F); }                                                   \
  } while (0)
#define MP_ROW_DISPATCH_F(PLAN, CALL, F)                                      \
  do {                                                                        \
    if ((PLAN).group == 32) MP_ROW_DISPATCH_G(PLAN, CALL, F, 32);             \
    else if ((PLAN).group == 128) MP_ROW_DISPATCH_G(PLAN, CALL, F, 128);      \
    else if ((PLAN).group == 256) MP_ROW_DISPATCH_G(PLAN, CALL, F, 256);      \
    else if ((PLAN).group == 512) MP_ROW_DISPATCH_G(PLAN, CALL, F, 512);      \
    else MP_ROW_DISPATCH_G(PLAN, CALL, F, 1024);                              \
  } while (0)
// `full`: the row has exactly group*ppt packs, the kernel drops its bounds guards
#define MP_ROW_DISPATCH(PLAN, CALL)                                           \
  do {                                                                        \
    if ((PLAN).full) MP_ROW_DISPATCH_F(PLAN, CALL, true);                     \
    else MP_ROW_DISPATCH_F(PLAN, CALL, false);                                \
  } while (0)

// Row groups each CTA of the RMSNorm reverse kernel walks (its gain-gradient
// partial costs one scratch row, so more rows per CTA = less scratch traffic,
// fewer rows = more CTAs in flight).
// `units` = row groups (register variant) or rows (staged variant) of the call: short matrices take
// fewer rows per CTA so that at least ~8 CTAs per SM exist.
inline size_t rms_rev_rows_per_cta(size_t units, int sm_count) {
  static const size_t cap = []() {      // initialised once, thread-safely (launchers may be called from any host thread)
    const char* e = getenv("MP_RMS_REV_ROWS");
    const long v = e ? strtol(e, nullptr, 10) : 0;
    return v > 0 ? static_cast<size_t>(v) : static_cast<size_t>(32);
  }();
  size_t r = units / (static_cast<size_t>(sm_count > 0 ? sm_count : 148) * 8);
  if (r < 1) r = 1;
  return r > cap ? cap : r;
}
// Staged (bulk-copy) plan of the RMSNorm reverse: rows of n*sizeof(T) bytes,
// 256 threads, up to 4 packs per thread, at least 2 stages in ~100 KB.
struct StagedPlan { bool ok; int ppt, stages; size_t smem_bytes; bool full; };
template <typename T>
StagedPlan plan_staged(size_t n, bool aligned) {
  constexpr int PN = Pack<T>::N;
  StagedPlan p{false, 0, 0, 0, false};
  if (!aligned || n % PN != 0 || getenv("MP_RMS_REV_NO_STAGING") != nullptr) return p;
  const size_t nv = n / PN;
  if (nv < 128 || nv > static_cast<size_t>(STG_THREADS) * 4) return p;
  const size_t stage_bytes = 2 * n * sizeof(T);
  const size_t need = (nv + STG_THREADS - 1) / STG_THREADS;
  const int ppt = need <= 1 ? 1 : (need <= 2 ? 2 : 4);
  // ring size: ~68 KB when three CTAs share an SM, ~100 KB when two do
  const int occ = ppt == 1 ? StgOcc<T, 1>::value : (ppt == 2 ? StgOcc<T, 2>::value : StgOcc<T, 4>::value);
  size_t budget_kb = occ >= 3 ? 68 : 100;
  if (const char* e = getenv("MP_RMS_STAGE_KB")) {
    const long v = strtol(e, nullptr, 10);
    if (v > 0) budget_kb = static_cast<size_t>(v);
  }
  size_t stages = (budget_kb * 1024) / stage_bytes;
  if (stages > 8) stages = 8;
  if (stages < 2) return p;
  p.ok = true;
  p.ppt = ppt;
  p.stages = static_cast<int>(stages);
  p.smem_bytes = 128 + stages * stage_bytes;
  p.full = nv == static_cast<size_t>(STG_THREADS) * p.ppt;
  return p;
}
// Warp-per-row plan of the RMSNorm reverse: packs per lane (0: the row does not fit it)
template <typename T>
int rms_rev_warp_packs(size_t n, bool aligned) {
  constexpr size_t PN = Pack<T>::N;
  if (!aligned || n % (32 * PN) != 0 || getenv("MP_RMS_REV_NO_WARP") != nullptr) return 0;
  const size_t np = n / (32 * PN);
  return np <= (sizeof(T) == 4 ? 5 : 4) ? static_cast<int>(np) : 0;   // wider rows spill the register plan
}
inline size_t rms_rev_warp_grid(size_t m, int sm_count, int per_sm = 3) {
  const size_t want = (m + WROW_THREADS / 32 - 1) / (WROW_THREADS / 32), cap = per_sm * static_cast<size_t>(sm_count > 0 ? sm_count : 148);
  return want < 1 ? 1 : (want < cap ? want : cap);
}
inline size_t rms_rev_grid(const RowPlan& p, size_t m, int sm_count) {
  const size_t groups = (m + p.rows - 1) / p.rows;
  const size_t rpc = rms_rev_rows_per_cta(groups, sm_count);
  size_t grid = (groups + rpc - 1) / rpc;
  return grid < 1 ? 1 : grid;
}

}  // namespace

template <typename T>
static void softmax_ij_j_impl(const void* src_, void* dst_, len_t m, len_t n, StreamContext ctx) {
  if (m == 0 || n == 0) return;
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  const RowPlan p = plan_rows<T>(n, mp_aligned16(src) && mp_aligned16(dst));
  cudaStream_t st = mp_stream(ctx);
  const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), 0));
  if (p.generic) {
    softmax_fwd_generic<T><<<grid, GEN_THREADS, 0, st>>>(src, dst, m, n);
  } else {
#define CALL(G, P, F) softmax_fwd_kernel<T, G, P, F><<<grid, RowCfg<G>::THREADS, 0, st>>>(src, dst, m, n)
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
  const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), 0));
  if (p.generic) {
    softmax_rev_generic<T><<<grid, GEN_THREADS, 0, st>>>(y, gy, gx, a, blend, m, n);
  } else if (blend) {
#define CALL(G, P, F) softmax_rev_kernel<T, G, P, F, true><<<grid, RowCfg<G>::THREADS, 0, st>>>(y, gy, gx, a, m, n)
    MP_ROW_DISPATCH(p, CALL);
#undef CALL
  } else {
#define CALL(G, P, F) softmax_rev_kernel<T, G, P, F, false><<<grid, RowCfg<G>::THREADS, 0, st>>>(y, gy, gx, a, m, n)
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
  const unsigned grid = static_cast<unsigned>(row_grid(p, m, mp_sm_count(ctx), 0));
  if (p.generic) {
    rmsnorm_fwd_generic<T><<<grid, GEN_THREADS, 0, st>>>(x, gain, e, y, rstd, m, n);
  } else {
#define CALL(G, P, F) rmsnorm_fwd_kernel<T, G, P, F><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, e, y, rstd, m, n)
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
  const RowPlan p = plan_rows_rev<T>(n, aligned);
  size_t slots = rms_rev_grid(p, m, sm_count) * p.rows;
  const size_t staged = (m + rms_rev_rows_per_cta(m, sm_count) - 1) / rms_rev_rows_per_cta(m, sm_count);  // one slot per CTA
  if (staged > slots) slots = staged;
  const size_t warp_rows = rms_rev_warp_grid(m, sm_count, 3);
  return slots > warp_rows ? slots : warp_rows;
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
    const RowPlan p = plan_rows_rev<T>(n, aligned);
    const StagedPlan sp = plan_staged<T>(n, aligned);
    const int sms = mp_sm_count(ctx);
    unsigned grid = static_cast<unsigned>(rms_rev_grid(p, m, sms));
    size_t rpc = rms_rev_rows_per_cta((m + p.rows - 1) / p.rows, sms);
    slots = static_cast<size_t>(grid) * p.rows;
    MpStreamState* state = mp_state_or_null(ctx);  // the staged kernel reports timeouts through the status word
    const int wnp = rms_rev_warp_packs<T>(n, aligned);
    bool half_plan = false;
    if constexpr (std::is_same<T, __half>::value) {
      // alpha must be exactly representable so that the packed blend equals the fp32 one (0, 1 and small powers of two are)
      half_plan = aligned && rstd != nullptr && n % 256 == 0 && n / 256 <= 4 && getenv("MP_RMS_REV_NO_WARP") == nullptr &&
                  static_cast<float>(__half2float(__float2half_rn(a))) == a;
      if (half_plan) {
        const size_t want = (m + WROWH_THREADS / 32 - 1) / (WROWH_THREADS / 32), cap = 2 * static_cast<size_t>(sms);
        grid = static_cast<unsigned>(want < cap ? want : cap);
        slots = grid;
#define WROWH(NPV)                                                                                                     \
  do {                                                                                                                 \
    if (blend) rmsnorm_rev_warp_h_kernel<NPV, true><<<grid, WROWH_THREADS, 0, st>>>(x, gain, rstd, gy, gx, a, partial, m);   \
    else rmsnorm_rev_warp_h_kernel<NPV, false><<<grid, WROWH_THREADS, 0, st>>>(x, gain, rstd, gy, gx, a, partial, m);        \
  } while (0)
        switch (n / 256) {
          case 1: WROWH(1); break;
          case 2: WROWH(2); break;
          case 3: WROWH(3); break;
          default: WROWH(4); break;
        }
#undef WROWH
      }
    }
    if (half_plan) {
    } else if (wnp > 0) {
      grid = static_cast<unsigned>(rms_rev_warp_grid(m, sms));
      slots = grid;
#define WROW(NPV)                                                                                                          \
  do {                                                                                                                     \
    if (blend) rmsnorm_rev_warp_kernel<T, NPV, true><<<grid, WROW_THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m);   \
    else rmsnorm_rev_warp_kernel<T, NPV, false><<<grid, WROW_THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m);        \
  } while (0)
      switch (wnp) {
        case 1: WROW(1); break;
        case 2: WROW(2); break;
        case 3: WROW(3); break;
        case 4: WROW(4); break;
        default: WROW(5); break;
      }
#undef WROW
    } else if (sp.ok && state != nullptr) {
      rpc = rms_rev_rows_per_cta(m, sms);
      // (one resident wave of CTAs with ~150 rows each was measured slower than waves of 32-row CTAs: 312 vs 277 us at
      // [65536, 4096] r16, 521 vs 498 us r32)
      grid = static_cast<unsigned>((m + rpc - 1) / rpc);
      slots = grid;
      uint32_t* status = state->status_dev;
#define STG(P, F, B)                                                                                       \
  do {                                                                                                     \
    MP_CUDA_CHECK(cudaFuncSetAttribute(rmsnorm_rev_staged_kernel<T, P, F, B>,                              \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));          \
    rmsnorm_rev_staged_kernel<T, P, F, B><<<grid, STG_THREADS, sp.smem_bytes, st>>>(                       \
        x, gain, rstd, gy, e, gx, a, partial, m, n, rpc, sp.stages, status);                               \
  } while (0)
#define STG_P(F, B)                                                                 \
  do { if (sp.ppt == 1) STG(1, F, B); else if (sp.ppt == 2) STG(2, F, B); else STG(4, F, B); } while (0)
      if (blend) { if (sp.full) STG_P(true, true); else STG_P(false, true); }
      else { if (sp.full) STG_P(true, false); else STG_P(false, false); }
#undef STG_P
#undef STG
    } else if (p.generic) {
      rmsnorm_rev_generic<T><<<grid, GEN_THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, blend, partial, m, n, rpc);
    } else if (blend) {
#define CALL(G, P, F) rmsnorm_rev_kernel<T, G, P, F, true><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m, n, rpc)
      MP_ROW_DISPATCH(p, CALL);
#undef CALL
    } else {
#define CALL(G, P, F) rmsnorm_rev_kernel<T, G, P, F, false><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m, n, rpc)
      MP_ROW_DISPATCH(p, CALL);
#undef CALL
    }
    MP_LAUNCH_CHECK();
  }
  constexpr int W = 16 / sizeof(A);
  if (slots >= 512 && n % W == 0 && mp_aligned16(partial)) {   // (a few hundred rows: one launch is cheaper than two)
    A* partial2 = partial + slots * n;  // FOLD_SPLITS rows after the per-CTA partials
    const dim3 g1(static_cast<unsigned>((n + 32 * W - 1) / (32 * W)), FOLD_SPLITS);
    rmsnorm_fold_stage1_kernel<A><<<g1, 256, 0, st>>>(partial, partial2, n, slots);
    MP_LAUNCH_CHECK();
    rmsnorm_fold_kernel<T><<<static_cast<unsigned>((n + 31) / 32), rmsnorm_fold_threads(FOLD_SPLITS), 0, st>>>(partial2, ggain, a, blend, n, FOLD_SPLITS);
  } else {
    rmsnorm_fold_kernel<T><<<static_cast<unsigned>((n + 31) / 32), rmsnorm_fold_threads(slots), 0, st>>>(partial, ggain, a, blend, n, slots);
  }
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
  return static_cast<len_t>((slots + FOLD_SPLITS) * n * sizeof(double));
}

MP_STAMP3(softmax_ij_j, (const void* src, void* dst, len_t m, len_t n, StreamContext ctx), (src, dst, m, n, ctx))
MP_STAMP3(softmax_ij_j_reverse, (const void* y, const void* gy, void* gx, double alpha, len_t m, len_t n, StreamContext ctx), (y, gy, gx, alpha, m, n, ctx))
MP_STAMP3(rmsnorm_ij_j, (const void* x, const void* gain, double eps, void* y, void* rstd, len_t m, len_t n, StreamContext ctx), (x, gain, eps, y, rstd, m, n, ctx))
MP_STAMP3(rmsnorm_ij_j_reverse, (const void* x, const void* gain, const void* rstd, const void* gy, double eps, void* gx, void* ggain, double alpha, void* scratch, len_t m, len_t n, StreamContext ctx), (x, gain, rstd, gy, eps, gx, ggain, alpha, scratch, m, n, ctx))

// ---------------------------------------------------------------------------
// RMSNorm reverse (r32) for callers that may not allocate device memory.
//
// Who needs it: a plug-in running inside a host runtime that has handed the
// whole device to its own memory pool and forbids cudaMalloc, or a
// latency-critical loop in which an allocation would synchronise the device.
// Such a caller cannot provide the gain-gradient scratch that
// launch_rmsnorm_ij_j_reverse_r32 asks for, so this variant keeps the scratch in
// a fixed array that is part of the library image: every GPU that loads the
// library holds MP_RMSNORM_STATIC_SCRATCH_BYTES (8 MiB) of it until the process
// exits.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
//
// The array's name is only a host-side stand-in for the device object, not a
// device address; the address is fetched once per device with
// cudaGetSymbolAddress (with that device current) and passed to the kernels.
// The first call on a device performs that look-up, so it should be made
// before the stream is put into capture mode.
//
// All calls share the one array and it keeps whatever the previous call left
// there.  Nothing in it has to start at zero: every partial row a launch reads
// is written earlier in the same launch sequence.  Two calls that overlap on
// the GPU (different streams) would race on it - keep calls stream-ordered.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_rmsnorm_static_scratch[MP_RMSNORM_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[64] = {nullptr};

// Device address of the static scratch on the current device (looked up once).
void* static_scratch_address() {
  int device = 0;
  MP_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64) MP_FATAL("device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    MP_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_rmsnorm_static_scratch));
    g_static_scratch_ptr[device] = ptr;
  }
  return g_static_scratch_ptr[device];
}
}  // namespace

// Same arguments and results as launch_rmsnorm_ij_j_reverse_r32 minus the
// scratch pointer.  Returns 0, or MP_STATUS_BAD_ARGUMENT (after printing why)
// when the row length does not fit the fixed scratch: it must hold at least one
// partial row per concurrently reduced row plus the 16 rows of the second fold
// stage, i.e. n <= MP_RMSNORM_STATIC_SCRATCH_BYTES / (4 * 20) = 104857 columns
// is always accepted.  Any number of rows is accepted (more rows per CTA are
// used when the scratch would otherwise overflow).
extern "C" int launch_rmsnorm_ij_j_reverse_static_r32(const void* x_, const void* gain_, const void* rstd_, const void* gy_,
                                                      double eps, void* gx_, void* ggain_, double alpha, len_t m, len_t n,
                                                      StreamContext ctx) {
  using T = float;
  using A = float;
  if (n == 0) return 0;
  if (MpStreamState* state = mp_state_or_null(ctx)) {
    // the scratch array is per device: the stream must belong to the device that is current in this thread
    int current = -1;
    MP_CUDA_CHECK(cudaGetDevice(&current));
    if (state->device != current) {
      fprintf(stderr, "launch_rmsnorm_ij_j_reverse_static_r32: the stream belongs to device %d, device %d is current\n", state->device, current);
      return static_cast<int>(MP_STATUS_BAD_ARGUMENT);
    }
  }
  const size_t cap_rows = MP_RMSNORM_STATIC_SCRATCH_BYTES / (n * sizeof(A));
  const T* x = static_cast<const T*>(x_);
  const T* gain = static_cast<const T*>(gain_);
  const A* rstd = static_cast<const A*>(rstd_);
  const T* gy = static_cast<const T*>(gy_);
  T* gx = static_cast<T*>(gx_);
  T* ggain = static_cast<T*>(ggain_);
  const bool aligned = mp_aligned16(x) && mp_aligned16(gain) && mp_aligned16(gy) && mp_aligned16(gx);
  const RowPlan p = plan_rows<T>(n, aligned);
  if (cap_rows < static_cast<size_t>(FOLD_SPLITS) + p.rows) {
    fprintf(stderr,
            "launch_rmsnorm_ij_j_reverse_static_r32: n = %lu columns does not fit the %u-byte static scratch "
            "(needs %lu bytes); use launch_rmsnorm_ij_j_reverse_r32 with caller scratch\n",
            static_cast<unsigned long>(n), static_cast<unsigned>(MP_RMSNORM_STATIC_SCRATCH_BYTES),
            static_cast<unsigned long>((FOLD_SPLITS + p.rows) * n * sizeof(A)));
    return static_cast<int>(MP_STATUS_BAD_ARGUMENT);
  }
  A* partial = static_cast<A*>(static_scratch_address());
  cudaStream_t st = mp_stream(ctx);
  const A a = static_cast<A>(alpha);
  const A e = static_cast<A>(eps);
  const bool blend = alpha != 0.0;
  size_t slots = 0;
  if (m > 0) {
    // CTAs (each owning p.rows partial rows) that fit beside the second-stage rows
    const size_t max_grid = (cap_rows - FOLD_SPLITS) / p.rows;
    const size_t groups = (m + p.rows - 1) / p.rows;
    size_t rpc = 32;
    if ((groups + rpc - 1) / rpc > max_grid) rpc = (groups + max_grid - 1) / max_grid;
    const unsigned grid = static_cast<unsigned>((groups + rpc - 1) / rpc);
    slots = static_cast<size_t>(grid) * p.rows;
    if (p.generic) {
      rmsnorm_rev_generic<T><<<grid, GEN_THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, blend, partial, m, n, rpc);
    } else if (blend) {
#define CALL(G, P, F) rmsnorm_rev_kernel<T, G, P, F, true><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m, n, rpc)
      MP_ROW_DISPATCH(p, CALL);
#undef CALL
    } else {
#define CALL(G, P, F) rmsnorm_rev_kernel<T, G, P, F, false><<<grid, RowCfg<G>::THREADS, 0, st>>>(x, gain, rstd, gy, e, gx, a, partial, m, n, rpc)
      MP_ROW_DISPATCH(p, CALL);
#undef CALL
    }
    MP_LAUNCH_CHECK();
  }
  constexpr int W = 16 / sizeof(A);
  if (slots >= 128 && n % W == 0) {
    A* partial2 = partial + slots * n;
    const dim3 g1(static_cast<unsigned>((n + 32 * W - 1) / (32 * W)), FOLD_SPLITS);
    rmsnorm_fold_stage1_kernel<A><<<g1, 256, 0, st>>>(partial, partial2, n, slots);
    MP_LAUNCH_CHECK();
    rmsnorm_fold_kernel<T><<<static_cast<unsigned>((n + 31) / 32), rmsnorm_fold_threads(FOLD_SPLITS), 0, st>>>(partial2, ggain, a, blend, n, FOLD_SPLITS);
  } else {
    rmsnorm_fold_kernel<T><<<static_cast<unsigned>((n + 31) / 32), rmsnorm_fold_threads(slots), 0, st>>>(partial, ggain, a, blend, n, slots);
  }
  MP_LAUNCH_CHECK();
  return 0;
}
