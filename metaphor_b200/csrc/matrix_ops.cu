// Rank-2 data-movement launchers: transpose, row/column sums, row/column
// broadcasts.  All HBM-bound; 128-bit global accesses where the shape and the
// pointers allow, scalar accesses otherwise, 64-bit indexing throughout.
//
// Replaces permutate_ij_ji.cu, reduce_ij_i.cu, reduce_ij_j.cu,
// broadcast_i_ij.cu, broadcast_j_ij.cu of the reference (src/cuda/nvcc_src/).
// Each kernel implements the documented formula `value + alpha*dst`; dst is
// not read when alpha == 0.
#include "mp_common.cuh"

namespace {

// ------------------------------ transpose ---------------------------------
constexpr int TP_THREADS = 256;
// tile edge in elements: 128 for 2-byte types (256-byte row segments), else 64
template <typename T> struct TpTile { static constexpr int value = sizeof(T) == 2 ? 128 : 64; };

// dst[c, r] = src[r, c] + alpha*dst[c, r]; src is [row, col] row-major.
// One square tile per CTA through padded shared memory; VL / VS select 128-bit
// global loads / stores (legal when col resp. row is a multiple of the pack
// width and the base pointer is 16-byte aligned).
template <typename T, bool VL, bool VS, bool BLEND>
__global__ void __launch_bounds__(TP_THREADS) transpose_kernel(const T* __restrict__ src, T* dst,
                                                               typename Acc<T>::type alpha, size_t row, size_t col) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int TP_TILE = TpTile<T>::value;
  constexpr int VPR = TP_TILE / PN;  // packs per tile row
  __shared__ T tile[TP_TILE][TP_TILE + 1];
  const size_t r0 = static_cast<size_t>(blockIdx.y) * TP_TILE;
  const size_t c0 = static_cast<size_t>(blockIdx.x) * TP_TILE;
  const int tid = threadIdx.x;

  if constexpr (VL) {
    // two stages: the loads of a group of trips are in flight before the first value is used (r16 / r32: all of the
    // thread's loads; r64: groups of 4, because holding all 8 costs a CTA per SM and measured 11 - 15 % slower)
    constexpr int TRIPS = TP_TILE * VPR / TP_THREADS;
    constexpr int GROUP = sizeof(T) == 8 ? 2 : TRIPS;
#pragma unroll
    for (int t0 = 0; t0 < TRIPS; t0 += GROUP) {
      Pack<T> p[GROUP];
#pragma unroll
      for (int t = 0; t < GROUP; ++t) {
        const int v = tid + (t0 + t) * TP_THREADS, tr = v / VPR, tc = (v % VPR) * PN;
        if (r0 + tr < row && c0 + tc < col) p[t] = ld_pack_stream(src, ((r0 + tr) * col + c0 + tc) / PN);
      }
#pragma unroll
      for (int t = 0; t < GROUP; ++t) {
        const int v = tid + (t0 + t) * TP_THREADS, tr = v / VPR, tc = (v % VPR) * PN;
        if (r0 + tr < row && c0 + tc < col) {
#pragma unroll
          for (int e = 0; e < PN; ++e) tile[tc + e][tr] = p[t].v[e];
        }
      }
    }
  } else {
    for (int v = tid; v < TP_TILE * TP_TILE; v += TP_THREADS) {
      const int tr = v / TP_TILE, tc = v % TP_TILE;
      if (r0 + tr < row && c0 + tc < col) tile[tc][tr] = src[(r0 + tr) * col + c0 + tc];
    }
  }
  __syncthreads();

  // tile[c][r] now holds src[r0 + r, c0 + c]; dst rows are indexed by c.
  if constexpr (VS) {
    for (int v = tid; v < TP_TILE * VPR; v += TP_THREADS) {
      const int tc = v / VPR, tr = (v % VPR) * PN;
      if (c0 + tc < col && r0 + tr < row) {
        const size_t vi = ((c0 + tc) * row + r0 + tr) / PN;
        Pack<T> p;
#pragma unroll
        for (int e = 0; e < PN; ++e) p.v[e] = tile[tc][tr + e];
        if constexpr (BLEND) {
          const Pack<T> old = ld_pack_stream(dst, vi);
#pragma unroll
          for (int e = 0; e < PN; ++e) p.v[e] = mp_down<T>(mp_up(p.v[e]) + alpha * mp_up(old.v[e]));
        }
        st_pack_stream(dst, vi, p);
      }
    }
  } else {
    for (int v = tid; v < TP_TILE * TP_TILE; v += TP_THREADS) {
      const int tc = v / TP_TILE, tr = v % TP_TILE;
      if (c0 + tc < col && r0 + tr < row) {
        const size_t di = (c0 + tc) * row + r0 + tr;
        T val = tile[tc][tr];
        if constexpr (BLEND) val = mp_down<T>(mp_up(val) + alpha * mp_up(dst[di]));
        dst[di] = val;
      }
    }
  }
}

template <typename T, bool VL, bool VS>
void transpose_dispatch(const T* src, T* dst, double alpha, size_t row, size_t col, dim3 grid, cudaStream_t st) {
  using A = typename Acc<T>::type;
  if (alpha == 0.0) transpose_kernel<T, VL, VS, false><<<grid, TP_THREADS, 0, st>>>(src, dst, A(0), row, col);
  else transpose_kernel<T, VL, VS, true><<<grid, TP_THREADS, 0, st>>>(src, dst, static_cast<A>(alpha), row, col);
}

// ------------------------------- row sums ---------------------------------
// dst[i] = sum_j src[i, j] + alpha*dst[i].  GROUP threads cooperate on a row
// (32 = one warp, several rows per CTA; otherwise the whole CTA), rows are
// visited grid-stride.
template <typename T, int GROUP, bool VEC>
__global__ void __launch_bounds__(256) row_sum_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                      bool blend, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  static_assert(GROUP == 32, "one warp per row");
  constexpr int ROWS = 256 / GROUP;
  const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
  for (size_t r = static_cast<size_t>(blockIdx.x) * ROWS + g; r < m; r += static_cast<size_t>(gridDim.x) * ROWS) {
    const T* p = src + r * n;
    A acc = A(0);
    if constexpr (VEC) {
      const size_t nv = n / PN;
      A part[4] = {A(0), A(0), A(0), A(0)};
      size_t v = t;
      for (; v + 3 * GROUP < nv; v += 4 * GROUP) {
        Pack<T> q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) q[u] = ld_pack_stream(p, v + u * GROUP);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < PN; ++e) part[u] += mp_up(q[u].v[e]);
      }
      for (; v < nv; v += GROUP) {
        const Pack<T> q = ld_pack_stream(p, v);
#pragma unroll
        for (int e = 0; e < PN; ++e) part[0] += mp_up(q.v[e]);
      }
      acc = (part[0] + part[1]) + (part[2] + part[3]);
    } else {
      for (size_t j = t; j < n; j += GROUP) acc += mp_up(p[j]);
    }
    acc = warp_reduce<SumOp>(acc);
    if (t == 0) dst[r] = mp_down<T>(blend ? acc + alpha * mp_up(dst[r]) : acc);
  }
}

// CTA-wide variant needs every thread of the CTA in the loop (barriers).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) row_sum_cta_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                          bool blend, size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  __shared__ A red[32];
  const int t = threadIdx.x;
  for (size_t r = blockIdx.x; r < m; r += gridDim.x) {
    const T* p = src + r * n;
    A acc = A(0);
    if constexpr (VEC) {
      const size_t nv = n / PN;
      A part[4] = {A(0), A(0), A(0), A(0)};
      size_t v = t;
      for (; v + 3 * 256 < nv; v += 4 * 256) {
        Pack<T> q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) q[u] = ld_pack_stream(p, v + u * 256);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < PN; ++e) part[u] += mp_up(q[u].v[e]);
      }
      for (; v < nv; v += 256) {
        const Pack<T> q = ld_pack_stream(p, v);
#pragma unroll
        for (int e = 0; e < PN; ++e) part[0] += mp_up(q.v[e]);
      }
      acc = (part[0] + part[1]) + (part[2] + part[3]);
    } else {
      for (size_t j = t; j < n; j += 256) acc += mp_up(p[j]);
    }
    acc = cta_reduce<SumOp, 256>(acc, red, A(0));
    if (t == 0) dst[r] = mp_down<T>(blend ? acc + alpha * mp_up(dst[r]) : acc);
  }
}

// ------------------------------ column sums -------------------------------
// Stage 1: CTA (strip s, split p) sums rows [p*rows_per_split, ...) of a strip
// of 32*W columns (W = pack width when VEC, else 1).  Warps stride the rows,
// lanes own columns; the eight warp partials meet in shared memory.  With one
// split the result goes straight to dst, else to partial[p][n] (arithmetic
// type) and stage 2 folds the splits in a fixed order: deterministic, no atomics.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) col_sum_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type* partial,
                                                      typename Acc<T>::type alpha, bool blend, size_t m, size_t n,
                                                      size_t rows_per_split) {
  using A = typename Acc<T>::type;
  constexpr int W = VEC ? Pack<T>::N : 1;
  __shared__ A sm[8][32 * W + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t c = (static_cast<size_t>(blockIdx.x) * 32 + lane) * W;
  const size_t rbeg = static_cast<size_t>(blockIdx.y) * rows_per_split;
  size_t rend = rbeg + rows_per_split; if (rend > m) rend = m;
  A acc[W];
#pragma unroll
  for (int e = 0; e < W; ++e) acc[e] = A(0);
  if (c < n) {
    if constexpr (VEC) {
      size_t r = rbeg + warp;
      for (; r + 24 < rend; r += 32) {
        Pack<T> q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) q[u] = ld_pack_stream(src, ((r + 8 * u) * n + c) / W);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < W; ++e) acc[e] += mp_up(q[u].v[e]);
      }
      for (; r < rend; r += 8) {
        const Pack<T> q = ld_pack_stream(src, (r * n + c) / W);
#pragma unroll
        for (int e = 0; e < W; ++e) acc[e] += mp_up(q.v[e]);
      }
    } else {
      for (size_t r = rbeg + warp; r < rend; r += 8) acc[0] += mp_up(src[r * n + c]);
    }
  }
#pragma unroll
  for (int e = 0; e < W; ++e) sm[warp][lane * W + e] = acc[e];
  __syncthreads();
  for (int j = threadIdx.x; j < 32 * W; j += 256) {
    const size_t col = static_cast<size_t>(blockIdx.x) * 32 * W + j;
    if (col < n) {
      A s = A(0);
#pragma unroll
      for (int w = 0; w < 8; ++w) s += sm[w][j];
      if (gridDim.y == 1) dst[col] = mp_down<T>(blend ? s + alpha * mp_up(dst[col]) : s);
      else partial[static_cast<size_t>(blockIdx.y) * n + col] = s;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) col_sum_fold_kernel(const typename Acc<T>::type* __restrict__ partial, T* dst,
                                                           typename Acc<T>::type alpha, bool blend, size_t n, int splits) {
  using A = typename Acc<T>::type;
  const size_t col = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (col >= n) return;
  A s = A(0);
  for (int p = 0; p < splits; ++p) s += partial[static_cast<size_t>(p) * n + col];
  dst[col] = mp_down<T>(blend ? s + alpha * mp_up(dst[col]) : s);
}

// ------------------------------- broadcasts -------------------------------
// BY_ROW: dst[i,j] = src[i] + alpha*dst[i,j];  else dst[i,j] = src[j] + alpha*dst[i,j].
template <typename T, bool BY_ROW, bool VEC, bool BLEND>
__global__ void __launch_bounds__(256) broadcast_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                        size_t m, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t total = m * n;
  if constexpr (VEC) {
    const size_t nvec = total / PN;  // n % PN == 0: a pack never straddles rows
    constexpr int U = 4;
    for (size_t base = static_cast<size_t>(blockIdx.x) * 256 * U; base < nvec;
         base += static_cast<size_t>(gridDim.x) * 256 * U) {
      Pack<T> out[U], old[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vi = base + u * 256 + threadIdx.x;
        if (vi < nvec) {
          const size_t e0 = vi * PN;
          if constexpr (BY_ROW) {
            const T s = src[e0 / n];
#pragma unroll
            for (int e = 0; e < PN; ++e) out[u].v[e] = s;
          } else {
            out[u] = ld_pack(src, (e0 % n) / PN);
          }
          if constexpr (BLEND) old[u] = ld_pack_stream(dst, vi);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vi = base + u * 256 + threadIdx.x;
        if (vi < nvec) {
          if constexpr (BLEND) {
#pragma unroll
            for (int e = 0; e < PN; ++e) out[u].v[e] = mp_down<T>(mp_up(out[u].v[e]) + alpha * mp_up(old[u].v[e]));
          }
          st_pack_stream(dst, vi, out[u]);
        }
      }
    }
  } else {
    for (size_t i = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * 256) {
      T s = BY_ROW ? src[i / n] : src[i % n];
      if constexpr (BLEND) s = mp_down<T>(mp_up(s) + alpha * mp_up(dst[i]));
      dst[i] = s;
    }
  }
}

template <typename T, bool BY_ROW>
void broadcast_launch(const void* src_, void* dst_, double alpha, len_t m, len_t n, StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (m == 0 || n == 0) return;
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  constexpr int PN = Pack<T>::N;
  const bool vec = (n % PN == 0) && mp_aligned16(dst) && (BY_ROW || mp_aligned16(src));
  const size_t work = vec ? ((m * n) / PN + 3) / 4 : m * n;  // 4 packs per thread when vectorised
  size_t grid = (work + 255) / 256;   // one trip per CTA streams fastest on B200
  const size_t cap = 1u << 30;
  if (grid > cap) grid = cap;
  cudaStream_t st = mp_stream(ctx);
  const A a = static_cast<A>(alpha);
  const unsigned g = static_cast<unsigned>(grid);
  if (vec) {
    if (alpha == 0.0) broadcast_kernel<T, BY_ROW, true, false><<<g, 256, 0, st>>>(src, dst, a, m, n);
    else broadcast_kernel<T, BY_ROW, true, true><<<g, 256, 0, st>>>(src, dst, a, m, n);
  } else {
    if (alpha == 0.0) broadcast_kernel<T, BY_ROW, false, false><<<g, 256, 0, st>>>(src, dst, a, m, n);
    else broadcast_kernel<T, BY_ROW, false, true><<<g, 256, 0, st>>>(src, dst, a, m, n);
  }
  MP_LAUNCH_CHECK();
}

}  // namespace

template <typename T>
static void permutate_ij_ji_impl(const void* src_, void* dst_, double alpha, len_t row, len_t col, StreamContext ctx) {
  if (row == 0 || col == 0) return;
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  constexpr int PN = Pack<T>::N;
  constexpr int TP_TILE = TpTile<T>::value;
  const size_t gx = (col + TP_TILE - 1) / TP_TILE, gy = (row + TP_TILE - 1) / TP_TILE;
  if (gy > 65535) MP_FATAL("permutate_ij_ji: more than 65535 row tiles is not supported");
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  const bool vl = (col % PN == 0) && mp_aligned16(src);
  const bool vs = (row % PN == 0) && mp_aligned16(dst);
  if constexpr (std::is_same<T, __half>::value) {
    if (vl && vs) {   // the general permutation's r16 tile kernel (row pairs as 32-bit words) is faster: 4.65 vs 4.1 TB/s
      const len_t sizes[2] = {row, col}, perm[2] = {1, 0};
      launch_permutate_r16(src_, dst_, alpha, sizes, perm, 2, ctx);
      return;
    }
  }
  cudaStream_t st = mp_stream(ctx);
  if (vl && vs) transpose_dispatch<T, true, true>(src, dst, alpha, row, col, grid, st);
  else if (vl) transpose_dispatch<T, true, false>(src, dst, alpha, row, col, grid, st);
  else if (vs) transpose_dispatch<T, false, true>(src, dst, alpha, row, col, grid, st);
  else transpose_dispatch<T, false, false>(src, dst, alpha, row, col, grid, st);
  MP_LAUNCH_CHECK();
}

template <typename T>
static void reduce_ij_i_impl(const void* src_, void* dst_, double alpha, len_t m, len_t n, StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (m == 0) return;
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  constexpr int PN = Pack<T>::N;
  const bool vec = (n % PN == 0) && mp_aligned16(src);
  const bool blend = alpha != 0.0;
  const A a = static_cast<A>(alpha);
  const size_t cap = 1u << 30;  // one row (group) per CTA; the loop only runs for larger m
  cudaStream_t st = mp_stream(ctx);
  if (n * sizeof(T) <= 4096) {  // short rows: one warp each, 8 rows per CTA
    size_t grid = (m + 7) / 8; if (grid > cap) grid = cap;
    if (vec) row_sum_kernel<T, 32, true><<<static_cast<unsigned>(grid), 256, 0, st>>>(src, dst, a, blend, m, n);
    else row_sum_kernel<T, 32, false><<<static_cast<unsigned>(grid), 256, 0, st>>>(src, dst, a, blend, m, n);
  } else {
    size_t grid = m; if (grid > cap) grid = cap;
    if (vec) row_sum_cta_kernel<T, true><<<static_cast<unsigned>(grid), 256, 0, st>>>(src, dst, a, blend, m, n);
    else row_sum_cta_kernel<T, false><<<static_cast<unsigned>(grid), 256, 0, st>>>(src, dst, a, blend, m, n);
  }
  MP_LAUNCH_CHECK();
}

template <typename T>
static void reduce_ij_j_impl(const void* src_, void* dst_, double alpha, len_t m, len_t n, StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (n == 0) return;
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  constexpr int PN = Pack<T>::N;
  const bool vec = (n % PN == 0) && mp_aligned16(src);
  const bool blend = alpha != 0.0;
  const A a = static_cast<A>(alpha);
  cudaStream_t st = mp_stream(ctx);
  const size_t strip = 32 * (vec ? PN : 1);
  const size_t strips = (n + strip - 1) / strip;
  // ~256 rows per CTA: many short-lived CTAs stream faster than a few long
  // ones; the partials (splits x n) must fit the stream's workspace
  MpStreamState* state = mp_state_or_null(ctx);
  size_t splits = 1;
  if (state != nullptr && m > 0) {
    const size_t by_rows = (m + 255) / 256;
    const size_t by_ws = state->workspace_bytes / (n * sizeof(A));
    splits = by_rows;
    if (splits > by_ws) splits = by_ws;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
  }
  size_t rows_per_split = (m + splits - 1) / splits;
  if (rows_per_split == 0) rows_per_split = 1;
  splits = m == 0 ? 1 : (m + rows_per_split - 1) / rows_per_split;
  A* partial = splits > 1 ? static_cast<A*>(state->workspace) : nullptr;
  const dim3 grid(static_cast<unsigned>(strips), static_cast<unsigned>(splits));
  if (vec) col_sum_kernel<T, true><<<grid, 256, 0, st>>>(src, dst, partial, a, blend, m, n, rows_per_split);
  else col_sum_kernel<T, false><<<grid, 256, 0, st>>>(src, dst, partial, a, blend, m, n, rows_per_split);
  MP_LAUNCH_CHECK();
  if (splits > 1) {
    col_sum_fold_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(partial, dst, a, blend, n,
                                                                                   static_cast<int>(splits));
    MP_LAUNCH_CHECK();
  }
}

template <typename T>
static void broadcast_i_ij_impl(const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext ctx) {
  broadcast_launch<T, true>(src, dst, alpha, m, n, ctx);
}
template <typename T>
static void broadcast_j_ij_impl(const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext ctx) {
  broadcast_launch<T, false>(src, dst, alpha, m, n, ctx);
}

MP_STAMP3(permutate_ij_ji, (const void* src, void* dst, double alpha, len_t row, len_t col, StreamContext ctx), (src, dst, alpha, row, col, ctx))
MP_STAMP3(reduce_ij_i, (const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext ctx), (src, dst, alpha, m, n, ctx))
MP_STAMP3(reduce_ij_j, (const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext ctx), (src, dst, alpha, m, n, ctx))
MP_STAMP3(broadcast_i_ij, (const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext ctx), (src, dst, alpha, m, n, ctx))
MP_STAMP3(broadcast_j_ij, (const void* src, void* dst, double alpha, len_t m, len_t n, StreamContext ctx), (src, dst, alpha, m, n, ctx))
