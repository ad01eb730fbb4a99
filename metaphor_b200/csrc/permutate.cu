// General permutation of a rank <= MAX_DIMS tensor: dst = permute(src) + alpha*dst.
//
// The reference names this operator ("General Permutation", NOTES.md:3-5; the
// expression grammar `ijk->jik` in src/ops/expression_parsing.zig:205-255) but
// ships only the rank-2 instance (src/cuda/nvcc_src/permutate_ij_ji.cu:43-67,
// bound in src/ops/permutate.zig:39-104).  `perm[i]` is the position of source
// dimension i in the output, the convention of `permutateSizes`.
//
// HBM-bound: every element is read once and written once.  The host collapses
// the shape (size-1 dimensions dropped, dimensions that stay adjacent merged)
// and picks one of two kernels:
//   * innermost dimension kept: whole rows move; groups of 1..32 lanes take a
//     row each (one index decode per row, 16-byte accesses along the row);
//   * innermost dimension moved: square tiles through padded shared memory over
//     (source innermost, output innermost), every other dimension is a batch
//     index decoded once per CTA; both global sides run along a contiguous
//     dimension.
#include "mp_common.cuh"

namespace {

constexpr int PERM_THREADS = 256;

struct PermDims {
  int rank;                                // number of (batch / outer) dimensions listed below
  unsigned long long size[MAX_DIMS];       // slowest first
  unsigned long long sstride[MAX_DIMS];    // source stride of each, in elements
  unsigned long long dstride[MAX_DIMS];    // output stride of each, in elements
};

// ---------------------------------------------------------------------------
// innermost dimension kept: dst rows (output order) <- src rows
// ---------------------------------------------------------------------------
template <typename T, typename I, bool VEC, bool BLEND>
__global__ void __launch_bounds__(PERM_THREADS) permute_rows_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                                    const PermDims o, I pieces, I segs, size_t inner_units,
                                                                    unsigned seg_units, int group_log2) {
  // a row of `inner_units` units (16-byte packs when VEC, else elements) is cut into `segs` pieces of `seg_units`
  constexpr int PN = Pack<T>::N;
  constexpr int UNIT = VEC ? PN : 1;
  const unsigned group_mask = (1u << group_log2) - 1u;
  const size_t tid = static_cast<size_t>(blockIdx.x) * PERM_THREADS + threadIdx.x;
  const size_t groups = (static_cast<size_t>(gridDim.x) * PERM_THREADS) >> group_log2;
  const unsigned sub = static_cast<unsigned>(tid) & group_mask;
  for (size_t piece = tid >> group_log2; piece < pieces; piece += groups) {
    I rem = static_cast<I>(piece);
    const I row = rem / segs;
    const size_t u0 = static_cast<size_t>(rem - row * segs) * seg_units;
    const size_t u1 = u0 + seg_units < inner_units ? u0 + seg_units : inner_units;
    rem = row;
    size_t soff = 0;
#pragma unroll
    for (int k = MAX_DIMS - 1; k >= 0; --k) {
      if (k < o.rank) {
        const I n = static_cast<I>(o.size[k]);
        const I q = rem / n;
        soff += static_cast<size_t>(rem - q * n) * o.sstride[k];
        rem = q;
      }
    }
    const size_t doff = static_cast<size_t>(row) * inner_units * UNIT;
    for (size_t u = u0 + sub; u < u1; u += group_mask + 1u) {
      if constexpr (VEC) {
        Pack<T> p = ld_pack_stream(src, soff / PN + u);
        if constexpr (BLEND) {
          const Pack<T> old = ld_pack_stream(dst, doff / PN + u);
#pragma unroll
          for (int e = 0; e < PN; ++e) p.v[e] = mp_down<T>(mp_up(p.v[e]) + alpha * mp_up(old.v[e]));
        }
        st_pack_stream(dst, doff / PN + u, p);
      } else {
        T v = src[soff + u];
        if constexpr (BLEND) v = mp_down<T>(mp_up(v) + alpha * mp_up(dst[doff + u]));
        dst[doff + u] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// innermost dimension moved: tiles over (S = source innermost, D = output innermost)
//   src element (iD, iS) of a batch at  sbase + iD * s_pitch + iS
//   dst element                     at  dbase + iS * d_pitch + iD
// ---------------------------------------------------------------------------
template <typename T> struct PermTile { static constexpr int value = sizeof(T) == 2 ? 128 : 64; };

template <typename T, bool VL, bool VS, bool BLEND>
__global__ void __launch_bounds__(PERM_THREADS) permute_tiles_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                                     const PermDims batch, size_t n_s, size_t n_d, size_t s_pitch,
                                                                     size_t d_pitch, unsigned tiles_s, unsigned tiles_d) {
  constexpr int PN = Pack<T>::N;
  constexpr int TILE = PermTile<T>::value;
  constexpr int VPR = TILE / PN;
  __shared__ T tile[TILE][TILE + 1];   // tile[s][d]
  size_t rem = blockIdx.x;
  const size_t s0 = (rem % tiles_s) * TILE;
  rem /= tiles_s;
  const size_t d0 = (rem % tiles_d) * TILE;
  rem /= tiles_d;
  size_t sbase = 0, dbase = 0;
#pragma unroll
  for (int k = MAX_DIMS - 1; k >= 0; --k) {
    if (k < batch.rank) {
      const size_t c = rem % batch.size[k];
      rem /= batch.size[k];
      sbase += c * batch.sstride[k];
      dbase += c * batch.dstride[k];
    }
  }
  const int tid = threadIdx.x;
  if constexpr (VL) {
    for (int v = tid; v < TILE * VPR; v += PERM_THREADS) {
      const int td = v / VPR, ts = (v % VPR) * PN;
      if (d0 + td < n_d && s0 + ts < n_s) {
        const Pack<T> p = ld_pack_stream(src, (sbase + (d0 + td) * s_pitch + s0 + ts) / PN);
#pragma unroll
        for (int e = 0; e < PN; ++e) tile[ts + e][td] = p.v[e];
      }
    }
  } else {
    for (int v = tid; v < TILE * TILE; v += PERM_THREADS) {
      const int td = v / TILE, ts = v % TILE;
      if (d0 + td < n_d && s0 + ts < n_s) tile[ts][td] = src[sbase + (d0 + td) * s_pitch + s0 + ts];
    }
  }
  __syncthreads();
  if constexpr (VS) {
    for (int v = tid; v < TILE * VPR; v += PERM_THREADS) {
      const int ts = v / VPR, td = (v % VPR) * PN;
      if (s0 + ts < n_s && d0 + td < n_d) {
        const size_t vi = (dbase + (s0 + ts) * d_pitch + d0 + td) / PN;
        Pack<T> p;
#pragma unroll
        for (int e = 0; e < PN; ++e) p.v[e] = tile[ts][td + e];
        if constexpr (BLEND) {
          const Pack<T> old = ld_pack_stream(dst, vi);
#pragma unroll
          for (int e = 0; e < PN; ++e) p.v[e] = mp_down<T>(mp_up(p.v[e]) + alpha * mp_up(old.v[e]));
        }
        st_pack_stream(dst, vi, p);
      }
    }
  } else {
    for (int v = tid; v < TILE * TILE; v += PERM_THREADS) {
      const int ts = v / TILE, td = v % TILE;
      if (s0 + ts < n_s && d0 + td < n_d) {
        const size_t di = dbase + (s0 + ts) * d_pitch + d0 + td;
        T val = tile[ts][td];
        if constexpr (BLEND) val = mp_down<T>(mp_up(val) + alpha * mp_up(dst[di]));
        dst[di] = val;
      }
    }
  }
}

template <typename T, typename I, bool VEC>
void rows_launch(const T* src, T* dst, double alpha, const PermDims& o, size_t pieces, size_t segs, size_t units, unsigned seg_units,
                 int glog, unsigned grid, cudaStream_t st) {
  using A = typename Acc<T>::type;
  if (alpha == 0.0)
    permute_rows_kernel<T, I, VEC, false><<<grid, PERM_THREADS, 0, st>>>(src, dst, A(0), o, static_cast<I>(pieces), static_cast<I>(segs), units, seg_units, glog);
  else
    permute_rows_kernel<T, I, VEC, true><<<grid, PERM_THREADS, 0, st>>>(src, dst, static_cast<A>(alpha), o, static_cast<I>(pieces), static_cast<I>(segs), units, seg_units, glog);
}

template <typename T, bool VL, bool VS>
void tiles_launch(const T* src, T* dst, double alpha, const PermDims& b, size_t n_s, size_t n_d, size_t s_pitch, size_t d_pitch,
                  unsigned tiles_s, unsigned tiles_d, unsigned grid, cudaStream_t st) {
  using A = typename Acc<T>::type;
  if (alpha == 0.0)
    permute_tiles_kernel<T, VL, VS, false><<<grid, PERM_THREADS, 0, st>>>(src, dst, A(0), b, n_s, n_d, s_pitch, d_pitch, tiles_s, tiles_d);
  else
    permute_tiles_kernel<T, VL, VS, true><<<grid, PERM_THREADS, 0, st>>>(src, dst, static_cast<A>(alpha), b, n_s, n_d, s_pitch, d_pitch, tiles_s, tiles_d);
}

}  // namespace

template <typename T>
static void permutate_impl(const void* src_, void* dst_, double alpha, const len_t* sizes, const len_t* perm, len_t rank,
                           StreamContext ctx) {
  constexpr int PN = Pack<T>::N;
  if (rank == 0 || rank > MAX_DIMS) MP_FATAL("permutate: rank %llu is outside 1..%d", static_cast<unsigned long long>(rank), MAX_DIMS);
  if (sizes == nullptr || perm == nullptr) MP_FATAL("permutate: sizes and perm must be host arrays of `rank` entries");
  const int r = static_cast<int>(rank);
  unsigned seen = 0;
  for (int i = 0; i < r; ++i) {
    if (perm[i] >= rank || (seen >> perm[i]) & 1u) MP_FATAL("permutate: perm is not a permutation of 0..rank-1");
    seen |= 1u << perm[i];
    if (sizes[i] == 0) return;
  }
  // strides of every source dimension on both sides (elements)
  size_t n[MAX_DIMS], ss[MAX_DIMS], ds[MAX_DIMS], out_size[MAX_DIMS], out_stride[MAX_DIMS];
  for (int i = 0; i < r; ++i) out_size[perm[i]] = sizes[i];
  size_t acc = 1;
  for (int j = r - 1; j >= 0; --j) { out_stride[j] = acc; acc *= out_size[j]; }
  const size_t total = acc;
  acc = 1;
  for (int i = r - 1; i >= 0; --i) { ss[i] = acc; acc *= sizes[i]; }
  // collapse: drop size-1 dimensions, merge neighbours that stay neighbours
  int m = 0;
  for (int i = 0; i < r; ++i) {
    if (sizes[i] == 1) continue;
    const size_t d = out_stride[perm[i]];
    if (m > 0 && ds[m - 1] == d * sizes[i]) {
      n[m - 1] *= sizes[i];
      ss[m - 1] = ss[i];
      ds[m - 1] = d;
    } else {
      n[m] = sizes[i];
      ss[m] = ss[i];
      ds[m] = d;
      ++m;
    }
  }
  if (m == 0) { n[0] = 1; ss[0] = 1; ds[0] = 1; m = 1; }
  const T* src = static_cast<const T*>(src_);
  T* dst = static_cast<T*>(dst_);
  cudaStream_t st = mp_stream(ctx);
  const bool aligned = mp_aligned16(src) && mp_aligned16(dst);

  if (ds[m - 1] == 1) {
    // rows of n[m-1] elements; outer dimensions in output order (slowest first)
    PermDims o{};
    int order[MAX_DIMS];
    for (int i = 0; i < m - 1; ++i) order[i] = i;
    for (int i = 1; i < m - 1; ++i)   // insertion sort by output stride, descending
      for (int j = i; j > 0 && ds[order[j]] > ds[order[j - 1]]; --j) { const int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
    o.rank = m - 1;
    for (int i = 0; i < m - 1; ++i) { o.size[i] = n[order[i]]; o.sstride[i] = ss[order[i]]; o.dstride[i] = ds[order[i]]; }
    const size_t inner = n[m - 1], rows = total / inner;
    const bool vec = aligned && inner % PN == 0;
    const size_t units = vec ? inner / PN : inner;
    // long rows are cut into pieces of 256 units (8 per lane) so that a few long rows still fill the machine
    constexpr unsigned SEG_UNITS = 256;
    const size_t segs = (units + SEG_UNITS - 1) / SEG_UNITS;
    const size_t pieces = rows * segs;
    const size_t piece_units = units < SEG_UNITS ? units : SEG_UNITS;
    int glog = 0;
    while (glog < 5 && (1ull << glog) < piece_units) ++glog;
    const size_t threads = pieces << glog;
    size_t blocks = (threads + PERM_THREADS - 1) / PERM_THREADS;
    const size_t cap = static_cast<size_t>(mp_sm_count(ctx)) * 32;   // grid-stride beyond this
    if (blocks > cap) blocks = cap;
    const unsigned grid = static_cast<unsigned>(blocks);
    const bool small = pieces < (1ull << 32);
    if (vec) {
      if (small) rows_launch<T, unsigned, true>(src, dst, alpha, o, pieces, segs, units, SEG_UNITS, glog, grid, st);
      else rows_launch<T, unsigned long long, true>(src, dst, alpha, o, pieces, segs, units, SEG_UNITS, glog, grid, st);
    } else {
      if (small) rows_launch<T, unsigned, false>(src, dst, alpha, o, pieces, segs, units, SEG_UNITS, glog, grid, st);
      else rows_launch<T, unsigned long long, false>(src, dst, alpha, o, pieces, segs, units, SEG_UNITS, glog, grid, st);
    }
    MP_LAUNCH_CHECK();
    return;
  }

  // the source's innermost dimension moves: find the dimension that is innermost in the output
  int d = -1;
  for (int i = 0; i < m; ++i) if (ds[i] == 1) d = i;
  if (d < 0) MP_FATAL("permutate: internal error (no unit output stride)");
  constexpr int TILE = PermTile<T>::value;
  PermDims b{};
  for (int i = 0; i < m - 1; ++i) {
    if (i == d) continue;
    b.size[b.rank] = n[i];
    b.sstride[b.rank] = ss[i];
    b.dstride[b.rank] = ds[i];
    ++b.rank;
  }
  const size_t n_s = n[m - 1], n_d = n[d], s_pitch = ss[d], d_pitch = ds[m - 1];
  const size_t tiles_s = (n_s + TILE - 1) / TILE, tiles_d = (n_d + TILE - 1) / TILE;
  size_t batches = 1;
  for (int i = 0; i < b.rank; ++i) batches *= b.size[i];
  const size_t blocks = tiles_s * tiles_d * batches;
  if (tiles_s >= (1ull << 32) || tiles_d >= (1ull << 32) || blocks >= (1ull << 31)) MP_FATAL("permutate: too many tiles (%llu)", static_cast<unsigned long long>(blocks));
  // 16-byte accesses: every source row start (multiples of n_s) resp. output row start (multiples of n_d) stays aligned
  const bool vl = aligned && n_s % PN == 0;
  const bool vs = aligned && n_d % PN == 0;
  const unsigned grid = static_cast<unsigned>(blocks);
  const unsigned ts = static_cast<unsigned>(tiles_s), td = static_cast<unsigned>(tiles_d);
  if (vl && vs) tiles_launch<T, true, true>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, grid, st);
  else if (vl) tiles_launch<T, true, false>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, grid, st);
  else if (vs) tiles_launch<T, false, true>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, grid, st);
  else tiles_launch<T, false, false>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, grid, st);
  MP_LAUNCH_CHECK();
}

MP_STAMP3(permutate, (const void* src, void* dst, double alpha, const len_t* sizes, const len_t* perm, len_t rank, StreamContext ctx),
          (src, dst, alpha, sizes, perm, rank, ctx))
