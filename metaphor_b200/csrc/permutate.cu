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

constexpr int PERM_DIMS = MAX_DIMS;
struct PermDims {
  int rank;                                // number of (batch / outer) dimensions listed below
  unsigned long long size[PERM_DIMS];      // slowest first (the order rows are visited in)
  unsigned long long sstride[PERM_DIMS];   // source stride of each, in elements
  unsigned long long dstride[PERM_DIMS];   // output stride of each, in elements
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
  const unsigned group_mask = (1u << group_log2) - 1u;
  const size_t tid = static_cast<size_t>(blockIdx.x) * PERM_THREADS + threadIdx.x;
  const size_t groups = (static_cast<size_t>(gridDim.x) * PERM_THREADS) >> group_log2;
  const unsigned sub = static_cast<unsigned>(tid) & group_mask;
  // two pieces per trip: both loads are issued before either store
  for (size_t piece = tid >> group_log2; piece < pieces; piece += 2 * groups) {
    size_t soff[2], doff[2], u0[2], u1[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const size_t pc = piece + h * groups;
      I rem = static_cast<I>(pc < pieces ? pc : piece);
      const I row = rem / segs;
      u0[h] = static_cast<size_t>(rem - row * segs) * seg_units;
      u1[h] = u0[h] + seg_units < inner_units ? u0[h] + seg_units : inner_units;
      if (pc >= pieces) u1[h] = u0[h];   // nothing to do
      rem = row;
      size_t so = 0, dof = 0;
#pragma unroll
      for (int k = PERM_DIMS - 1; k >= 0; --k) {
        if (k < o.rank) {
          const I n = static_cast<I>(o.size[k]);
          const I q = rem / n;
          const size_t c = static_cast<size_t>(rem - q * n);
          so += c * o.sstride[k];
          dof += c * o.dstride[k];
          rem = q;
        }
      }
      soff[h] = so;
      doff[h] = dof;
    }
    const size_t len0 = u1[0] - u0[0], len1 = u1[1] - u0[1];
    const size_t len = len0 > len1 ? len0 : len1;
    for (size_t u = sub; u < len; u += group_mask + 1u) {
      const bool on0 = u < len0, on1 = u < len1;
      if constexpr (VEC) {
        Pack<T> p0, p1;
        if (on0) p0 = ld_pack_stream(src, soff[0] / PN + u0[0] + u);
        if (on1) p1 = ld_pack_stream(src, soff[1] / PN + u0[1] + u);
        if constexpr (BLEND) {
          if (on0) {
            const Pack<T> old = ld_pack_stream(dst, doff[0] / PN + u0[0] + u);
#pragma unroll
            for (int e = 0; e < PN; ++e) p0.v[e] = mp_down<T>(mp_up(p0.v[e]) + alpha * mp_up(old.v[e]));
          }
          if (on1) {
            const Pack<T> old = ld_pack_stream(dst, doff[1] / PN + u0[1] + u);
#pragma unroll
            for (int e = 0; e < PN; ++e) p1.v[e] = mp_down<T>(mp_up(p1.v[e]) + alpha * mp_up(old.v[e]));
          }
        }
        if (on0) st_pack_stream(dst, doff[0] / PN + u0[0] + u, p0);
        if (on1) st_pack_stream(dst, doff[1] / PN + u0[1] + u, p1);
      } else {
        T v0 = T(), v1 = T();
        if (on0) v0 = src[soff[0] + u0[0] + u];
        if (on1) v1 = src[soff[1] + u0[1] + u];
        if constexpr (BLEND) {
          if (on0) v0 = mp_down<T>(mp_up(v0) + alpha * mp_up(dst[doff[0] + u0[0] + u]));
          if (on1) v1 = mp_down<T>(mp_up(v1) + alpha * mp_up(dst[doff[1] + u0[1] + u]));
        }
        if (on0) dst[doff[0] + u0[0] + u] = v0;
        if (on1) dst[doff[1] + u0[1] + u] = v1;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// innermost dimension moved: tiles over (S = source innermost, D = output innermost)
//   src element (iD, iS) of a batch at  sbase + iD * s_pitch + iS
//   dst element                     at  dbase + iS * d_pitch + iD
// A short S or D (fewer elements than a tile edge) is extended by the next dimension on its contiguous side,
// which has a stride of its own on the other side:
//   iD = hi * d_lo + lo  ->  source row at  lo * s_pitch + hi * s_pitch_hi      (d_lo = extent of the short D)
//   iS = hi * s_lo + lo  ->  output row at  lo * d_pitch + hi * d_pitch_hi
// (unsplit: d_lo resp. s_lo = 0).
// ---------------------------------------------------------------------------
struct PermSplit { unsigned d_lo, s_lo; unsigned long long s_pitch_hi, d_pitch_hi; };
template <typename T> struct PermTile { static constexpr int value = sizeof(T) == 2 ? 128 : 64; };

template <typename T, bool VL, bool VS, bool BLEND>
__global__ void __launch_bounds__(PERM_THREADS) permute_tiles_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                                     const PermDims batch, size_t n_s, size_t n_d, size_t s_pitch,
                                                                     size_t d_pitch, unsigned tiles_s, unsigned tiles_d,
                                                                     const PermSplit sp) {
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
  for (int k = PERM_DIMS - 1; k >= 0; --k) {
    if (k < batch.rank) {
      const size_t c = rem % batch.size[k];
      rem /= batch.size[k];
      sbase += c * batch.sstride[k];
      dbase += c * batch.dstride[k];
    }
  }
  const int tid = threadIdx.x;
  auto src_row = [&](size_t id) -> size_t {   // offset of source row iD (split extents stay below 2^31)
    if (sp.d_lo == 0) return id * s_pitch;
    const unsigned hi = static_cast<unsigned>(id) / sp.d_lo;
    return static_cast<size_t>(static_cast<unsigned>(id) - hi * sp.d_lo) * s_pitch + hi * sp.s_pitch_hi;
  };
  auto dst_row = [&](size_t is) -> size_t {   // offset of output row iS
    if (sp.s_lo == 0) return is * d_pitch;
    const unsigned hi = static_cast<unsigned>(is) / sp.s_lo;
    return static_cast<size_t>(static_cast<unsigned>(is) - hi * sp.s_lo) * d_pitch + hi * sp.d_pitch_hi;
  };
  if constexpr (VL) {
    for (int v = tid; v < TILE * VPR; v += PERM_THREADS) {
      const int td = v / VPR, ts = (v % VPR) * PN;
      if (d0 + td < n_d && s0 + ts < n_s) {
        const Pack<T> p = ld_pack_stream(src, (sbase + src_row(d0 + td) + s0 + ts) / PN);
#pragma unroll
        for (int e = 0; e < PN; ++e) tile[ts + e][td] = p.v[e];
      }
    }
  } else {
    for (int v = tid; v < TILE * TILE; v += PERM_THREADS) {
      const int td = v / TILE, ts = v % TILE;
      if (d0 + td < n_d && s0 + ts < n_s) tile[ts][td] = src[sbase + src_row(d0 + td) + s0 + ts];
    }
  }
  __syncthreads();
  if constexpr (VS) {
    for (int v = tid; v < TILE * VPR; v += PERM_THREADS) {
      const int ts = v / VPR, td = (v % VPR) * PN;
      if (s0 + ts < n_s && d0 + td < n_d) {
        const size_t vi = (dbase + dst_row(s0 + ts) + d0 + td) / PN;
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
        const size_t di = dbase + dst_row(s0 + ts) + d0 + td;
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
                  unsigned tiles_s, unsigned tiles_d, const PermSplit& sp, unsigned grid, cudaStream_t st) {
  using A = typename Acc<T>::type;
  if (alpha == 0.0)
    permute_tiles_kernel<T, VL, VS, false><<<grid, PERM_THREADS, 0, st>>>(src, dst, A(0), b, n_s, n_d, s_pitch, d_pitch, tiles_s, tiles_d, sp);
  else
    permute_tiles_kernel<T, VL, VS, true><<<grid, PERM_THREADS, 0, st>>>(src, dst, static_cast<A>(alpha), b, n_s, n_d, s_pitch, d_pitch, tiles_s, tiles_d, sp);
}

}  // namespace

// Runs a collapsed permutation: m dimensions of sizes n, source strides ss, output strides ds (elements of T;
// the source is contiguous, so ss[m-1] == 1).
template <typename T>
static void permutate_run(const T* src, T* dst, double alpha, const size_t* n, const size_t* ss, const size_t* ds, int m,
                          StreamContext ctx) {
  constexpr int PN = Pack<T>::N;
  cudaStream_t st = mp_stream(ctx);
  const bool aligned = mp_aligned16(src) && mp_aligned16(dst);
  size_t total = 1;
  for (int i = 0; i < m; ++i) total *= n[i];

  if (ds[m - 1] == 1) {
    // rows of n[m-1] elements; outer dimensions in output order (slowest first)
    PermDims o{};
    int order[MAX_DIMS];
    for (int i = 0; i < m - 1; ++i) order[i] = i;
    for (int i = 1; i < m - 1; ++i)   // insertion sort by output stride, descending
      for (int j = i; j > 0 && ds[order[j]] > ds[order[j - 1]]; --j) { const int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t; }
    const size_t inner = n[m - 1], rows = total / inner;
    // rows are visited in output order (a blocked order over the fastest output / source dimensions was
    // measured slower: 2.9 instead of 4.2 TB/s on [8, 2048, 32, 128] r16 "blhd->bhld")
    o.rank = m - 1;
    for (int i = 0; i < m - 1; ++i) { o.size[i] = n[order[i]]; o.sstride[i] = ss[order[i]]; o.dstride[i] = ds[order[i]]; }
    const bool vec = aligned && inner % PN == 0;
    const size_t units = vec ? inner / PN : inner;
    // long rows are cut into pieces of 256 units (8 per lane) so that a few long rows still fill the machine
    constexpr unsigned SEG_UNITS = 256;
    const size_t segs = (units + SEG_UNITS - 1) / SEG_UNITS;
    const size_t pieces = rows * segs;
    const size_t piece_units = units < SEG_UNITS ? units : SEG_UNITS;
    int glog = 0;
    while (glog < 5 && (1ull << glog) < piece_units) ++glog;
    const size_t threads = ((pieces + 1) / 2) << glog;   // a lane group takes two pieces per trip
    size_t blocks = (threads + PERM_THREADS - 1) / PERM_THREADS;
    const size_t cap = static_cast<size_t>(mp_sm_count(ctx)) * 32;   // grid-stride beyond this
    if (blocks > cap) blocks = cap;
    const unsigned grid = static_cast<unsigned>(blocks);
    const bool small = pieces < (1ull << 31);
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
  size_t n_s = n[m - 1], n_d = n[d];
  const size_t s_pitch = ss[d], d_pitch = ds[m - 1];
  PermSplit sp{0, 0, 0, 0};
  int d_hi = -1, s_hi = -1;
  if (n_d < TILE) {   // the dimension that follows D in the output (stride n_d there)
    for (int i = 0; i < m - 1; ++i)
      if (i != d && ds[i] == n_d && n_d * n[i] < (1ull << 31)) d_hi = i;
    if (d_hi >= 0) { sp.d_lo = static_cast<unsigned>(n_d); sp.s_pitch_hi = ss[d_hi]; n_d *= n[d_hi]; }
  }
  if (n_s < TILE && m >= 2 && m - 2 != d && m - 2 != d_hi && n_s * n[m - 2] < (1ull << 31)) {   // the dimension before S in the source
    s_hi = m - 2;
    sp.s_lo = static_cast<unsigned>(n_s);
    sp.d_pitch_hi = ds[s_hi];
    n_s *= n[s_hi];
  }
  PermDims b{};
  for (int i = 0; i < m - 1; ++i) {
    if (i == d || i == d_hi || i == s_hi) continue;
    b.size[b.rank] = n[i];
    b.sstride[b.rank] = ss[i];
    b.dstride[b.rank] = ds[i];
    ++b.rank;
  }
  const size_t tiles_s = (n_s + TILE - 1) / TILE, tiles_d = (n_d + TILE - 1) / TILE;
  size_t batches = 1;
  for (int i = 0; i < b.rank; ++i) batches *= b.size[i];
  const size_t blocks = tiles_s * tiles_d * batches;
  if (tiles_s >= (1ull << 32) || tiles_d >= (1ull << 32) || blocks >= (1ull << 31)) MP_FATAL("permutate: too many tiles (%llu)", static_cast<unsigned long long>(blocks));
  // 16-byte accesses: every source run (multiples of the short S extent) resp. output run stays aligned
  const bool vl = aligned && n[m - 1] % PN == 0;
  const bool vs = aligned && n[d] % PN == 0;
  const unsigned grid = static_cast<unsigned>(blocks);
  const unsigned ts = static_cast<unsigned>(tiles_s), td = static_cast<unsigned>(tiles_d);
  if (vl && vs) tiles_launch<T, true, true>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, sp, grid, st);
  else if (vl) tiles_launch<T, true, false>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, sp, grid, st);
  else if (vs) tiles_launch<T, false, true>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, sp, grid, st);
  else tiles_launch<T, false, false>(src, dst, alpha, b, n_s, n_d, s_pitch, d_pitch, ts, td, sp, grid, st);
  MP_LAUNCH_CHECK();
}

template <typename T>
static void permutate_impl(const void* src_, void* dst_, double alpha, const len_t* sizes, const len_t* perm, len_t rank,
                           StreamContext ctx) {
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
  // A pure move (alpha == 0) of short kept rows is a permutation of wider elements: rows of 4 or 8 bytes become one
  // r32- resp. r64-sized element and the kept dimension disappears (tiles instead of scalar row copies).
  if (alpha == 0.0 && m >= 2 && ds[m - 1] == 1) {
    const size_t row_bytes = n[m - 1] * sizeof(T);
    if ((row_bytes == 4 || row_bytes == 8) && row_bytes > sizeof(T) && reinterpret_cast<uintptr_t>(src) % row_bytes == 0 &&
        reinterpret_cast<uintptr_t>(dst) % row_bytes == 0) {
      const size_t w = n[m - 1];
      for (int i = 0; i < m - 1; ++i) { ss[i] /= w; ds[i] /= w; }
      // the remaining dimensions may merge further now, which the run does not need: strides stay valid as they are
      if (row_bytes == 4) permutate_run<float>(reinterpret_cast<const float*>(src), reinterpret_cast<float*>(dst), 0.0, n, ss, ds, m - 1, ctx);
      else permutate_run<double>(reinterpret_cast<const double*>(src), reinterpret_cast<double*>(dst), 0.0, n, ss, ds, m - 1, ctx);
      return;
    }
  }
  permutate_run<T>(src, dst, alpha, n, ss, ds, m, ctx);
}

MP_STAMP3(permutate, (const void* src, void* dst, double alpha, const len_t* sizes, const len_t* perm, len_t rank, StreamContext ctx),
          (src, dst, alpha, sizes, perm, rank, ctx))
