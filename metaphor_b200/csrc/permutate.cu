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
  // A row of `inner_units` units (16-byte packs when VEC, else elements) is cut into `segs` pieces of `seg_units`.
  // A warp takes 32 consecutive pieces: every lane decodes ONE piece (the index arithmetic costs more than the
  // copy of a short row), then the warp walks the 32 pieces with 2^group_log2 lanes per piece, the offsets
  // handed around by shuffles; two steps are in flight at a time.
  constexpr int PN = Pack<T>::N;
  constexpr int UNIT = VEC ? PN : 1;
  const int lane = threadIdx.x & 31;
  const int group = 1 << group_log2;
  const int sub = lane & (group - 1);
  const int per_step = 32 >> group_log2;   // pieces per step
  const size_t warp = (static_cast<size_t>(blockIdx.x) * PERM_THREADS + threadIdx.x) >> 5;
  const size_t warps = (static_cast<size_t>(gridDim.x) * PERM_THREADS) >> 5;
  for (size_t base = warp * 32; base < pieces; base += warps * 32) {
    const size_t piece = base + lane;
    size_t my_s = 0, my_d = 0;     // first unit of the piece on both sides
    unsigned my_len = 0;           // units in the piece (0: past the end)
    if (piece < pieces) {
      I rem = static_cast<I>(piece);
      const I row = rem / segs;
      const size_t u0 = static_cast<size_t>(rem - row * segs) * seg_units;
      my_len = static_cast<unsigned>(u0 + seg_units < inner_units ? seg_units : inner_units - u0);
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
      my_s = so / UNIT + u0;       // every stride is a multiple of the row length, hence of UNIT
      my_d = dof / UNIT + u0;
    }
    for (int t = 0; t < 32; t += 2 * per_step) {
      size_t so[2], dof[2];
      unsigned len[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int from = (t + h * per_step + (lane >> group_log2)) & 31;
        so[h] = __shfl_sync(0xffffffffu, my_s, from);
        dof[h] = __shfl_sync(0xffffffffu, my_d, from);
        len[h] = __shfl_sync(0xffffffffu, my_len, from);
        if (t + h * per_step >= 32) len[h] = 0;   // one lane per piece: a single step covers all 32
      }
      const unsigned longest = len[0] > len[1] ? len[0] : len[1];
      for (unsigned u = sub; u < longest; u += group) {
        const bool on0 = u < len[0], on1 = u < len[1];
        if constexpr (VEC) {
          Pack<T> p0, p1;
          if (on0) p0 = ld_pack_stream(src, so[0] + u);
          if (on1) p1 = ld_pack_stream(src, so[1] + u);
          if constexpr (BLEND) {
            if (on0) {
              const Pack<T> old = ld_pack_stream(dst, dof[0] + u);
#pragma unroll
              for (int e = 0; e < PN; ++e) p0.v[e] = mp_down<T>(mp_up(p0.v[e]) + alpha * mp_up(old.v[e]));
            }
            if (on1) {
              const Pack<T> old = ld_pack_stream(dst, dof[1] + u);
#pragma unroll
              for (int e = 0; e < PN; ++e) p1.v[e] = mp_down<T>(mp_up(p1.v[e]) + alpha * mp_up(old.v[e]));
            }
          }
          if (on0) st_pack_stream(dst, dof[0] + u, p0);
          if (on1) st_pack_stream(dst, dof[1] + u, p1);
        } else {
          T v0 = T(), v1 = T();
          if (on0) v0 = src[so[0] + u];
          if (on1) v1 = src[so[1] + u];
          if constexpr (BLEND) {
            if (on0) v0 = mp_down<T>(mp_up(v0) + alpha * mp_up(dst[dof[0] + u]));
            if (on1) v1 = mp_down<T>(mp_up(v1) + alpha * mp_up(dst[dof[1] + u]));
          }
          if (on0) dst[dof[0] + u] = v0;
          if (on1) dst[dof[1] + u] = v1;
        }
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

// blockIdx.x -> origin of the CTA's tile and the offsets of its batch indices.  The block index has 32 bits, so
// the divisions have too (a 64-bit division is ~4 times the instructions, and every warp of the CTA decodes).
__device__ __forceinline__ void decode_tile(const PermDims& batch, unsigned tiles_s, unsigned tiles_d, int tile, size_t& s0, size_t& d0,
                                            size_t& sbase, size_t& dbase) {
  unsigned rem = blockIdx.x;
  unsigned q = rem / tiles_s;
  s0 = static_cast<size_t>(rem - q * tiles_s) * tile;
  rem = q;
  q = rem / tiles_d;
  d0 = static_cast<size_t>(rem - q * tiles_d) * tile;
  rem = q;
  sbase = 0;
  dbase = 0;
#pragma unroll
  for (int k = PERM_DIMS - 1; k >= 0; --k) {
    if (k < batch.rank) {
      const unsigned extent = batch.size[k] > 0xffffffffull ? 0xffffffffu : static_cast<unsigned>(batch.size[k]);   // > rem either way
      q = rem / extent;
      const unsigned c = rem - q * extent;
      rem = q;
      sbase += static_cast<size_t>(c) * batch.sstride[k];
      dbase += static_cast<size_t>(c) * batch.dstride[k];
    }
  }
}

template <typename T, bool VL, bool VS, bool BLEND>
__global__ void __launch_bounds__(PERM_THREADS) permute_tiles_kernel(const T* __restrict__ src, T* dst, typename Acc<T>::type alpha,
                                                                     const PermDims batch, size_t n_s, size_t n_d, size_t s_pitch,
                                                                     size_t d_pitch, unsigned tiles_s, unsigned tiles_d,
                                                                     const PermSplit sp) {
  constexpr int PN = Pack<T>::N;
  constexpr int TILE = PermTile<T>::value;
  constexpr int VPR = TILE / PN;
  __shared__ T tile[TILE][TILE + 1];   // tile[s][d]
  size_t s0, d0, sbase, dbase;
  decode_tile(batch, tiles_s, tiles_d, TILE, s0, d0, sbase, dbase);
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
    // two stages: the loads of a group of trips are in flight before the first value is used (r16 / r32: all of the
    // thread's loads; r64: groups of 4, because holding all 8 costs a CTA per SM and measured 11 - 15 % slower)
    constexpr int TRIPS = TILE * VPR / PERM_THREADS;
    constexpr int GROUP = sizeof(T) == 8 ? 2 : TRIPS;
#pragma unroll
    for (int t0 = 0; t0 < TRIPS; t0 += GROUP) {
      Pack<T> p[GROUP];
#pragma unroll
      for (int t = 0; t < GROUP; ++t) {
        const int v = tid + (t0 + t) * PERM_THREADS, td = v / VPR, ts = (v % VPR) * PN;
        if (d0 + td < n_d && s0 + ts < n_s) p[t] = ld_pack_stream(src, (sbase + src_row(d0 + td) + s0 + ts) / PN);
      }
#pragma unroll
      for (int t = 0; t < GROUP; ++t) {
        const int v = tid + (t0 + t) * PERM_THREADS, td = v / VPR, ts = (v % VPR) * PN;
        if (d0 + td < n_d && s0 + ts < n_s) {
#pragma unroll
          for (int e = 0; e < PN; ++e) tile[ts + e][td] = p[t].v[e];
        }
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
#pragma unroll
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

// r16 tiles with 16-byte accesses on both sides: two neighbouring output-innermost rows (d, d + 1) travel through
// shared memory as one 32-bit word per source column, which halves the shared-memory instructions of the
// 2-byte version and removes its sub-word bank conflicts.  Rows of TILE / 2 words, the column XOR-ed with twice the
// row's 8-row group (bits 1-4): the 32 words of a warp's store (16 row groups x 2 columns) fall into 32 banks, and a
// 16-byte chunk stays whole and aligned (at most its halves swap), so the second pass reads it with one 128-bit load.
template <bool BLEND>
__global__ void __launch_bounds__(PERM_THREADS, 5) permute_tiles_h2_kernel(const __half* __restrict__ src, __half* dst, float alpha,
                                                                        const PermDims batch, size_t n_s, size_t n_d, size_t s_pitch,
                                                                        size_t d_pitch, unsigned tiles_s, unsigned tiles_d,
                                                                        const PermSplit sp) {
  constexpr int TILE = 128, PN = 8, VPR = TILE / PN;
  __shared__ __align__(16) uint32_t tile[TILE][TILE / 2];   // tile[s][(d / 2) ^ swz(s)] = (value at d, value at d + 1)
  size_t s0, d0, sbase, dbase;
  decode_tile(batch, tiles_s, tiles_d, TILE, s0, d0, sbase, dbase);
  auto src_row = [&](size_t id) -> size_t {
    if (sp.d_lo == 0) return id * s_pitch;
    const unsigned hi = static_cast<unsigned>(id) / sp.d_lo;
    return static_cast<size_t>(static_cast<unsigned>(id) - hi * sp.d_lo) * s_pitch + hi * sp.s_pitch_hi;
  };
  auto dst_row = [&](size_t is) -> size_t {
    if (sp.s_lo == 0) return is * d_pitch;
    const unsigned hi = static_cast<unsigned>(is) / sp.s_lo;
    return static_cast<size_t>(static_cast<unsigned>(is) - hi * sp.s_lo) * d_pitch + hi * sp.d_pitch_hi;
  };
  const int tid = threadIdx.x;
  // a warp covers two row pairs x 16 packs: whole 256-byte source rows.  Two stages: all 8 loads of a thread are in
  // flight before the first value is used (written as one loop, each trip waited for its own two loads)
  constexpr int TRIPS = (TILE / 2) * VPR / PERM_THREADS;   // 4
  uint4 lo[TRIPS], hi[TRIPS];
#pragma unroll
  for (int t = 0; t < TRIPS; ++t) {
    const int v = tid + t * PERM_THREADS;
    const int td = (v >> 4) * 2, ts = (v & 15) * PN;
    if (d0 + td < n_d && s0 + ts < n_s) {   // n_d and n_s are multiples of 8: the pair and the pack are whole
      lo[t] = __ldcs(reinterpret_cast<const uint4*>(src + sbase + src_row(d0 + td) + s0 + ts));
      hi[t] = __ldcs(reinterpret_cast<const uint4*>(src + sbase + src_row(d0 + td + 1) + s0 + ts));
    }
  }
#pragma unroll
  for (int t = 0; t < TRIPS; ++t) {
    const int v = tid + t * PERM_THREADS;
    const int td = (v >> 4) * 2, ts = (v & 15) * PN;
    if (d0 + td < n_d && s0 + ts < n_s) {
      const uint32_t a[4] = {lo[t].x, lo[t].y, lo[t].z, lo[t].w}, b[4] = {hi[t].x, hi[t].y, hi[t].z, hi[t].w};
      const int col = (td >> 1) ^ (((ts >> 3) & 15) << 1);   // rows ts .. ts + 7 share these bits
#pragma unroll
      for (int e = 0; e < 4; ++e) {   // (a.lo, b.lo) and (a.hi, b.hi) of each word pair: one byte permute each
        tile[ts + 2 * e][col] = __byte_perm(a[e], b[e], 0x5410);
        tile[ts + 2 * e + 1][col] = __byte_perm(a[e], b[e], 0x7632);
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int v = tid; v < TILE * VPR; v += PERM_THREADS) {
    const int ts = v / VPR, td = (v % VPR) * PN;
    if (s0 + ts < n_s && d0 + td < n_d) {
      __half* out = dst + dbase + dst_row(s0 + ts) + d0 + td;
      union { uint4 u; uint32_t w[4]; __half2 h2[4]; } p;
      const int key = ((ts >> 3) & 15) << 1;             // bits 2-4 move the 16-byte chunk, bit 1 swaps its halves
      const uint4 raw = *reinterpret_cast<const uint4*>(&tile[ts][((td >> 1) ^ key) & ~3]);
      p.u = (key & 2) ? make_uint4(raw.z, raw.w, raw.x, raw.y) : raw;
      if constexpr (BLEND) {
        union { uint4 u; __half2 h2[4]; } old;
        old.u = *reinterpret_cast<const uint4*>(out);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __half22float2(p.h2[e]), y = __half22float2(old.h2[e]);
          p.h2[e] = __floats2half2_rn(x.x + alpha * y.x, x.y + alpha * y.y);
        }
      }
      *reinterpret_cast<uint4*>(out) = p.u;
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
    const size_t threads = ((pieces + 31) / 32) * 32;    // a warp takes 32 pieces per trip
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
  if constexpr (std::is_same<T, __half>::value) {
    if (vl && vs) {
      if (alpha == 0.0) permute_tiles_h2_kernel<false><<<grid, PERM_THREADS, 0, st>>>(src, dst, 0.f, b, n_s, n_d, s_pitch, d_pitch, ts, td, sp);
      else permute_tiles_h2_kernel<true><<<grid, PERM_THREADS, 0, st>>>(src, dst, static_cast<float>(alpha), b, n_s, n_d, s_pitch, d_pitch, ts, td, sp);
      MP_LAUNCH_CHECK();
      return;
    }
  }
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
