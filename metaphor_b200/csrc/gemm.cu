// Contractions C[M,N] = alpha * op(A) * op(B) (+ bias) + beta * C, row-major.
//
//   launch_inner_product_ij_jk_ik : A[M,K]      B[K,N]       (reference: cuBLAS via
//                                                             inner_product_ij_jk_ik.cu:3-27)
//   launch_inner_product_ij_kj_ik : A[M,K]      B[N,K]^T     (reference: transpose to
//   launch_inner_product_ji_jk_ik : A[K,M]^T    B[K,N]        scratch + the call above)
//   launch_linear_ij_jk_ik        : A[M,K]      B[K,N] + bias[N]
//   launch_linear_ij_jk_ik_ik     : A[M,K]      B[K,N] + R[M,N]
//
// r16 and r32 run on the tcgen05 tensor cores: operand tiles are brought into
// 128-byte-swizzled shared memory by TMA (one warp's elected thread), a single
// thread issues tcgen05.mma with the fp32 accumulator tile in TMEM, and four
// epilogue warps read the accumulator back with tcgen05.ld and apply alpha,
// beta, bias on the way to global memory.  The kernel is persistent (one CTA per
// SM walking the output tiles) with two TMEM accumulators, so one tile's
// epilogue overlaps the next tile's main loop.  Transposed operands need no scratch
// copy: the shared-memory descriptor and the instruction descriptor carry the
// operand's major-ness.  r32 uses kind::tf32 on an error-compensated split
// (hi + lo, three MMAs) unless MP_GEMM_TF32X1 is set; r64 and shapes TMA cannot
// address (row pitch not a multiple of 16 bytes) use an FP-pipe tile kernel.
#include "mp_tcgen05.cuh"

#include <cuda.h>
#include <mutex>

namespace {

// ---------------------------------------------------------------------------
// SIMT tile kernel: any dtype, any shape.  64x64 output tile, 16-deep k-slices
// through shared memory, 4x4 outputs per thread, accumulation in Acc<T>.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                        const T* __restrict__ bias, typename Acc<T>::type alpha, T* c,
                                                        typename Acc<T>::type beta, size_t M, size_t N, size_t K, int a_mn,
                                                        int b_mn, size_t bias_pitch = 0) {
  using A = typename Acc<T>::type;
  constexpr int TS = 64, KS = 16;
  a += static_cast<size_t>(blockIdx.z) * M * K;   // batch entries are densely packed
  b += static_cast<size_t>(blockIdx.z) * K * N;
  c += static_cast<size_t>(blockIdx.z) * M * N;
  __shared__ A sa[KS][TS + 1];
  __shared__ A sb[KS][TS + 1];
  const size_t m0 = static_cast<size_t>(blockIdx.y) * TS, n0 = static_cast<size_t>(blockIdx.x) * TS;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  A acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = A(0);
  for (size_t k0 = 0; k0 < K; k0 += KS) {
    for (int idx = threadIdx.x; idx < TS * KS; idx += 256) {
      // A element (m, k): a_mn ? a[k*M + m] : a[m*K + k]
      int kk, mm;
      if (a_mn) { mm = idx % TS; kk = idx / TS; } else { kk = idx % KS; mm = idx / KS; }
      const size_t gm = m0 + mm, gk = k0 + kk;
      sa[kk][mm] = (gm < M && gk < K) ? mp_up(a_mn ? a[gk * M + gm] : a[gm * K + gk]) : A(0);
      int kb, nb;
      if (b_mn) { nb = idx % TS; kb = idx / TS; } else { kb = idx % KS; nb = idx / KS; }
      const size_t gn = n0 + nb, gkb = k0 + kb;
      sb[kb][nb] = (gn < N && gkb < K) ? mp_up(b_mn ? b[gkb * N + gn] : b[gn * K + gkb]) : A(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      A av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      A r = alpha * acc[i][j];
      if (bias != nullptr) r += mp_up(bias[gm * bias_pitch + gn]);
      if (beta != A(0)) r += beta * mp_up(c[gm * N + gn]);
      c[gm * N + gn] = mp_down<T>(r);
    }
  }
}

// ---------------------------------------------------------------------------
// tcgen05 kernel.
// ---------------------------------------------------------------------------
constexpr int BM = 128;               // UMMA M (one TMEM lane per output row)
constexpr int SWIZZLE_BYTES = 128;    // one operand row / k-row in shared memory
constexpr int GEMM_THREADS = 320;     // warp 0: TMA, warp 1: MMA + TMEM, warps 2-9: epilogue
constexpr int GEMM_MAX_THREADS = 448; // + warps 10-13: operand split (r32)
constexpr int EPI_THREADS = 256;      // two epilogue warps per TMEM lane quarter, each takes half of the columns
constexpr int MAX_STAGES = 8;

// Staging blocks per epilogue warp.  r16: one per 32-column block of the warp's half tile (4 at BN = 256), so
// a tile's TMA stores are issued back to back and the staging is only waited for at the next tile.
template <typename T> struct EpiBufs { static constexpr int value = sizeof(T) == 2 ? 4 : 1; };

template <typename T> struct GemmT;
template <> struct GemmT<__half> {
  static constexpr int BK = 64;       // elements per 128-byte row
  static constexpr int UMMA_K = 16;
  static constexpr bool TF32 = false;
  static constexpr uint32_t FMT = UMMA_FMT_F16;
};
template <> struct GemmT<float> {
  static constexpr int BK = 32;
  static constexpr int UMMA_K = 8;
  static constexpr bool TF32 = true;
  static constexpr uint32_t FMT = UMMA_FMT_TF32;
};

struct GemmArgs {
  const void* bias;   // N values of T (bias_pitch = 0), a full [M, N] matrix (bias_pitch = N), or nullptr
  size_t bias_pitch = 0;
  void* c;            // [M, N] row-major
  float alpha, beta;
  int M, N, K;
  int a_mn, b_mn;     // operand major-ness: 0 = K contiguous, 1 = M resp. N contiguous
  int stages;
  int epi_boxes = 2;  // pair kernel: 64-column staging boxes per epilogue warp
  int split;          // r32 only: 1 = error-compensated hi/lo split (3 MMAs per k-slice)
  int ksplit;         // > 1: the K range of every tile is cut into ksplit work units whose raw fp32
  float* partial;     //      accumulators go to partial[unit_split][M][N]; a fold kernel finishes C
  int batch;          // > 1: densely packed [batch, M, K] x [batch, K, N] -> [batch, M, N] over 3-D tensor maps (ksplit = 1)
  uint32_t* status;
};

// Shared memory of one stage: A tile (BM x 128 B), B tile (BN x 128 B), and for
// the split mode the "lo" copies of both.
template <int BN> constexpr int stage_bytes(bool split) {
  return (BM * SWIZZLE_BYTES + BN * SWIZZLE_BYTES) * (split ? 2 : 1);
}

// Persistent kernel: grid = min(tiles, SMs); every CTA walks output tiles
// t = blockIdx.x, blockIdx.x + gridDim.x, ... (consecutive tiles share the B
// tile, which therefore stays in L2).  The shared-memory ring runs across tile
// boundaries and there are two TMEM accumulators, so the epilogue of tile i
// (tcgen05.ld -> registers -> global) overlaps the main loop of tile i+1.
//   warp 0      TMA producer (one elected thread)
//   warp 1      MMA issuer (one elected thread), owns the TMEM allocation
//   warps 2-9   epilogue: warp w reads TMEM lane quarter w % 4 and one half of the tile's columns;
//               32x32 blocks go registers -> shared staging -> TMA store (coalesced, edge-clipped)
//   warps 10-13 r32 split mode only: write the hi / lo operand tiles
template <typename T, int BN>
__global__ void __launch_bounds__(GEMM_MAX_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                          const __grid_constant__ CUtensorMap tmap_b,
                                                                          const __grid_constant__ CUtensorMap tmap_c,
                                                                          const GemmArgs g) {
  using G = GemmT<T>;
  constexpr int BK = G::BK;
  constexpr int A_BYTES = BM * SWIZZLE_BYTES, B_BYTES = BN * SWIZZLE_BYTES;
  constexpr int KSLICES = BK / G::UMMA_K;  // 4
  constexpr int ACC_BUFS = 2;
  constexpr int EPI_TILE_BYTES = 32 * 32 * sizeof(T);   // one 32 x 32 staging block for the TMA store
  constexpr int EPI_BUFS = EpiBufs<T>::value;           // staging blocks per warp: no wait between the blocks of a tile
  // r16, BN >= 128: two 32-column blocks share one [32 rows][64 columns] staging box in the 128-byte swizzle,
  // written out by one TMA store with full 128-byte rows (64-byte rows halve the store engine's throughput)
  constexpr bool WIDE_STORE = sizeof(T) == 2 && BN >= 128;
  extern __shared__ unsigned char gemm_smem_raw[];
  // 1024-byte alignment: swizzle atoms are 8 rows x 128 bytes
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = g.stages;
  const int stage_sz = (A_BYTES + B_BYTES) * (g.split ? 2 : 1);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(stages) * stage_sz);
  uint64_t* ready = full + MAX_STAGES;      // split mode: hi / lo tiles written
  uint64_t* empty = ready + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;  // [2] accumulator complete
  uint64_t* acc_empty = acc_full + ACC_BUFS;  // [2] accumulator drained by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned char* epi_stage = smem + static_cast<size_t>(stages) * stage_sz + 1024;   // 8 warps x EPI_BUFS x EPI_TILE_BYTES, 1024-aligned

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (g.K + BK - 1) / BK;
  const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  // work unit u = (tile u % num_tiles, K split u / num_tiles) covering k-blocks [kb0, kb1)
  // batched: unit = batch entry * num_tiles + tile (ksplit is 1)
  const int num_units = num_tiles * g.ksplit * g.batch;
  const int kb_per = (num_kb + g.ksplit - 1) / g.ksplit;
  const bool batched = g.batch > 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(ready + s, 128);
      mbar_init(empty + s, 1);
    }
    for (int a = 0; a < ACC_BUFS; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, EPI_THREADS); }
    *abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) tmem_alloc(tmem_slot, ACC_BUFS * BN);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        const int bz = batched ? unit / num_tiles : 0;
        const int tile = batched ? unit - bz * num_tiles : unit % num_tiles, sp = batched ? 0 : unit / num_tiles;
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        const int kb0 = sp * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_abortable(empty + s, phase ^ 1u, g.status, abort)) { ok = false; break; }
          unsigned char* sa = smem + static_cast<size_t>(s) * stage_sz;
          unsigned char* sb = sa + A_BYTES;
          mbar_arrive_expect_tx(full + s, A_BYTES + B_BYTES);
          const int k0 = kb * BK;
          if (batched) {   // the same boxes over 3-D maps
            if (!g.a_mn) {
              tma_load_3d(sa, &tmap_a, k0, m0, bz, full + s);
            } else {
#pragma unroll 1
              for (int j = 0; j < BM / BK; ++j) tma_load_3d(sa + j * (BK * SWIZZLE_BYTES), &tmap_a, m0 + j * BK, k0, bz, full + s);
            }
            if (!g.b_mn) {
              tma_load_3d(sb, &tmap_b, k0, n0, bz, full + s);
            } else {
#pragma unroll 1
              for (int j = 0; j < BN / BK; ++j) tma_load_3d(sb + j * (BK * SWIZZLE_BYTES), &tmap_b, n0 + j * BK, k0, bz, full + s);
            }
          } else {
            if (!g.a_mn) {
              tma_load_2d(sa, &tmap_a, k0, m0, full + s);            // box {BK, BM}
            } else {
#pragma unroll 1
              for (int j = 0; j < BM / BK; ++j)                        // boxes {BK along M, BK k-rows}
                tma_load_2d(sa + j * (BK * SWIZZLE_BYTES), &tmap_a, m0 + j * BK, k0, full + s);
            }
            if (!g.b_mn) {
              tma_load_2d(sb, &tmap_b, k0, n0, full + s);            // box {BK, BN}
            } else {
#pragma unroll 1
              for (int j = 0; j < BN / BK; ++j)
                tma_load_2d(sb + j * (BK * SWIZZLE_BYTES), &tmap_b, n0 + j * BK, k0, full + s);
            }
          }
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_instr_desc(G::FMT, g.a_mn, g.b_mn, BM, BN);
      // K-major: rows of 128 B, 8-row groups 1024 B apart, k-slice = +32 B.
      // MN-major: k-rows of 128 B, 64/32-column blocks BK*128 B apart, k-slice = +UMMA_K*128 B.
      const uint32_t a_lbo = g.a_mn ? BK * SWIZZLE_BYTES : 16, b_lbo = g.b_mn ? BK * SWIZZLE_BYTES : 16;
      const uint32_t a_kstep = g.a_mn ? G::UMMA_K * SWIZZLE_BYTES : 32, b_kstep = g.b_mn ? G::UMMA_K * SWIZZLE_BYTES : 32;
      // 32-bit MN-major tiles use the 32-byte-atom swizzle (groups of 4 k-rows, 512 B)
      const uint32_t a_lay = (G::TF32 && g.a_mn) ? UMMA_LAYOUT_SW128_BASE32B : UMMA_LAYOUT_SW128;
      const uint32_t b_lay = (G::TF32 && g.b_mn) ? UMMA_LAYOUT_SW128_BASE32B : UMMA_LAYOUT_SW128;
      const uint32_t a_sbo = (G::TF32 && g.a_mn) ? 512 : 1024, b_sbo = (G::TF32 && g.b_mn) ? 512 : 1024;
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        // the epilogue must have drained this accumulator (passes at once on its first use)
        if (!mbar_wait_abortable(acc_empty + buf, (use & 1u) ^ 1u, g.status, abort)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        const int sp = batched ? 0 : unit / num_tiles;
        const int kb0 = sp * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          uint64_t* wait_on = g.split ? (ready + s) : (full + s);
          if (!mbar_wait_abortable(wait_on, phase, g.status, abort)) { ok = false; break; }
          tcgen05_fence_after_sync();
          const uint32_t sa = mp_smem_u32(smem + static_cast<size_t>(s) * stage_sz);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t sa_lo = sb + B_BYTES, sb_lo = sa_lo + A_BYTES;
#pragma unroll
          for (int ks = 0; ks < KSLICES; ++ks) {
            const uint64_t ad = umma_smem_desc(sa + ks * a_kstep, a_lbo, a_sbo, a_lay);
            const uint64_t bd = umma_smem_desc(sb + ks * b_kstep, b_lbo, b_sbo, b_lay);
            umma<G::TF32>(tmem_acc, ad, bd, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
            if (g.split) {
              const uint64_t adl = umma_smem_desc(sa_lo + ks * a_kstep, a_lbo, a_sbo, a_lay);
              const uint64_t bdl = umma_smem_desc(sb_lo + ks * b_kstep, b_lbo, b_sbo, b_lay);
              umma<G::TF32>(tmem_acc, ad, bdl, idesc, 1u);   // hi * lo
              umma<G::TF32>(tmem_acc, adl, bd, idesc, 1u);   // lo * hi
            }
          }
          umma_commit(empty + s);  // the stage may be refilled once these MMAs have read it
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(acc_full + buf);
      }
    }
  } else if (warp >= 10) {
    // ---------------- r32 split mode: hi / lo operand tiles --------------------
    // hi = x with the 13 low mantissa bits cleared (exactly representable in
    // tf32, so the tensor core's own fp32 -> tf32 conversion cannot change it),
    // lo = x - hi (exact in fp32; its tf32 conversion error is ~2^-21 |x|).
    const int et = threadIdx.x - 320;  // 0..127
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
      const int sp = batched ? 0 : unit / num_tiles;
      const int kb0 = sp * kb_per, kb1 = min(num_kb, kb0 + kb_per);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_abortable(full + s, phase, g.status, abort)) { ok = false; break; }
        unsigned char* hi = smem + static_cast<size_t>(s) * stage_sz;
        unsigned char* lo = hi + A_BYTES + B_BYTES;
        for (int off = et * 16; off < A_BYTES + B_BYTES; off += 128 * 16) {
          const uint4 v = *reinterpret_cast<const uint4*>(hi + off);
          uint4 h, r;
          h.x = v.x & 0xFFFFE000u; h.y = v.y & 0xFFFFE000u; h.z = v.z & 0xFFFFE000u; h.w = v.w & 0xFFFFE000u;
          r.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x));
          r.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y));
          r.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z));
          r.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w));
          *reinterpret_cast<uint4*>(hi + off) = h;
          *reinterpret_cast<uint4*>(lo + off) = r;
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
        mbar_arrive(ready + s);
        if (++s == stages) { s = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------ epilogue -----------------------------------
    const int quarter = warp & 3;                 // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;             // which half of the tile's columns
    const T* bias = static_cast<const T*>(g.bias);
    const bool vec_ok = (static_cast<size_t>(g.N) * sizeof(T)) % 16 == 0 && mp_aligned16(g.c);
    const bool use_tma = vec_ok && g.beta == 0.0f && g.ksplit == 1;   // overwrite: stage 32x32 blocks and let TMA write them
    unsigned char* stage_base = epi_stage + (warp - 2) * (EPI_BUFS * EPI_TILE_BYTES);
    int local = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++local) {
      const int bz = batched ? unit / num_tiles : 0;
      const int tile = batched ? unit - bz * num_tiles : unit % num_tiles, sp = batched ? 0 : unit / num_tiles;
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      const bool acc_ready = mbar_wait_abortable(acc_full + buf, use & 1u, g.status, abort);
      __syncwarp();  // tcgen05.ld is warp-collective
      if (!acc_ready) break;
      tcgen05_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + buf * BN;
      const int row = m0 + quarter * 32 + lane;
      T* crow = static_cast<T*>(g.c) + (static_cast<size_t>(bz) * g.M + row) * g.N;
      int blk = 0;
#pragma unroll 1
      for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32, ++blk) {
        const int col0 = n0 + c0;
        if (col0 >= g.N) break;   // uniform across the warp
        unsigned char* stage = stage_base + (blk % EPI_BUFS) * EPI_TILE_BYTES;
        uint32_t v[32];
        tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
        tmem_ld_wait();
        if (g.ksplit > 1) {   // raw partial sums; alpha, bias and beta are applied by the fold
          if (row < g.M) {
            float* prow = g.partial + (static_cast<size_t>(sp) * g.M + row) * g.N + col0;
            if ((g.N & 3) == 0 && col0 + 32 <= g.N) {
#pragma unroll
              for (int p = 0; p < 8; ++p) *reinterpret_cast<uint4*>(prow + p * 4) = make_uint4(v[p * 4], v[p * 4 + 1], v[p * 4 + 2], v[p * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < g.N) prow[j] = __uint_as_float(v[j]);
            }
          }
          continue;
        }
        float r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = g.alpha * __uint_as_float(v[j]);
        if (bias != nullptr && (g.bias_pitch == 0 || row < g.M)) {
          const T* brow = bias + static_cast<size_t>(row) * g.bias_pitch;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < g.N) r[j] += mp_up(brow[col0 + j]);
        }
        if (use_tma) {
          constexpr int PN = Pack<T>::N;
          if constexpr (WIDE_STORE) {
            if (blk == 0) {   // the previous tile's stores have finished reading the staging boxes
              if (lane == 0) bulk_wait_read<0>();
              __syncwarp();
            }
            const int in_box = blk & 1;
            unsigned char* box = stage_base + (blk >> 1) * (2 * EPI_TILE_BYTES);
#pragma unroll
            for (int p = 0; p < 4; ++p)   // 16-byte chunk (4 in_box + p) of this lane's 128-byte row, XOR-swizzled
              *reinterpret_cast<Pack<T>*>(box + lane * 128 + (((4 * in_box + p) ^ (lane & 7)) << 4)) = pack<T>(r + p * PN);
            if (in_box == 1 || col0 + 32 >= g.N) {   // box complete (columns past N are clipped by the store)
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                if (batched) tma_store_3d(&tmap_c, box, col0 - 32 * in_box, m0 + quarter * 32, bz);
                else tma_store_2d(&tmap_c, box, col0 - 32 * in_box, m0 + quarter * 32);
                bulk_commit();
              }
            }
            continue;
          }
          // the store that last used this staging block has finished reading it
          if (lane == 0) { if (EPI_BUFS == 1 || blk < EPI_BUFS) { if (EPI_BUFS == 1 || blk == 0) bulk_wait_read<0>(); } else bulk_wait_read<EPI_BUFS - 1>(); }
          __syncwarp();
          // r32: 128-byte rows in the 128-byte swizzle (conflict-free); r16 at BN = 64: linear 64-byte rows.
          // Register indices stay compile-time constants (a lane-dependent slot order would push r[] to local memory).
          unsigned char* srow = stage + lane * (32 * sizeof(T));
#pragma unroll
          for (int p = 0; p < 32 / PN; ++p) {
            const int slot = sizeof(T) == 4 ? (p ^ (lane & 7)) : p;
            *reinterpret_cast<Pack<T>*>(srow + slot * 16) = pack<T>(r + p * PN);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (batched) tma_store_3d(&tmap_c, stage, col0, m0 + quarter * 32, bz);
            else tma_store_2d(&tmap_c, stage, col0, m0 + quarter * 32);
            bulk_commit();
          }
        } else if (row < g.M) {
          if (vec_ok && col0 + 32 <= g.N) {
            constexpr int PN = Pack<T>::N;
            if (g.beta != 0.0f) {
#pragma unroll
              for (int p = 0; p < 32 / PN; ++p) {
                float old[PN];
                unpack<T>(ld_pack(crow + col0, p), old);
#pragma unroll
                for (int e = 0; e < PN; ++e) r[p * PN + e] += g.beta * old[e];
              }
            }
#pragma unroll
            for (int p = 0; p < 32 / PN; ++p) st_pack(crow + col0, p, pack<T>(r + p * PN));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < g.N) {
                float o = r[j];
                if (g.beta != 0.0f) o += g.beta * mp_up(crow[col0 + j]);
                crow[col0 + j] = mp_down<T>(o);
              }
            }
          }
        }
      }
      // hand the accumulator back to the MMA warp
      tcgen05_fence_before_sync();
      mbar_arrive(acc_empty + buf);
    }
    if (use_tma && lane == 0) bulk_wait_all<0>();   // all of this warp's stores have completed
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, ACC_BUFS * BN);
}


// ---------------------------------------------------------------------------
// CTA-pair kernel (r16): a cluster of two CTAs owns a 256 x 256 output tile.  Rank r loads its 128 rows of
// A and columns [128 r, 128 r + 128) of B, so every CTA moves 32 KB per 64-deep k-block for a 128 x 256
// accumulator instead of 48 KB: the single-CTA kernel is bound by the L2 -> shared-memory feed, not by the
// tensor pipe (measured 1.25-1.7 k cycles per k-block against 0.5 k at the tensor peak).
//   both ranks  warp 0: TMA producer; warps 2-9: epilogue of the rank's own 128 rows
//   rank 0      warp 1: issues the pair MMAs, commits to its own barriers
// Barriers live at the same offsets in both CTAs.  full[s]: rank 0 only, credited by both ranks' loads.
// empty[s] / acc_full[b]: the MMA commit arrives on both CTAs' barriers (tcgen05.commit to a CTA mask).
// acc_empty[b]: rank 0 only, one arrival per epilogue warp of both ranks.  Every wait is bounded and suspends between
// polls: polling the ring barriers without a suspend hint (as the scan's chunk walk does) made every shape 5 - 8 % slower.
// ---------------------------------------------------------------------------
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGE_BYTES = BM * SWIZZLE_BYTES + (PAIR_BN / 2) * SWIZZLE_BYTES;   // 32 KB

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             const __grid_constant__ CUtensorMap tmap_c, const GemmArgs g) {
  using T = __half;
  using G = GemmT<T>;
  constexpr int BK = G::BK, BN = PAIR_BN;
  constexpr int A_BYTES = BM * SWIZZLE_BYTES, B_BYTES = (BN / 2) * SWIZZLE_BYTES;
  constexpr int KSLICES = BK / G::UMMA_K;
  constexpr int ACC_BUFS = 2;
  constexpr int BOX_BYTES = 32 * 64 * sizeof(T);   // one [32 rows][64 columns] staging box
  extern __shared__ unsigned char gemm_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = g.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(stages) * PAIR_STAGE_BYTES);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;
  uint64_t* acc_empty = acc_full + ACC_BUFS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned char* epi_stage = smem + static_cast<size_t>(stages) * PAIR_STAGE_BYTES + 1024;   // 8 warps x 1 or 2 boxes
  const int epi_boxes = g.epi_boxes;   // 1: a deeper operand ring; every box then waits for the previous store's read

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_kb = (g.K + BK - 1) / BK;
  const int tiles_m = (g.M + 2 * BM - 1) / (2 * BM), tiles_n = (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  // work unit u = (tile u % num_tiles, K split u / num_tiles) covering k-blocks [kb0, kb1)
  const int num_units = num_tiles * g.ksplit;
  const int kb_per = (num_kb + g.ksplit - 1) / g.ksplit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < ACC_BUFS; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 16); }
    *abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, ACC_BUFS * BN);
  tcgen05_fence_before_sync();
  cluster_sync_all();   // both CTAs' barriers and TMEM exist before anything crosses the pair
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both ranks) ------------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      long it = 0;
      bool ok = true;
      for (int unit = pair; unit < num_units && ok; unit += num_pairs) {
        const int tile = unit % num_tiles, sp = unit / num_tiles;
        const int m0 = (tile % tiles_m) * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = (tile / tiles_m) * BN + static_cast<int>(rank) * (BN / 2);
        const int kb0 = sp * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (!mbar_wait_abortable(empty + s, phase ^ 1u, g.status, abort)) { ok = false; break; }
          if (rank == 0) mbar_arrive_expect_tx(full + s, 2 * (A_BYTES + B_BYTES));
          unsigned char* sa = smem + static_cast<size_t>(s) * PAIR_STAGE_BYTES;
          unsigned char* sb = sa + A_BYTES;
          const int k0 = kb * BK;
          if (!g.a_mn) {
            tma_load_2d_pair(sa, &tmap_a, k0, m0, full + s);
          } else {
#pragma unroll 1
            for (int j = 0; j < BM / BK; ++j) tma_load_2d_pair(sa + j * (BK * SWIZZLE_BYTES), &tmap_a, m0 + j * BK, k0, full + s);
          }
          if (!g.b_mn) {
            tma_load_2d_pair(sb, &tmap_b, k0, n0, full + s);
          } else {
#pragma unroll 1
            for (int j = 0; j < (BN / 2) / BK; ++j) tma_load_2d_pair(sb + j * (BK * SWIZZLE_BYTES), &tmap_b, n0 + j * BK, k0, full + s);
          }
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (rank 0) -------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_instr_desc(G::FMT, g.a_mn, g.b_mn, 2 * BM, BN);
      const uint32_t a_lbo = g.a_mn ? BK * SWIZZLE_BYTES : 16, b_lbo = g.b_mn ? BK * SWIZZLE_BYTES : 16;
      const uint32_t a_kstep = g.a_mn ? G::UMMA_K * SWIZZLE_BYTES : 32, b_kstep = g.b_mn ? G::UMMA_K * SWIZZLE_BYTES : 32;
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int unit = pair; unit < num_units && ok; unit += num_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!mbar_wait_abortable(acc_empty + buf, (use & 1u) ^ 1u, g.status, abort)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        const int sp = unit / num_tiles;
        const int kb0 = sp * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_abortable(full + s, phase, g.status, abort)) { ok = false; break; }
          tcgen05_fence_after_sync();
          const uint32_t sa = mp_smem_u32(smem + static_cast<size_t>(s) * PAIR_STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int ks = 0; ks < KSLICES; ++ks) {
            const uint64_t ad = umma_smem_desc(sa + ks * a_kstep, a_lbo, 1024);
            const uint64_t bd = umma_smem_desc(sb + ks * b_kstep, b_lbo, 1024);
            umma_pair_f16(tmem_acc, ad, bd, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
          }
          umma_commit_pair_to(empty + s, 3);   // the stage is free in both CTAs
          if (++s == stages) { s = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair_to(acc_full + buf, 3);
      }
    }
  } else {
    // ------------------------------ epilogue (both ranks) -----------------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const T* bias = static_cast<const T*>(g.bias);
    const bool vec_ok = (static_cast<size_t>(g.N) * sizeof(T)) % 16 == 0 && mp_aligned16(g.c);
    const bool use_tma = vec_ok && g.beta == 0.0f && g.ksplit == 1;
    unsigned char* stage_base = epi_stage + (warp - 2) * (epi_boxes * BOX_BYTES);
    int local = 0;
    for (int unit = pair; unit < num_units; unit += num_pairs, ++local) {
      const int tile = unit % num_tiles, sp = unit / num_tiles;
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      const int m0 = (tile % tiles_m) * 2 * BM + static_cast<int>(rank) * BM, n0 = (tile / tiles_m) * BN;
      const bool acc_ready = mbar_wait_abortable(acc_full + buf, use & 1u, g.status, abort);
      __syncwarp();
      if (!acc_ready) break;
      tcgen05_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + buf * BN;
      const int row = m0 + quarter * 32 + lane;
      T* crow = static_cast<T*>(g.c) + static_cast<size_t>(row) * g.N;
      // one staging box (64 columns) per iteration: both TMEM loads are in flight before the wait
      int boxi = 0;
#pragma unroll 1
      for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 64, ++boxi) {
        const int col0 = n0 + c0;
        if (col0 >= g.N) break;
        uint32_t v[2][32];
        tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v[0]);
        tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0 + 32, v[1]);
        tmem_ld_wait();
        if (g.ksplit > 1) {   // raw partial sums; alpha, bias and beta are applied by the fold
          if (row < g.M) {
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
              const int colb = col0 + 32 * hb;
              float* prow = g.partial + (static_cast<size_t>(sp) * g.M + row) * g.N + colb;
              if ((g.N & 3) == 0 && colb + 32 <= g.N) {
#pragma unroll
                for (int p = 0; p < 8; ++p)
                  *reinterpret_cast<uint4*>(prow + p * 4) = make_uint4(v[hb][p * 4], v[hb][p * 4 + 1], v[hb][p * 4 + 2], v[hb][p * 4 + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (colb + j < g.N) prow[j] = __uint_as_float(v[hb][j]);
              }
            }
          }
          continue;
        }
        constexpr int PN = Pack<T>::N;
        unsigned char* box = stage_base + (epi_boxes == 2 ? boxi : 0) * BOX_BYTES;
        if (use_tma && (boxi == 0 || epi_boxes == 1)) {   // the earlier stores have finished reading the staging box(es)
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
        }
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {   // (no early exit: the register arrays must stay statically indexed)
          const int colb = col0 + 32 * hb;
          if (colb < g.N) {
          float r[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = g.alpha * __uint_as_float(v[hb][j]);
          if (bias != nullptr && (g.bias_pitch == 0 || row < g.M)) {
            const T* brow = bias + static_cast<size_t>(row) * g.bias_pitch;
            if (g.bias_pitch != 0 && colb + 32 <= g.N && (g.bias_pitch * sizeof(T)) % 16 == 0 && mp_aligned16(bias)) {
              // a full-matrix term (a residual): the lane's 32 values are one contiguous 64-byte piece of its row
#pragma unroll
              for (int p = 0; p < 32 / PN; ++p) {
                float add[PN];
                unpack<T>(ld_pack(brow + colb, p), add);
#pragma unroll
                for (int e = 0; e < PN; ++e) r[p * PN + e] += add[e];
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (colb + j < g.N) r[j] += mp_up(brow[colb + j]);
            }
          }
          if (use_tma) {
#pragma unroll
            for (int p = 0; p < 4; ++p)
              *reinterpret_cast<Pack<T>*>(box + lane * 128 + (((4 * hb + p) ^ (lane & 7)) << 4)) = pack<T>(r + p * PN);
          } else if (row < g.M) {
            if (vec_ok && colb + 32 <= g.N) {
              if (g.beta != 0.0f) {
#pragma unroll
                for (int p = 0; p < 32 / PN; ++p) {
                  float old[PN];
                  unpack<T>(ld_pack(crow + colb, p), old);
#pragma unroll
                  for (int e = 0; e < PN; ++e) r[p * PN + e] += g.beta * old[e];
                }
              }
#pragma unroll
              for (int p = 0; p < 32 / PN; ++p) st_pack(crow + colb, p, pack<T>(r + p * PN));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (colb + j < g.N) {
                  float o = r[j];
                  if (g.beta != 0.0f) o += g.beta * mp_up(crow[colb + j]);
                  crow[colb + j] = mp_down<T>(o);
                }
              }
            }
          }
          }
        }
        if (use_tma) {   // columns past N are clipped by the store
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_c, box, col0, m0 + quarter * 32);
            bulk_commit();
          }
        }
      }
      // hand the accumulator back to rank 0's MMA thread: one arrival per warp of either rank
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(acc_empty + buf);
        else mbar_arrive_cluster(acc_empty + buf, 0);
      }
    }
    if (use_tma && lane == 0) bulk_wait_all<0>();
  }
  __syncwarp();         // the cluster barrier below is warp-aligned: lanes that skipped the role loops wait here
  tcgen05_fence_before_sync();
  cluster_sync_all();   // neither CTA frees TMEM or leaves while its partner may still read its memory
  if (warp == 1) tmem_dealloc_pair(tmem_base, ACC_BUFS * BN);
}

// C = alpha * sum_s partial[s] + bias + beta * C  (finishes a split-K contraction)
template <typename T>
__global__ void __launch_bounds__(256) gemm_fold_kernel(const float* __restrict__ partial, int ksplit, size_t mn, int N, float alpha,
                                                        const T* __restrict__ bias, float beta, T* __restrict__ c, size_t bias_pitch = 0) {
  const size_t i0 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 4;
  if (i0 >= mn) return;
  const bool vec = (mn & 3) == 0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int cnt = vec ? 4 : static_cast<int>(mn - i0 < 4 ? mn - i0 : 4);
  for (int sidx = 0; sidx < ksplit; ++sidx) {
    const float* p = partial + sidx * mn + i0;
    if (vec) {
      const float4 v = *reinterpret_cast<const float4*>(p);
      acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    } else {
      for (int e = 0; e < cnt; ++e) acc[e] += p[e];
    }
  }
  for (int e = 0; e < cnt; ++e) {
    float o = alpha * acc[e];
    if (bias != nullptr) o += mp_up(bias_pitch != 0 ? bias[(i0 + e) / N * bias_pitch + (i0 + e) % N] : bias[(i0 + e) % N]);
    if (beta != 0.0f) o += beta * mp_up(c[i0 + e]);
    c[i0 + e] = mp_down<T>(o);
  }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps and dispatch.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    MP_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
    if (p == nullptr || qres != cudaDriverEntryPointSuccess) MP_FATAL("cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D row-major matrix [rows, cols] of T, box = {box_cols (128 bytes), box_rows}, 128-byte swizzle
// (16-byte atoms, or 32-byte atoms when `atom32`), out-of-range elements read as zero.
// batch > 1: [batch, rows, cols] densely packed as a 3-D tensor, boxes one batch entry deep.
template <typename T>
CUtensorMap make_map(const void* base, size_t rows, size_t cols, uint32_t box_cols, uint32_t box_rows, bool atom32 = false,
                     size_t batch = 1) {
  CUtensorMap map;
  const cuuint64_t dims[3] = {cols, rows, batch};
  const cuuint64_t strides[2] = {cols * sizeof(T), rows * cols * sizeof(T)};
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  MP_CU_CHECK(encode_tiled()(&map, dt, batch > 1 ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return map;
}

// Row-major [rows, cols] output, box {32 cols, 32 rows} unswizzled, or (wide) {64 cols, 32 rows} of r16 in the
// 128-byte swizzle.
template <typename T>
CUtensorMap make_store_map(void* base, size_t rows, size_t cols, bool wide = false, size_t batch = 1) {
  CUtensorMap map;
  const cuuint64_t dims[3] = {cols, rows, batch};
  const cuuint64_t strides[2] = {cols * sizeof(T), rows * cols * sizeof(T)};
  const cuuint32_t box[3] = {wide ? 64u : 32u, 32, 1};
  const bool swizzle = wide || sizeof(T) == 4;   // 128-byte rows: r16 wide boxes and every r32 box
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  MP_CU_CHECK(encode_tiled()(&map, dt, batch > 1 ? 3 : 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return map;
}

template <typename T, int BN>
void launch_tc(const T* a, const T* b, const GemmArgs& args, int sm_count, cudaStream_t st) {
  using G = GemmT<T>;
  const int M = args.M, N = args.N, K = args.K;
  // A: K-major [M,K] box {BK, BM};  MN-major [K,M] box {BK (along M), BK (k-rows)}
  // (32-bit MN-major tiles: 128-byte swizzle with 32-byte atoms, the only MN-major layout tf32 accepts)
  const size_t nb = static_cast<size_t>(args.batch);
  const CUtensorMap ta = args.a_mn ? make_map<T>(a, K, M, G::BK, G::BK, G::TF32, nb) : make_map<T>(a, M, K, G::BK, BM, false, nb);
  const CUtensorMap tb = args.b_mn ? make_map<T>(b, K, N, G::BK, G::BK, G::TF32, nb) : make_map<T>(b, N, K, G::BK, BN, false, nb);
  // C as a TMA store target: 32 x 32 blocks, no swizzle (only used when the row pitch is a multiple of 16 bytes)
  CUtensorMap tc = ta;
  if ((static_cast<size_t>(N) * sizeof(T)) % 16 == 0 && mp_aligned16(args.c)) tc = make_store_map<T>(args.c, M, N, sizeof(T) == 2 && BN >= 128, nb);
  const size_t smem = static_cast<size_t>(args.stages) * stage_bytes<BN>(args.split != 0) + 1024 /*align*/ + 1024 /*barriers*/ +
                      8 * EpiBufs<T>::value * 32 * 32 * sizeof(T) /*epilogue staging*/;
  MP_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  const long tiles = static_cast<long>((N + BN - 1) / BN) * ((M + BM - 1) / BM) * args.ksplit * args.batch;
  const int grid = tiles < sm_count ? static_cast<int>(tiles) : sm_count;   // persistent: one CTA per SM
  gemm_tcgen05_kernel<T, BN><<<grid, args.split ? GEMM_MAX_THREADS : GEMM_THREADS, smem, st>>>(ta, tb, tc, args);
  MP_LAUNCH_CHECK();
  if (args.ksplit > 1) {
    const size_t mn = static_cast<size_t>(M) * N;
    gemm_fold_kernel<T><<<static_cast<unsigned>((mn / 4 + 256) / 256), 256, 0, st>>>(args.partial, args.ksplit, mn, N, args.alpha,
                                                                                  static_cast<const T*>(args.bias), args.beta,
                                                                                  static_cast<T*>(args.c), args.bias_pitch);
    MP_LAUNCH_CHECK();
  }
}

void launch_pair(const __half* a, const __half* b, GemmArgs args, int sm_count, cudaStream_t st) {
  using T = __half;
  using G = GemmT<T>;
  const int M = args.M, N = args.N, K = args.K;
  const CUtensorMap ta = args.a_mn ? make_map<T>(a, K, M, G::BK, G::BK) : make_map<T>(a, M, K, G::BK, BM);
  const CUtensorMap tb = args.b_mn ? make_map<T>(b, K, N, G::BK, G::BK) : make_map<T>(b, N, K, G::BK, PAIR_BN / 2);
  CUtensorMap tc = ta;
  if ((static_cast<size_t>(N) * sizeof(T)) % 16 == 0 && mp_aligned16(args.c)) tc = make_store_map<T>(args.c, M, N, true);
  // 227 KB: six 32 KB stages + one 4 KB staging box per epilogue warp, or five stages + two boxes.  The ring depth is what
  // feeds the tensor pipe: a stage is refilled only after its MMAs have completed, so (stages - 1) x 32 KB are in flight
  // per SM against an L2 latency of 2 - 3 k cycles under load (measured: the MMA thread waited for operands 35 - 40 % of
  // every tile with five stages).
  args.stages = 6;
  args.epi_boxes = 1;
  if (const char* e = getenv("MP_GEMM_PAIR_STAGES")) { if (atoi(e) == 5) { args.stages = 5; args.epi_boxes = 2; } }
  const size_t smem = static_cast<size_t>(args.stages) * PAIR_STAGE_BYTES + 1024 /*align*/ + 1024 /*barriers*/ +
                      8 * args.epi_boxes * 32 * 64 * sizeof(T);
  MP_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const int tiles = ((N + PAIR_BN - 1) / PAIR_BN) * ((M + 2 * BM - 1) / (2 * BM)) * args.ksplit;
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  gemm_tcgen05_pair_kernel<<<2 * pairs, GEMM_THREADS, smem, st>>>(ta, tb, tc, args);
  MP_LAUNCH_CHECK();
  if (args.ksplit > 1) {
    const size_t mn = static_cast<size_t>(M) * N;
    gemm_fold_kernel<T><<<static_cast<unsigned>((mn / 4 + 256) / 256), 256, 0, st>>>(args.partial, args.ksplit, mn, N, args.alpha,
                                                                                  static_cast<const T*>(args.bias), args.beta,
                                                                                  static_cast<T*>(args.c), args.bias_pitch);
    MP_LAUNCH_CHECK();
  }
}

bool env_flag(const char* name) {
  const char* e = getenv(name);
  return e != nullptr && e[0] != '\0' && e[0] != '0';
}

// Output-tile width: wide tiles for wide problems, narrower ones when they are
// needed to put at least ~one CTA on every SM.
int pick_bn(int M, int N, int sms, int batch = 1) {
  const long tiles_m = static_cast<long>((M + BM - 1) / BM) * batch;
  if (N > 128 && tiles_m * ((N + 255) / 256) >= sms) return 256;
  if (N > 64 && tiles_m * ((N + 127) / 128) >= sms / 2) return 128;
  return N > 64 && tiles_m * ((N + 127) / 128) >= 4 ? 128 : 64;
}

// Split-K: contractions with few output tiles and a long K (weight gradients: K = tokens) leave SMs
// idle or run a mostly empty last wave.  Cost model in k-block steps of one CTA:
//   waves(tiles * ks / SMs) * (k-blocks per unit + fixed cost per unit) * step time(BN)  [+ fold traffic]
// The unsplit choice of pick_bn stays unless a split is predicted to be at least 15 % faster.
void pick_split_k(GemmArgs& args, size_t elem, int sms, size_t workspace_bytes, int* bn_io) {
  const int bk = static_cast<int>(128 / elem);
  const long num_kb = (args.K + bk - 1) / bk;
  if (num_kb < 32) return;
  const double mn_bytes = static_cast<double>(args.M) * args.N * 4.0;
  auto cost = [&](int bn, int ks) {
    const long tiles = static_cast<long>((args.M + BM - 1) / BM) * ((args.N + bn - 1) / bn);
    const long waves = (tiles * ks + sms - 1) / sms;
    // one k-block step of a CTA at ~1000 TFLOP/s over all SMs (r32: half the rate, three MMAs per slice), in microseconds
    const double step_us = 2.0 * BM * bn * bk / (1000.0e6 / sms) * (args.split ? 3.0 : 1.0) * (elem == 4 ? 2.0 : 1.0);
    double t = waves * ((num_kb + ks - 1) / ks + 8.0) * step_us;
    if (ks > 1) t += 2.0 * ks * mn_bytes / 6.0e6 + 3.0;   // partial write + read at ~6 TB/s, one more launch
    return t;
  };
  const double base = cost(*bn_io, 1);
  double best = base;
  int best_bn = *bn_io, best_ks = 1;
  const int bns[2] = {128, 256};
  for (int bi = 0; bi < 2; ++bi) {
    const int bn = bns[bi];
    if (bn == 256 && args.N <= 128) continue;
    for (int ks = 2; ks <= 16; ++ks) {
      if (static_cast<double>(ks) * mn_bytes > static_cast<double>(workspace_bytes)) break;
      if (num_kb / ks < 8) break;
      if ((ks - 1) * ((num_kb + ks - 1) / ks) >= num_kb) continue;   // the last unit would be empty
      const double t = cost(bn, ks);
      if (t < best) { best = t; best_bn = bn; best_ks = ks; }
    }
  }
  if (best_ks > 1 && best < 0.85 * base) { args.ksplit = best_ks; *bn_io = best_bn; }
}

template <typename T>
void gemm_dispatch(const void* a_, const void* b_, const void* bias, double alpha, void* c_, double beta, len_t M, len_t N,
                   len_t K, int a_mn, int b_mn, StreamContext ctx, len_t batch = 1, len_t bias_pitch = 0) {
  using A = typename Acc<T>::type;
  if (M == 0 || N == 0 || batch == 0) return;
  cudaStream_t st = mp_stream(ctx);
  const T* a = static_cast<const T*>(a_);
  const T* b = static_cast<const T*>(b_);
  T* c = static_cast<T*>(c_);
  bool tensor_path = !std::is_same<T, double>::value && K > 0 && !env_flag("MP_GEMM_FORCE_SIMT");
  if (tensor_path) {
    // TMA needs 16-byte aligned bases and row pitches, and 32-bit coordinates
    const size_t a_pitch = (a_mn ? M : K) * sizeof(T), b_pitch = (b_mn ? N : K) * sizeof(T);
    tensor_path = mp_aligned16(a) && mp_aligned16(b) && a_pitch % 16 == 0 && b_pitch % 16 == 0 &&
                  M < (1ull << 31) && N < (1ull << 31) && K < (1ull << 31) && mp_state_or_null(ctx) != nullptr;
    if (batch > 1) {
      // 3-D maps: the batch pitch must keep 16-byte alignment, and the work-unit count stays in 32 bits
      const double units = static_cast<double>((M + BM - 1) / BM) * static_cast<double>((N + 63) / 64) * static_cast<double>(batch);
      tensor_path = tensor_path && (M * K * sizeof(T)) % 16 == 0 && (K * N * sizeof(T)) % 16 == 0 && units < 2.0e9;
    }
  }
  if (!tensor_path) {
    if ((M + 63) / 64 > 65535) MP_FATAL("inner_product: M too large for the FP-pipe kernel");
    for (len_t b0 = 0; b0 < batch; b0 += 65535) {   // grid.z carries the batch index
      const len_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
      const dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((M + 63) / 64), static_cast<unsigned>(nb));
      gemm_simt_kernel<T><<<grid, 256, 0, st>>>(a + b0 * M * K, b + b0 * K * N, static_cast<const T*>(bias), static_cast<A>(alpha),
                                                c + b0 * M * N, static_cast<A>(beta), M, N, K, a_mn, b_mn, bias_pitch);
      MP_LAUNCH_CHECK();
    }
    return;
  }
  if constexpr (!std::is_same<T, double>::value) {
    MpStreamState* state = mp_state(ctx);
    GemmArgs args;
    args.bias = bias;
    args.bias_pitch = bias_pitch;
    args.c = c;
    args.alpha = static_cast<float>(alpha);
    args.beta = static_cast<float>(beta);
    args.M = static_cast<int>(M);
    args.N = static_cast<int>(N);
    args.K = static_cast<int>(K);
    args.a_mn = a_mn;
    args.b_mn = b_mn;
    args.split = (std::is_same<T, float>::value && !env_flag("MP_GEMM_TF32X1")) ? 1 : 0;
    args.status = state->status_dev;
    args.batch = static_cast<int>(batch);
    int bn = pick_bn(args.M, args.N, state->sm_count, args.batch);
    args.ksplit = 1;
    args.partial = static_cast<float*>(state->workspace);
    if (batch == 1 && !env_flag("MP_GEMM_NO_SPLITK")) pick_split_k(args, sizeof(T), state->sm_count, state->workspace_bytes, &bn);
    // shared memory of the ring: 227 KB per CTA minus alignment slack, barriers and the epilogue staging (r16: 64 KB, r32: 32 KB)
    const int budget = (sizeof(T) == 2 ? 159 : 168) * 1024;
    auto stages_for = [&](int per_stage) {   // the ring runs across tiles, so depth is bounded by memory only
      int s = budget / per_stage;
      if (s > MAX_STAGES) s = MAX_STAGES;
      return s < 2 ? 2 : s;
    };
    if constexpr (std::is_same<T, __half>::value) {
      // CTA pairs for wide problems with enough 256 x 256 tiles to fill the pairs
      const long pair_tiles = static_cast<long>((args.M + 255) / 256) * ((args.N + 255) / 256);
      if (batch == 1 && !env_flag("MP_GEMM_NO_PAIRS") && args.M >= 256 && args.N >= 256) {
        if (args.ksplit == 1 && bn == 256 && pair_tiles >= state->sm_count / 2) {
          launch_pair(a, b, args, state->sm_count, st);
          return;
        }
        if (args.ksplit > 1) {
          // long K, few tiles: 256 x 256 pair tiles with the K range cut so that the units fill the pairs about evenly
          const long num_kb = (args.K + 63) / 64;
          const int pairs = state->sm_count / 2;
          int best = 0; double best_cost = 1e30;
          for (int ks = 1; ks <= 16; ++ks) {
            if (num_kb / ks < 8 || (ks - 1) * ((num_kb + ks - 1) / ks) >= num_kb) continue;
            if (static_cast<double>(ks) * args.M * args.N * 4.0 > static_cast<double>(state->workspace_bytes)) break;
            const long waves = (pair_tiles * ks + pairs - 1) / pairs;
            const double cost = waves * ((num_kb + ks - 1) / ks + 10.0) + (ks > 1 ? 2.0 * ks * args.M * args.N * 4.0 / 6.0e6 / 0.5 : 0.0);
            if (cost < best_cost) { best_cost = cost; best = ks; }
          }
          if (best >= 1) {
            args.ksplit = best;
            launch_pair(a, b, args, state->sm_count, st);
            return;
          }
        }
      }
    }
    if (bn == 256) { args.stages = stages_for(stage_bytes<256>(args.split != 0)); launch_tc<T, 256>(a, b, args, state->sm_count, st); }
    else if (bn == 128) { args.stages = stages_for(stage_bytes<128>(args.split != 0)); launch_tc<T, 128>(a, b, args, state->sm_count, st); }
    else { args.stages = stages_for(stage_bytes<64>(args.split != 0)); launch_tc<T, 64>(a, b, args, state->sm_count, st); }
  }
}

}  // namespace

template <typename T>
static void inner_product_ij_jk_ik_impl(const void* a, const void* b, double alpha, void* c, double beta, len_t m, len_t n,
                                        len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, nullptr, alpha, c, beta, m, k, n, 0, 1, ctx);  // A[m,n] K-major, B[n,k] N-contiguous
}
template <typename T>
static void inner_product_ij_kj_ik_impl(const void* a, const void* b, double alpha, void* c, double beta, len_t m, len_t n,
                                        len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, nullptr, alpha, c, beta, m, k, n, 0, 0, ctx);  // B[k,n] K-major
}
template <typename T>
static void inner_product_ji_jk_ik_impl(const void* a, const void* b, double alpha, void* c, double beta, len_t m, len_t n,
                                        len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, nullptr, alpha, c, beta, m, k, n, 1, 1, ctx);  // A[n,m] M-contiguous
}
// C = alpha * A B + R + beta * C with a full [m, k] term R (a residual stream: R may be C itself when beta = 0)
template <typename T>
static void linear_ij_jk_ik_ik_impl(const void* a, const void* b, const void* r, double alpha, void* c, double beta, len_t m, len_t n, len_t k,
                                    StreamContext ctx) {
  gemm_dispatch<T>(a, b, r, alpha, c, beta, m, k, n, 0, 1, ctx, 1, r != nullptr ? k : 0);
}

template <typename T>
static void linear_ij_jk_ik_impl(const void* a, const void* b, const void* bias, double alpha, void* c, double beta, len_t m,
                                 len_t n, len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, bias, alpha, c, beta, m, k, n, 0, 1, ctx);
}

// Batched forms ("_ij,_jk->_ik" of the reference's roadmap, NOTES.md:18): densely packed [batch, ., .] operands.
template <typename T>
static void inner_product_bij_bjk_bik_impl(const void* a, const void* b, double alpha, void* c, double beta, len_t batch, len_t m,
                                           len_t n, len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, nullptr, alpha, c, beta, m, k, n, 0, 1, ctx, batch);
}
template <typename T>
static void inner_product_bij_bkj_bik_impl(const void* a, const void* b, double alpha, void* c, double beta, len_t batch, len_t m,
                                           len_t n, len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, nullptr, alpha, c, beta, m, k, n, 0, 0, ctx, batch);
}
template <typename T>
static void inner_product_bji_bjk_bik_impl(const void* a, const void* b, double alpha, void* c, double beta, len_t batch, len_t m,
                                           len_t n, len_t k, StreamContext ctx) {
  gemm_dispatch<T>(a, b, nullptr, alpha, c, beta, m, k, n, 1, 1, ctx, batch);
}

MP_STAMP3(inner_product_bij_bjk_bik, (const void* a, const void* b, const double alpha, void* c, const double beta, len_t batch, len_t m, len_t n, len_t k, StreamContext s), (a, b, alpha, c, beta, batch, m, n, k, s))
MP_STAMP3(inner_product_bij_bkj_bik, (const void* a, const void* b, const double alpha, void* c, const double beta, len_t batch, len_t m, len_t n, len_t k, StreamContext s), (a, b, alpha, c, beta, batch, m, n, k, s))
MP_STAMP3(inner_product_bji_bjk_bik, (const void* a, const void* b, const double alpha, void* c, const double beta, len_t batch, len_t m, len_t n, len_t k, StreamContext s), (a, b, alpha, c, beta, batch, m, n, k, s))
MP_STAMP3(inner_product_ij_jk_ik, (const void* a, const void* b, const double alpha, void* c, const double beta, len_t m, len_t n, len_t k, StreamContext s), (a, b, alpha, c, beta, m, n, k, s))
MP_STAMP3(inner_product_ij_kj_ik, (const void* a, const void* b, const double alpha, void* c, const double beta, len_t m, len_t n, len_t k, StreamContext s), (a, b, alpha, c, beta, m, n, k, s))
MP_STAMP3(inner_product_ji_jk_ik, (const void* a, const void* b, const double alpha, void* c, const double beta, len_t m, len_t n, len_t k, StreamContext s), (a, b, alpha, c, beta, m, n, k, s))
MP_STAMP3(linear_ij_jk_ik_ik, (const void* a, const void* b, const void* r, const double alpha, void* c, const double beta, len_t m, len_t n, len_t k, StreamContext s), (a, b, r, alpha, c, beta, m, n, k, s))
MP_STAMP3(linear_ij_jk_ik, (const void* a, const void* b, const void* bias, const double alpha, void* c, const double beta, len_t m, len_t n, len_t k, StreamContext s), (a, b, bias, alpha, c, beta, m, n, k, s))
