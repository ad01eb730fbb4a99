// Mamba-2 SSD scan as a chunk walk: a CTA goes through a (batch, head) sequence
// 128 steps at a time and keeps the carried state on chip, so no chunk state is
// written to or scanned from global memory.  The grid is one CTA per SM slot and
// every CTA walks the same number of chunks: where a CTA's range ends inside a
// sequence, the state crosses to the next CTA once, through global memory
// (walk_segment).  The same kernel evaluates the operator in both directions,
//     out_i = r_i * sum_j mask(i,j) * decay(i,j) * c_j * <q_i, k_j> * v_j
//   causal      : j <= i, decay = exp(cum_i - cum_j), c_j = dt_j, r_i = 1       (chunks first to last)
//   anti-causal : j >= i, decay = exp(cum_j - cum_i), c_j = 1,    r_i = dt_i    (chunks last to first)
// with cum the inclusive prefix sum of dt*A inside the 128-step chunk:
//   forward pass   y  = causal(q, k, v) = (C, B, x)
//   reverse pass   gx = anti(q, k, v)   = (B, C, gy),   v_t = <gx_t, x_t>
//                  u_t = <gy_t, y_t> from a second causal walk that keeps the row dots and drops y.
// Per chunk (all on the 5th-generation tensor core, operands in 128-byte
// swizzled shared memory, fp32 accumulators in TMEM):
//   G   = q k^T                         128 x 128, K = 128   -> TMEM
//   P   = G o F  (mask, decay, c_j)     TMEM -> registers -> r16 operand tile in shared memory
//   Yd  = P v                           128 x 64,  K = 128
//   Yo  = q H                           128 x 64,  K = 128   (H = state received by the chunk, r16 copy in smem)
//   S   = k^T (w o v)                   128 x 64,  K = 128   (w_j = decay of step j to the chunk's far end)
//   out = r o (Yd + f o Yo),  H' = D H + S   (H in fp32 registers of the eight worker warps)
// Warp 0 feeds the two-stage ring by TMA, one thread of warp 1 issues the MMAs, warps 2-9
// (two warps per TMEM lane quarter, one per half of the columns) do the element-wise parts.
// The chunk length of the walk is fixed (128); the `chunk` argument of the public launcher
// only selects the evaluation order of a result that does not depend on it.
#include "mp_tcgen05.cuh"

#include <cuda.h>
#include <mutex>

namespace {

constexpr int WQ = 128;                       // steps per chunk
constexpr int WN = 128;                       // state size (columns of q and k)
constexpr int WP = 64;                        // head size (columns of v)
constexpr int W_THREADS = 320;        // warps 0-1 control (TMA, MMA), warps 2-9 workers
constexpr int W_TILE_QK = 2 * WQ * 128;       // [2 k-blocks][128 rows][128 B]
constexpr int W_TILE_V = WQ * 128;            // [128 rows][128 B]
constexpr int W_STAGE = 2 * W_TILE_QK + W_TILE_V;
constexpr int W_OFF_P = 2 * W_STAGE;
constexpr int W_OFF_H = W_OFF_P + W_TILE_QK;
constexpr int W_OFF_VS = W_OFF_H + W_TILE_V;
constexpr int W_OFF_TAIL = W_OFF_VS + W_TILE_V;   // 229376
constexpr int W_TAIL_BYTES = 2048;
constexpr int W_SMEM_BYTES = W_OFF_TAIL + W_TAIL_BYTES + 1024;   // + alignment slack = 232448 (the per-CTA maximum)
// TMEM columns
constexpr uint32_t TC_G = 0, TC_S = 128, TC_Y = 192, TC_COLS = 512;   // Yd / Yo of chunk parity p at TC_Y + p * 128 (+ 64)

enum { B_FULL0 = 0, B_FULL1, B_EMPTY0, B_EMPTY1, B_GFULL, B_PREADY, B_VSREADY, B_HREADY, B_YFULL, B_SFULL, B_SCAL, B_COUNT };

struct WalkArgs {
  int B, L, H, G, nc;
  const float* cum;        // [B, H, L] inclusive prefix sums of dt*A inside each 128-step chunk
  const float* dtt;        // [B, H, L] dt
  const float* colf;       // [B, H, L] column factor of every step relative to the far end of its 8-step piece
  __half* out;             // [B*L, H*64] or null
  const __half* z;         // dot partner, same indexing as out, or null
  float* dot_out;          // [2][B, H, L] row dots <z, out> from the fp32 accumulators, one array per half of the columns, or null
  __half* hs_out;          // [B, H, nc][128][64]: state every chunk receives, or null
  float* carry;            // [B * H][128][64] fp32: state handed from the CTA that walked the first part of a sequence to the next
  int* carry_flag;         // [B * H]: number of worker warps (of 8) that have written their part of `carry`; zero before the launch
  uint32_t* status;
};

// A CTA walks a contiguous range of the B * H * nc chunk positions (position = index in walk order, so that every CTA
// gets the same number of chunks whatever B * H is against the number of SMs).  A range is at least one sequence
// long, hence: the last part of one sequence, whole sequences, the first part of another.  The first part is walked
// FIRST and leaves its final state in `carry`; the last part is walked LAST and starts from the state the
// neighbouring CTA left there - long before, so the wait on `carry_flag` does not hold anything up (it is bounded).
struct WalkSeg { int seq, p0, n, cin, cout; };
__host__ __device__ __forceinline__ bool walk_segment(int cta, int ncta, int nseq, int nc, int idx, WalkSeg& sg) {
  const long long U = static_cast<long long>(nseq) * nc;
  const long long lo = cta * U / ncta, hi = (cta + 1) * U / ncta;
  const int s_lo = static_cast<int>(lo / nc), j_lo = static_cast<int>(lo % nc);
  const int s_hi = static_cast<int>(hi / nc), j_hi = static_cast<int>(hi % nc);
  const int first_whole = s_lo + (j_lo != 0 ? 1 : 0), n_whole = s_hi - first_whole;
  int i = idx;
  if (j_hi != 0) {
    if (i == 0) { sg.seq = s_hi; sg.p0 = 0; sg.n = j_hi; sg.cin = 0; sg.cout = 1; return true; }
    --i;
  }
  if (i < n_whole) { sg.seq = first_whole + i; sg.p0 = 0; sg.n = nc; sg.cin = 0; sg.cout = 0; return true; }
  i -= n_whole;
  if (j_lo != 0 && i == 0) { sg.seq = s_lo; sg.p0 = j_lo; sg.n = nc - j_lo; sg.cin = 1; sg.cout = 0; return true; }
  return false;
}

__device__ __forceinline__ float w_exp(float x) { return __expf(x); }

// One arrival per warp: every lane has made its shared-memory writes visible to the asynchronous proxy (and
// finished its TMEM reads) before lane 0 arrives for the warp.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  fence_proxy_async_smem();
  tcgen05_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// The hand-offs of the walk sit on its critical path: poll without a suspend hint first (a suspended warp
// wakes up hundreds of cycles after the phase completes), then fall back to the bounded, abortable wait.
__device__ __forceinline__ bool walk_wait(uint64_t* bar, uint32_t parity, uint32_t* status, volatile int* abort) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(mp_smem_u32(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return mbar_wait_abortable(bar, parity, status, abort);
}

// DOT: the row dots <z, out> are wanted (the reverse pass); a template parameter, so that the forward pass does not
// carry the registers of the dot partner's rows.
template <int ANTI, bool DOT>
__global__ void __launch_bounds__(W_THREADS, 1) ssd_walk_kernel(const __grid_constant__ CUtensorMap map_q,
                                                               const __grid_constant__ CUtensorMap map_k,
                                                               const __grid_constant__ CUtensorMap map_v,
                                                               const __grid_constant__ CUtensorMap map_hs, const WalkArgs g) {
  extern __shared__ unsigned char walk_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(walk_smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sP = smem + W_OFF_P;
  unsigned char* sH = smem + W_OFF_H;
  unsigned char* sVs = smem + W_OFF_VS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + W_OFF_TAIL);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + W_OFF_TAIL + 112);
  volatile int* abort = reinterpret_cast<volatile int*>(smem + W_OFF_TAIL + 116);
  float* s_cum = reinterpret_cast<float*>(smem + W_OFF_TAIL + 128);   // [128]
  float* s_colf = s_cum + WQ;                                         // [128]
  float* s_dt = s_colf + WQ;                                          // [128]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nc = g.nc;
  const int nseq = g.B * g.H, cta = blockIdx.x, ncta = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(bars + B_FULL0, 1); mbar_init(bars + B_FULL1, 1);
    mbar_init(bars + B_EMPTY0, 1); mbar_init(bars + B_EMPTY1, 1);
    mbar_init(bars + B_GFULL, 1); mbar_init(bars + B_YFULL, 1); mbar_init(bars + B_SFULL, 1);
    mbar_init(bars + B_PREADY, 8); mbar_init(bars + B_VSREADY, 8); mbar_init(bars + B_HREADY, 8);
    mbar_init(bars + B_SCAL, 4);
    *abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TC_COLS);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = *tmem_slot;


  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      WalkSeg sg;
      int qb = 0;   // chunks walked by this CTA before the segment in hand: the barriers' phases run on across segments
      bool ok = true;
      for (int si = 0; ok && walk_segment(cta, ncta, nseq, nc, si, sg); ++si) {
        const int h = sg.seq % g.H, b = sg.seq / g.H;
        const int grp = h / (g.H / g.G);
        for (int k = 0; k < sg.n; ++k) {
          const int q = qb + k;
          const int c = ANTI ? nc - 1 - (sg.p0 + k) : sg.p0 + k;
          const int s = q & 1;
          if (!walk_wait(bars + B_EMPTY0 + s, ((q >> 1) & 1) ^ 1u, g.status, abort)) { ok = false; break; }
          unsigned char* st = smem + s * W_STAGE;
          const int row0 = b * g.L + c * WQ;
          mbar_arrive_expect_tx(bars + B_FULL0 + s, W_STAGE);
          tma_load_2d(st, &map_q, grp * WN, row0, bars + B_FULL0 + s);
          tma_load_2d(st + WQ * 128, &map_q, grp * WN + 64, row0, bars + B_FULL0 + s);
          tma_load_2d(st + W_TILE_QK, &map_k, grp * WN, row0, bars + B_FULL0 + s);
          tma_load_2d(st + W_TILE_QK + WQ * 128, &map_k, grp * WN + 64, row0, bars + B_FULL0 + s);
          tma_load_2d(st + 2 * W_TILE_QK, &map_v, h * WP, row0, bars + B_FULL0 + s);
        }
        qb += sg.n;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // Order per chunk k: Yd(k) as soon as its P tile is written, Yo(k) as soon as the state the chunk
    // receives is in shared memory, S(k), then the scores of chunk k+1.
    if (lane == 0) {
      const uint32_t id_g = umma_instr_desc(UMMA_FMT_F16, 0u, 0u, 128, 128);   // q (K-major) x k (K-major)
      const uint32_t id_y = umma_instr_desc(UMMA_FMT_F16, 0u, 1u, 128, 64);    // K-major A x MN-major B
      const uint32_t id_s = umma_instr_desc(UMMA_FMT_F16, 1u, 1u, 128, 64);    // k^T (MN-major A) x MN-major B
      const uint32_t sp = mp_smem_u32(sP), sh = mp_smem_u32(sH), svs = mp_smem_u32(sVs);
      auto issue_g = [&](int s) {
        const uint32_t sq = mp_smem_u32(smem + s * W_STAGE), sk = sq + W_TILE_QK;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t o = (ks >> 2) * (WQ * 128) + (ks & 3) * 32;
          umma<false>(tmem + TC_G, umma_smem_desc(sq + o, 16, 1024), umma_smem_desc(sk + o, 16, 1024), id_g, ks != 0 ? 1u : 0u);
        }
        umma_commit(bars + B_GFULL);
      };
      WalkSeg sg;
      int qb = 0;          // chunks walked before this segment
      uint32_t hq = 0;     // completions of B_HREADY consumed so far (one per received state, incl. a carried-in one)
      bool ok = true;
      for (int si = 0; ok && walk_segment(cta, ncta, nseq, nc, si, sg); ++si) {
        ok = walk_wait(bars + B_FULL0 + (qb & 1), (qb >> 1) & 1, g.status, abort);
        if (ok) { tcgen05_fence_after_sync(); issue_g(qb & 1); }
        for (int k = 0; ok && k < sg.n; ++k) {
          const int q = qb + k;
          const int s = q & 1;
          const uint32_t sq = mp_smem_u32(smem + s * W_STAGE), sk = sq + W_TILE_QK, sv = sk + W_TILE_QK;
          const uint32_t ty = tmem + TC_Y + (q & 1) * 128;
          if (!walk_wait(bars + B_PREADY, q & 1, g.status, abort)) { ok = false; break; }
          tcgen05_fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t o = (ks >> 2) * (WQ * 128) + (ks & 3) * 32;
            umma<false>(ty, umma_smem_desc(sp + o, 16, 1024), umma_smem_desc(sv + ks * 2048, W_TILE_V, 1024), id_y, ks != 0 ? 1u : 0u);
          }
          const bool has_state = k > 0 || sg.cin != 0;
          if (has_state) {
            if (!walk_wait(bars + B_HREADY, hq & 1u, g.status, abort)) { ok = false; break; }
            ++hq;
            tcgen05_fence_after_sync();
            if (g.hs_out != nullptr) {   // the state this chunk receives, straight from its operand tile
              const int c = ANTI ? nc - 1 - (sg.p0 + k) : sg.p0 + k;
              tma_store_2d(&map_hs, sH, 0, static_cast<int>((static_cast<size_t>(sg.seq) * nc + c) * WN));
              bulk_commit();
            }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint32_t o = (ks >> 2) * (WQ * 128) + (ks & 3) * 32;
              umma<false>(ty + 64, umma_smem_desc(sq + o, 16, 1024), umma_smem_desc(sh + ks * 2048, W_TILE_V, 1024), id_y, ks != 0 ? 1u : 0u);
            }
          }
          umma_commit(bars + B_YFULL);
          // scores of the next chunk (its stage was released by S(k-1); the workers are past G(k))
          if (k + 1 < sg.n) {
            const int s1 = (q + 1) & 1;
            if (!walk_wait(bars + B_FULL0 + s1, ((q + 1) >> 1) & 1, g.status, abort)) { ok = false; break; }
            tcgen05_fence_after_sync();
            issue_g(s1);
          }
          if (!walk_wait(bars + B_VSREADY, q & 1, g.status, abort)) { ok = false; break; }
          tcgen05_fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma<false>(tmem + TC_S, umma_smem_desc(sk + ks * 2048, WQ * 128, 1024), umma_smem_desc(svs + ks * 2048, W_TILE_V, 1024), id_s,
                        ks != 0 ? 1u : 0u);
          // The workers rewrite the state tile once S(k) is complete: the store issued above must have read it by then.
          // (Waiting here, behind the next chunk's score MMAs, costs nothing; waiting right after the store held back
          // the commit of the output accumulators by the store's whole latency in every chunk.)
          if (g.hs_out != nullptr && has_state) bulk_wait_read<0>();
          umma_commit(bars + B_SFULL);
          umma_commit(bars + B_EMPTY0 + s);
        }
        qb += sg.n;
      }
      if (g.hs_out != nullptr) bulk_wait_all<0>();
    }
  } else {
    // ------------------------------ workers -----------------------------------
    // Software pipeline: in iteration k the warps write the P tile of chunk k+1, fold S(k) into the carried
    // state, scale the values of chunk k+1 and only then read chunk k's accumulators, so that every MMA of
    // chunk k+1 is in flight while chunk k's epilogue runs.
    const int quarter = warp & 3;              // TMEM lane quarter this warp may read
    const int ch = (warp - 2) >> 2;            // column half
    const int r = quarter * 32 + lane;         // row of every 128-row tile
    const uint32_t tl = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const int pitch = g.H * WP;
    WalkSeg sg;
    int qb = 0;          // chunks walked before this segment (barrier phases run on across segments)
    bool alive = true;
    for (int si = 0; alive && walk_segment(cta, ncta, nseq, nc, si, sg); ++si) {
    const int n = sg.n;
    const int h = sg.seq % g.H, b = sg.seq / g.H;
    const size_t bh = static_cast<size_t>(sg.seq);
    const float* cum_g = g.cum + bh * g.L;
    const float* dt_g = g.dtt + bh * g.L;
    const float* colf_g = g.colf + bh * g.L;
    float state[32];
    const int c_first = ANTI ? nc - 1 - sg.p0 : sg.p0;
    if (sg.cin) {
      // the state the first part of this sequence ended with: written by all eight worker warps of the CTA that walked it
      if (lane == 0) {
        const uint64_t t0 = mp_globaltimer_ns();
        const uint64_t limit = mp_wait_limit_ns(g.status);
        while (true) {
          int seen;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(g.carry_flag + sg.seq) : "memory");
          if (seen >= 8) break;
          if (*abort != 0) break;
          if (mp_globaltimer_ns() - t0 > limit) {
            *abort = 1;
            if (g.status != nullptr) atomicExch(g.status, MP_STATUS_WAIT_TIMEOUT);
            break;
          }
          __nanosleep(200);
        }
      }
      __syncwarp();
      if (*abort != 0) { alive = false; break; }
      const float4* src = reinterpret_cast<const float4*>(g.carry + (bh * WN + r) * WP + ch * 32);
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4) {
        const float4 v4 = __ldcg(src + q4);
        state[q4 * 4] = v4.x; state[q4 * 4 + 1] = v4.y; state[q4 * 4 + 2] = v4.z; state[q4 * 4 + 3] = v4.w;
      }
      // its r16 copy is the operand of the first chunk's q H (the tile is free: the previous segment's last readers,
      // q H and the state store, were complete before that segment's last S accumulator was released)
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 pk;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __half2 hv = __floats2half2_rn(state[q4 * 8 + 2 * e], state[q4 * 8 + 2 * e + 1]);
          ow[e] = *reinterpret_cast<const uint32_t*>(&hv);
        }
        *reinterpret_cast<uint4*>(sH + r * 128 + (((ch * 4 + q4) ^ (r & 7)) << 4)) = pk;
      }
      warp_arrive(bars + B_HREADY, lane);
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) state[e] = 0.f;
      if (g.hs_out != nullptr) {   // the first chunk of a sequence's walk receives nothing
        uint4* dst = reinterpret_cast<uint4*>(g.hs_out + ((bh * nc + c_first) * WN + r) * WP + ch * 32);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) dst[q4] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    // scalars of the walk: chunk in hand (cur), the one after it (nxt), and one more in flight (pre), so that
    // their loads are never waited for
    float cum_cur = 0.f, dt_cur = 0.f, last_cur = 0.f;
    float cum_nxt = cum_g[c_first * WQ + r], dt_nxt = dt_g[c_first * WQ + r], colf_nxt = colf_g[c_first * WQ + r];
    float last_nxt = 0.f;
    float cum_pre = 0.f, dt_pre = 0.f, colf_pre = 0.f;
    if (n > 1) {
      const int c1 = ANTI ? c_first - 1 : c_first + 1;
      cum_pre = cum_g[c1 * WQ + r]; dt_pre = dt_g[c1 * WQ + r]; colf_pre = colf_g[c1 * WQ + r];
    }

    // Iteration k finishes chunk k of the segment and prepares chunk k+1; k = -1 is the lead-in that only prepares chunk 0.
#pragma unroll 1
    for (int k = -1; k < n; ++k) {
      const bool cur = k >= 0;
      const bool more = k + 1 < n;
      const int c = ANTI ? c_first - k : c_first + k;      // chunk in hand (meaningless in the lead-in)
      const int q = qb + k;                                // its index among the chunks this CTA walks
      const uint32_t par = static_cast<uint32_t>(q) & 1u;
      const uint32_t parn = static_cast<uint32_t>(q + 1) & 1u;
      const bool has_state = k > 0 || sg.cin != 0;         // the chunk in hand received a state
      uint4 zc[4];
      if (cur) {
        cum_cur = cum_nxt; dt_cur = dt_nxt; last_cur = last_nxt;
        if (more) {
          cum_nxt = cum_pre; dt_nxt = dt_pre; colf_nxt = colf_pre;
          if (k + 2 < n) {
            const int c2 = ANTI ? c_first - k - 2 : c_first + k + 2;
            cum_pre = cum_g[c2 * WQ + r]; dt_pre = dt_g[c2 * WQ + r]; colf_pre = colf_g[c2 * WQ + r];
          }
        }
        // Yd(k) has consumed the P tile, and every warp is past the shared scalars of chunk k
        if (!walk_wait(bars + B_YFULL, par, g.status, abort)) { alive = false; break; }
      }
      if (more) {
        // ---- scalars of chunk k+1 into shared memory ------------------------------------------
        if (ch == 0) {
          s_cum[r] = cum_nxt; s_colf[r] = colf_nxt; s_dt[r] = dt_nxt;
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + B_SCAL);
        }
        if (!walk_wait(bars + B_SCAL, parn, g.status, abort)) { alive = false; break; }
        last_nxt = s_cum[WQ - 1];
        // ---- P = G o F of chunk k+1 ----------------------------------------------------------------
        if (!walk_wait(bars + B_GFULL, parn, g.status, abort)) { alive = false; break; }
        tcgen05_fence_after_sync();
#pragma unroll 1
        for (int pp = 0; pp < 2; ++pp) {
          const int pc = ch * 2 + pp;              // 32-column piece of the chunk
          const int j0 = pc * 32;
          unsigned char* prow = sP + ch * (WQ * 128) + r * 128;
          const bool zero = ANTI ? (pc < quarter) : (pc > quarter);   // warp-uniform: the whole piece is masked
          if (zero) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) *reinterpret_cast<uint4*>(prow + (((pp * 4 + q4) ^ (r & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
            continue;
          }
          uint32_t v[32];
          tmem_ld_32x32(tl + TC_G + j0, v);
          // F = row factor x column factor, both relative to the far end of the 8-column sub-piece, so that neither
          // leaves the fp32 range unless eight steps decay by more than e^-80; there (rare, and only on the
          // diagonal sub-piece) the exponent is taken per element.
          const bool diag = pc == quarter;
          tmem_ld_wait();
#pragma unroll
          for (int sp = 0; sp < 4; ++sp) {
            const int jb = j0 + sp * 8;
            const float cref = s_cum[ANTI ? jb : jb + 7];
            const float rarg = ANTI ? cref - cum_nxt : cum_nxt - cref;   // <= 0 off the diagonal
            const bool direct = rarg > 80.f;
            const float rowf = w_exp(direct ? 0.f : rarg);
            const float4 c0 = *reinterpret_cast<const float4*>(s_colf + jb);
            const float4 c1 = *reinterpret_cast<const float4*>(s_colf + jb + 4);
            float f[8] = {c0.x * rowf, c0.y * rowf, c0.z * rowf, c0.w * rowf, c1.x * rowf, c1.y * rowf, c1.z * rowf, c1.w * rowf};
            if (direct) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float cj = s_cum[jb + e];
                f[e] = ANTI ? w_exp(fminf(cj - cum_nxt, 0.f)) : w_exp(fminf(cum_nxt - cj, 0.f)) * s_dt[jb + e];
              }
            }
            if (diag) {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (ANTI ? (sp * 8 + e < lane) : (sp * 8 + e > lane)) f[e] = 0.f;
            }
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __half2 hv = __floats2half2_rn(__uint_as_float(v[sp * 8 + 2 * e]) * f[2 * e], __uint_as_float(v[sp * 8 + 2 * e + 1]) * f[2 * e + 1]);
              ow[e] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            *reinterpret_cast<uint4*>(prow + (((pp * 4 + sp) ^ (r & 7)) << 4)) = o;
          }
        }
        warp_arrive(bars + B_PREADY, lane);
      }
      if (cur) {
        if (DOT) {    // the dot partner's rows of chunk k, whole 64-byte row pieces per load
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const size_t zrow = static_cast<size_t>(b) * g.L + c * WQ + quarter * 32 + it * 8 + (lane >> 2);
            zc[it] = *reinterpret_cast<const uint4*>(g.z + zrow * pitch + h * WP + ch * 32 + (lane & 3) * 8);
          }
        }
        // ---- H' = D H + S ---------------------------------------------------------------
        if (!walk_wait(bars + B_SFULL, par, g.status, abort)) { alive = false; break; }
        tcgen05_fence_after_sync();
        if (more || sg.cout) {
          uint32_t sv[32];
          tmem_ld_32x32(tl + TC_S + ch * 32, sv);
          const float D = w_exp(last_cur);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) state[e] = D * state[e] + __uint_as_float(sv[e]);
          if (more) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 pk;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __half2 hv = __floats2half2_rn(state[q4 * 8 + 2 * e], state[q4 * 8 + 2 * e + 1]);
                ow[e] = *reinterpret_cast<const uint32_t*>(&hv);
              }
              *reinterpret_cast<uint4*>(sH + r * 128 + (((ch * 4 + q4) ^ (r & 7)) << 4)) = pk;
            }
            warp_arrive(bars + B_HREADY, lane);
          } else {
            // the first part of a sequence ends here: its state goes to the CTA that walks the rest
            float4* dst = reinterpret_cast<float4*>(g.carry + (bh * WN + r) * WP + ch * 32);
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) __stcg(dst + q4, make_float4(state[q4 * 4], state[q4 * 4 + 1], state[q4 * 4 + 2], state[q4 * 4 + 3]));
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(g.carry_flag + sg.seq, 1);
          }
        }
        // ---- out = r o (Yd + f o Yo) of chunk k -------------------------------------------
        // staging = this warp's own positions of the scaled-value tile (S(k), its last reader, has completed, and the
        // warp refills exactly these positions for chunk k+1 right after the epilogue)
        unsigned char* stg = sVs;
        if (DOT) {
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int lr = quarter * 32 + it * 8 + (lane >> 2), cc = ch * 4 + (lane & 3);
            *reinterpret_cast<uint4*>(stg + lr * 128 + ((cc ^ (lr & 7)) << 4)) = zc[it];
          }
          __syncwarp();
        }
        uint32_t yd[32], yo[32];
        const uint32_t ty = tl + TC_Y + par * 128 + ch * 32;
        tmem_ld_32x32(ty, yd);
        if (has_state) tmem_ld_32x32(ty + 64, yo);
        const float fo = has_state ? (ANTI ? w_exp(last_cur - cum_cur) : w_exp(cum_cur)) : 0.f;
        const float ro = ANTI ? dt_cur : 1.f;
        tmem_ld_wait();
        if (!has_state) {
#pragma unroll
          for (int e = 0; e < 32; ++e) yo[e] = 0u;
        }
        float o[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = ro * (__uint_as_float(yd[e]) + fo * __uint_as_float(yo[e]));
        tcgen05_fence_before_sync();
        if (DOT) {   // this thread's row of z comes back from the staging positions before the output overwrites them
          float dot = 0.f;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 zq = *reinterpret_cast<const uint4*>(stg + r * 128 + (((ch * 4 + q4) ^ (r & 7)) << 4));
            const __half2* z2 = reinterpret_cast<const __half2*>(&zq);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 zf = __half22float2(z2[e]);
              dot += zf.x * o[q4 * 8 + 2 * e] + zf.y * o[q4 * 8 + 2 * e + 1];
            }
          }
          g.dot_out[static_cast<size_t>(ch) * g.B * g.H * g.L + bh * g.L + c * WQ + r] = dot;
          __syncwarp();
        }
        if (g.out != nullptr) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 pk;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __half2 hv = __floats2half2_rn(o[q4 * 8 + 2 * e], o[q4 * 8 + 2 * e + 1]);
              ow[e] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            *reinterpret_cast<uint4*>(stg + r * 128 + (((ch * 4 + q4) ^ (r & 7)) << 4)) = pk;
          }
          __syncwarp();
          // whole 64-byte row pieces per store instruction
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int lr = quarter * 32 + it * 8 + (lane >> 2), cc = ch * 4 + (lane & 3);
            const uint4 val = *reinterpret_cast<const uint4*>(stg + lr * 128 + ((cc ^ (lr & 7)) << 4));
            const size_t orow = static_cast<size_t>(b) * g.L + c * WQ + lr;
            *reinterpret_cast<uint4*>(g.out + orow * pitch + h * WP + cc * 8) = val;
          }
          __syncwarp();
        }
      }
      if (more) {
        // ---- w o v of chunk k+1 -> operand of its state update ------------------------------------
        const int s1 = (q + 1) & 1;
        if (!walk_wait(bars + B_FULL0 + s1, static_cast<uint32_t>((q + 1) >> 1) & 1u, g.status, abort)) { alive = false; break; }
        const float wt = ANTI ? w_exp(cum_nxt) : w_exp(last_nxt - cum_nxt) * dt_nxt;
        const __half2 wt2 = __float2half2_rn(wt);
        const unsigned char* src = smem + s1 * W_STAGE + 2 * W_TILE_QK + r * 128;
        unsigned char* dst = sVs + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int off = ((ch * 4 + q4) ^ (r & 7)) << 4;
          uint4 v = *reinterpret_cast<const uint4*>(src + off);
          __half2* h2 = reinterpret_cast<__half2*>(&v);
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = __hmul2(h2[e], wt2);
          *reinterpret_cast<uint4*>(dst + off) = v;
        }
        warp_arrive(bars + B_VSREADY, lane);
      }
    }
    qb += n;
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TC_COLS);
}

// ---------------------------------------------------------------------------
// Gradients of B and C (summed over the heads of a group).  One CTA per (batch, 128-step chunk, group)
// walks the group's heads; per head h
//     Sc  = gy_h x_h^T                       128 x 128, K = 64      -> TMEM
//     acc += Sc o L_h                        in registers (L_h = causal mask * exp(cum_i - cum_j) * dt_j)
//     gC += (e_h o gy_h) Hc_h^T,  gB += (w_h o x_h) Ha_h^T          128 x 128, K = 64, accumulated over the heads in TMEM
// (Hc_h / Ha_h = the state the chunk receives from its predecessors / successors, left by the two walks;
//  e_i = exp(cum_i), w_j = exp(cum_last - cum_j) dt_j; the row factors are multiplied into the operand
//  tiles in place once the score MMA has read them).  After the last head the summed scores go to shared memory once
// and serve both products, as a K-major operand for gC += acc B and as an MN-major one for gB += acc^T C.
// No per-head score tile and no per-head partial output ever reaches global memory.
// ---------------------------------------------------------------------------
constexpr int GG_TILE = WQ * 128;                 // [128 rows][128 B]
constexpr int GG_STAGE = 4 * GG_TILE;             // gy, x, Hc, Ha
constexpr int GG_OFF_ACC = 2 * GG_STAGE;          // summed scores, [2 k-blocks][128 rows][128 B]
constexpr int GG_OFF_TAIL = GG_OFF_ACC + 2 * GG_TILE;
constexpr int GG_SMEM_BYTES = GG_OFF_TAIL + 4096 + 1024;
constexpr uint32_t GT_SC = 0, GT_C = 256, GT_B = 384;   // score buffers at 0 / 128
enum { GB_FULL0 = 0, GB_FULL1, GB_EMPTY0, GB_EMPTY1, GB_SC0, GB_SC1, GB_SCALED, GB_SCAL, GB_GG, GB_BCFULL, GB_ACC, GB_OUT, GB_COUNT };

struct GroupArgs {
  int B, L, H, G, nc;
  const float* cum; const float* dtt; const float* colf;   // [B, H, L], causal column factors
  uint32_t* status;
};

__global__ void __launch_bounds__(W_THREADS, 1) ssd_group_grads_kernel(const __grid_constant__ CUtensorMap map_gy,
                                                                      const __grid_constant__ CUtensorMap map_x,
                                                                      const __grid_constant__ CUtensorMap map_hc,
                                                                      const __grid_constant__ CUtensorMap map_ha,
                                                                      const __grid_constant__ CUtensorMap map_b,
                                                                      const __grid_constant__ CUtensorMap map_c,
                                                                      const __grid_constant__ CUtensorMap map_gb,
                                                                      const __grid_constant__ CUtensorMap map_gc, const GroupArgs g) {
  extern __shared__ unsigned char walk_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(walk_smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sGG = smem + GG_OFF_ACC;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GG_OFF_TAIL);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + GG_OFF_TAIL + 112);
  volatile int* abort = reinterpret_cast<volatile int*>(smem + GG_OFF_TAIL + 116);
  float* s_cum = reinterpret_cast<float*>(smem + GG_OFF_TAIL + 128);   // [2][128]
  float* s_colf = s_cum + 2 * WQ;                                      // [2][128]
  float* s_dt = s_colf + 2 * WQ;                                       // [2][128]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hpg = g.H / g.G;
  const int grp = blockIdx.x % g.G;
  const int c = (blockIdx.x / g.G) % g.nc;
  const int b = blockIdx.x / (g.G * g.nc);
  const int row0 = b * g.L + c * WQ;
  const int nh = hpg;

  if (threadIdx.x == 0) {
    mbar_init(bars + GB_FULL0, 1); mbar_init(bars + GB_FULL1, 1);
    mbar_init(bars + GB_EMPTY0, 1); mbar_init(bars + GB_EMPTY1, 1);
    mbar_init(bars + GB_SC0, 1); mbar_init(bars + GB_SC1, 1);
    mbar_init(bars + GB_SCALED, 8); mbar_init(bars + GB_SCAL, 8); mbar_init(bars + GB_GG, 8);
    mbar_init(bars + GB_BCFULL, 1); mbar_init(bars + GB_ACC, 1); mbar_init(bars + GB_OUT, 8);
    *abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TC_COLS);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA: loads, then the output stores -------------
    if (lane == 0) {
      bool ok = true;
      for (int hi = 0; hi < nh; ++hi) {
        const int h = grp * hpg + hi, s = hi & 1;
        if (!walk_wait(bars + GB_EMPTY0 + s, ((hi >> 1) & 1) ^ 1u, g.status, abort)) { ok = false; break; }
        unsigned char* st = smem + s * GG_STAGE;
        const int srow = ((b * g.H + h) * g.nc + c) * WN;
        mbar_arrive_expect_tx(bars + GB_FULL0 + s, GG_STAGE);
        tma_load_2d(st, &map_gy, h * WP, row0, bars + GB_FULL0 + s);
        tma_load_2d(st + GG_TILE, &map_x, h * WP, row0, bars + GB_FULL0 + s);
        tma_load_2d(st + 2 * GG_TILE, &map_hc, 0, srow, bars + GB_FULL0 + s);
        tma_load_2d(st + 3 * GG_TILE, &map_ha, 0, srow, bars + GB_FULL0 + s);
      }
      // B and C of the chunk take the place of the two stages once their last MMAs have completed
      for (int s = 0; ok && s < 2; ++s) {
        const int uses = (nh + 1 - s) / 2;       // heads that went through stage s
        if (uses > 0 && !walk_wait(bars + GB_EMPTY0 + s, (uses - 1) & 1, g.status, abort)) { ok = false; break; }
      }
      if (ok) {
        mbar_arrive_expect_tx(bars + GB_BCFULL, 4 * GG_TILE);
        tma_load_2d(smem, &map_b, grp * WN, row0, bars + GB_BCFULL);
        tma_load_2d(smem + GG_TILE, &map_b, grp * WN + 64, row0, bars + GB_BCFULL);
        tma_load_2d(smem + GG_STAGE, &map_c, grp * WN, row0, bars + GB_BCFULL);
        tma_load_2d(smem + GG_STAGE + GG_TILE, &map_c, grp * WN + 64, row0, bars + GB_BCFULL);
        if (walk_wait(bars + GB_OUT, 0, g.status, abort)) {
          // staged outputs: gC behind the B tiles of stage 0, gB behind the C tiles of stage 1
          tma_store_2d(&map_gc, smem + 2 * GG_TILE, grp * WN, row0);
          tma_store_2d(&map_gc, smem + 3 * GG_TILE, grp * WN + 64, row0);
          tma_store_2d(&map_gb, smem + GG_STAGE + 2 * GG_TILE, grp * WN, row0);
          tma_store_2d(&map_gb, smem + GG_STAGE + 3 * GG_TILE, grp * WN + 64, row0);
          bulk_commit();
          bulk_wait_all<0>();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t id_kk = umma_instr_desc(UMMA_FMT_F16, 0u, 0u, 128, 128);   // K-major x K-major
      const uint32_t id_kn = umma_instr_desc(UMMA_FMT_F16, 0u, 1u, 128, 128);   // K-major A x MN-major B
      const uint32_t id_nn = umma_instr_desc(UMMA_FMT_F16, 1u, 1u, 128, 128);   // MN-major A x MN-major B
      auto issue_score = [&](int hi) {
        const uint32_t st = mp_smem_u32(smem + (hi & 1) * GG_STAGE);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma<false>(tmem + GT_SC + (hi & 1) * 128, umma_smem_desc(st + ks * 32, 16, 1024), umma_smem_desc(st + GG_TILE + ks * 32, 16, 1024),
                      id_kk, ks != 0 ? 1u : 0u);
        umma_commit(bars + GB_SC0 + (hi & 1));
      };
      bool ok = walk_wait(bars + GB_FULL0, 0, g.status, abort);
      if (ok) { tcgen05_fence_after_sync(); issue_score(0); }
      for (int hi = 0; ok && hi < nh; ++hi) {
        const int s = hi & 1;
        if (hi + 1 < nh) {   // the next head's scores run while the workers transform this head's
          if (!walk_wait(bars + GB_FULL0 + ((hi + 1) & 1), ((hi + 1) >> 1) & 1, g.status, abort)) { ok = false; break; }
          tcgen05_fence_after_sync();
          issue_score(hi + 1);
        }
        if (!walk_wait(bars + GB_SCALED, hi & 1, g.status, abort)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t st = mp_smem_u32(smem + s * GG_STAGE);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma<false>(tmem + GT_C, umma_smem_desc(st + ks * 32, 16, 1024), umma_smem_desc(st + 2 * GG_TILE + ks * 32, 16, 1024), id_kk,
                      (hi | ks) != 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma<false>(tmem + GT_B, umma_smem_desc(st + GG_TILE + ks * 32, 16, 1024), umma_smem_desc(st + 3 * GG_TILE + ks * 32, 16, 1024), id_kk,
                      (hi | ks) != 0 ? 1u : 0u);
        umma_commit(bars + GB_EMPTY0 + s);
      }
      // summed scores x B and (summed scores)^T x C
      if (ok) ok = walk_wait(bars + GB_GG, 0, g.status, abort) && walk_wait(bars + GB_BCFULL, 0, g.status, abort);
      if (ok) {
        tcgen05_fence_after_sync();
        const uint32_t sg = mp_smem_u32(sGG), sb = mp_smem_u32(smem), sc = mp_smem_u32(smem + GG_STAGE);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)     // K = step j: A K-major over the two 64-column blocks, B rows j (MN-major, two 64-column blocks)
          umma<false>(tmem + GT_C, umma_smem_desc(sg + (ks >> 2) * GG_TILE + (ks & 3) * 32, 16, 1024), umma_smem_desc(sb + ks * 2048, GG_TILE, 1024),
                      id_kn, 1u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)     // K = step i: A = transposed view of the same tile (MN-major), C rows i
          umma<false>(tmem + GT_B, umma_smem_desc(sg + ks * 2048, GG_TILE, 1024), umma_smem_desc(sc + ks * 2048, GG_TILE, 1024), id_nn, 1u);
        umma_commit(bars + GB_ACC);
      }
    }
  } else {
    // ------------------------------ workers -----------------------------------
    const int quarter = warp & 3;
    const int ch = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t tl = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    float acc[64];
#pragma unroll
    for (int e = 0; e < 64; ++e) acc[e] = 0.f;
    auto scal_ptr = [&](const float* base, int hi) { return base + (static_cast<size_t>(b) * g.H + grp * hpg + hi) * g.L + c * WQ + r; };
    float cum_n = *scal_ptr(g.cum, 0), dt_n = *scal_ptr(g.dtt, 0), colf_n = *scal_ptr(g.colf, 0);
    float cum_p = 0.f, dt_p = 0.f, colf_p = 0.f;
    if (nh > 1) { cum_p = *scal_ptr(g.cum, 1); dt_p = *scal_ptr(g.dtt, 1); colf_p = *scal_ptr(g.colf, 1); }
    bool ok = true;
    for (int hi = 0; hi < nh; ++hi) {
      const int s = hi & 1;
      const float cum_r = cum_n, dt_r = dt_n;
      float* cumb = s_cum + s * WQ;
      float* colfb = s_colf + s * WQ;
      float* dtb = s_dt + s * WQ;
      // every warp arrives: the phase also tells the writers of the other buffer that all warps are done with it
      if (ch == 0) { cumb[r] = cum_n; colfb[r] = colf_n; dtb[r] = dt_n; }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + GB_SCAL);
      cum_n = cum_p; dt_n = dt_p; colf_n = colf_p;
      if (hi + 2 < nh) { cum_p = *scal_ptr(g.cum, hi + 2); dt_p = *scal_ptr(g.dtt, hi + 2); colf_p = *scal_ptr(g.colf, hi + 2); }
      if (!walk_wait(bars + GB_SCAL, hi & 1, g.status, abort)) { ok = false; break; }
      const float cum_last = cumb[WQ - 1];
      // ---- acc += Sc o L ------------------------------------------------------------
      if (!walk_wait(bars + GB_SC0 + s, (hi >> 1) & 1, g.status, abort)) { ok = false; break; }
      tcgen05_fence_after_sync();
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        const int pc = ch * 2 + pp;
        const int j0 = pc * 32;
        if (pc > quarter) continue;                 // above the diagonal for every row of the warp
        uint32_t v[32];
        tmem_ld_32x32(tl + GT_SC + s * 128 + j0, v);
        const bool diag = pc == quarter;
        tmem_ld_wait();
#pragma unroll
        for (int sp = 0; sp < 4; ++sp) {      // factors relative to the last column of each 8-column sub-piece (see the walk kernel)
          const int jb = j0 + sp * 8;
          const float rarg = cum_r - cumb[jb + 7];
          const bool direct = rarg > 80.f;
          const float rowf = w_exp(direct ? 0.f : rarg);
          const float4 c0 = *reinterpret_cast<const float4*>(colfb + jb);
          const float4 c1 = *reinterpret_cast<const float4*>(colfb + jb + 4);
          float f[8] = {c0.x * rowf, c0.y * rowf, c0.z * rowf, c0.w * rowf, c1.x * rowf, c1.y * rowf, c1.z * rowf, c1.w * rowf};
          if (direct) {
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = w_exp(fminf(cum_r - cumb[jb + e], 0.f)) * dtb[jb + e];
          }
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (!diag || sp * 8 + e <= lane) acc[pp * 32 + sp * 8 + e] += __uint_as_float(v[sp * 8 + e]) * f[e];
        }
      }
      // ---- row factors into the operand tiles, in place (the score MMA has read them) ----
      {
        const __half2 e2 = __float2half2_rn(w_exp(cum_r));
        const __half2 w2 = __float2half2_rn(w_exp(cum_last - cum_r) * dt_r);
        unsigned char* gyrow = smem + s * GG_STAGE + r * 128;
        unsigned char* xrow = gyrow + GG_TILE;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int off = ((ch * 4 + q4) ^ (r & 7)) << 4;
          uint4 a = *reinterpret_cast<const uint4*>(gyrow + off);
          uint4 x4 = *reinterpret_cast<const uint4*>(xrow + off);
          __half2* ha = reinterpret_cast<__half2*>(&a);
          __half2* hx = reinterpret_cast<__half2*>(&x4);
#pragma unroll
          for (int e = 0; e < 4; ++e) { ha[e] = __hmul2(ha[e], e2); hx[e] = __hmul2(hx[e], w2); }
          *reinterpret_cast<uint4*>(gyrow + off) = a;
          *reinterpret_cast<uint4*>(xrow + off) = x4;
        }
      }
      warp_arrive(bars + GB_SCALED, lane);
    }
    if (ok) {
      // ---- summed scores -> r16 operand tile ------------------------------------------
      unsigned char* prow = sGG + ch * GG_TILE + r * 128;
#pragma unroll
      for (int q8 = 0; q8 < 8; ++q8) {
        uint4 pk;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __half2 hv = __floats2half2_rn(acc[q8 * 8 + 2 * e], acc[q8 * 8 + 2 * e + 1]);
          ow[e] = *reinterpret_cast<const uint32_t*>(&hv);
        }
        *reinterpret_cast<uint4*>(prow + ((q8 ^ (r & 7)) << 4)) = pk;
      }
      warp_arrive(bars + GB_GG, lane);
      // ---- outputs ---------------------------------------------------------------------
      if (walk_wait(bars + GB_ACC, 0, g.status, abort)) {
        tcgen05_fence_after_sync();
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {   // 0: gC (staged behind B in stage 0), 1: gB (behind C in stage 1)
          unsigned char* stg = smem + which * GG_STAGE + 2 * GG_TILE + ch * GG_TILE + r * 128;
#pragma unroll
          for (int pp = 0; pp < 2; ++pp) {
            uint32_t v[32];
            tmem_ld_32x32(tl + (which ? GT_B : GT_C) + ch * 64 + pp * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 pk;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __half2 hv = __floats2half2_rn(__uint_as_float(v[q4 * 8 + 2 * e]), __uint_as_float(v[q4 * 8 + 2 * e + 1]));
                ow[e] = *reinterpret_cast<const uint32_t*>(&hv);
              }
              *reinterpret_cast<uint4*>(stg + (((pp * 4 + q4) ^ (r & 7)) << 4)) = pk;
            }
          }
        }
        warp_arrive(bars + GB_OUT, lane);
      }
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TC_COLS);
}

// dt*A prefix sums inside every 128-step chunk, dt, and the column factors of both walk directions, all in
// [B, H, L] order.  One CTA per (b, h, chunk).  Column factor of step t relative to the far end of its 8-step
// piece: causal exp(cum[t | 7] - cum[t]) dt[t], anti-causal exp(cum[t] - cum[t & ~7]); both are at most one (dt).
// RAW: the step sizes arrive as the projection's raw r16 output (row pitch `raw_pitch`) and the decay rates as A_log:
//   dt = softplus(raw + bias[h]), A = -exp(A_log[h])  (the arithmetic of launch_softplus_bias / launch_neg_exp),
// both also written out (dt_out [B, L, H], A_out [H]) for the reverse pass.
template <bool RAW>
__global__ void __launch_bounds__(WQ) ssd_walk_cumsum_kernel(const float* __restrict__ dt, const float* __restrict__ A, float* __restrict__ cum,
                                                             float* __restrict__ dtt, float* __restrict__ colf_c, float* __restrict__ colf_a,
                                                             int L, int H, int* __restrict__ carry_flags, int n_flags,
                                                             const __half* __restrict__ raw, size_t raw_pitch, const float* __restrict__ bias,
                                                             float* __restrict__ dt_out, float* __restrict__ A_out) {
  __shared__ float warp_tot[4];
  if (blockIdx.x == 0)   // the walks that follow in stream order hand states from CTA to CTA through these counters
    for (int i = threadIdx.x; i < n_flags; i += WQ) carry_flags[i] = 0;
  const int nc = L / WQ;
  const int c = blockIdx.x % nc, h = (blockIdx.x / nc) % H, b = blockIdx.x / (nc * H);
  const int t = threadIdx.x;
  float d, a;
  if (RAW) {
    const size_t row = static_cast<size_t>(b) * L + c * WQ + t;
    const float pre = __half2float(raw[row * raw_pitch + h]) + bias[h];
    d = pre > 20.f ? pre : log1pf(__expf(pre));
    a = -__expf(A[h]);
    dt_out[row * H + h] = d;
    if (b == 0 && c == 0 && t == 0) A_out[h] = a;
  } else {
    d = dt[(static_cast<size_t>(b) * L + c * WQ + t) * H + h];
    a = A[h];
  }
  float v = d * a;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, off);
    if ((t & 31) >= off) v += n;
  }
  if ((t & 31) == 31) warp_tot[t >> 5] = v;
  __syncthreads();
  float base = 0.f;
  for (int w = 0; w < (t >> 5); ++w) base += warp_tot[w];
  const float cv = v + base;
  const float c_hi = __shfl_sync(0xffffffffu, cv, (t & 31) | 7), c_lo = __shfl_sync(0xffffffffu, cv, (t & 31) & ~7);
  const size_t o = (static_cast<size_t>(b) * H + h) * L + c * WQ + t;
  cum[o] = cv;
  dtt[o] = d;
  colf_c[o] = w_exp(c_hi - cv) * d;
  if (colf_a != nullptr) colf_a[o] = w_exp(cv - c_lo);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn walk_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    MP_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (p == nullptr || q != cudaDriverEntryPointSuccess) MP_FATAL("cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// r16 matrix [rows, cols] (row-major), box {64 columns, 128 rows}, 128-byte swizzle
CUtensorMap walk_map(const void* base, size_t rows, size_t cols) {
  CUtensorMap m;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * sizeof(__half)};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t es[2] = {1, 1};
  MP_CU_CHECK(walk_encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return m;
}

}  // namespace

// Host-side view of the chunk walk's work partition (the function the kernels use, compiled for the host): segment
// `idx` of CTA `cta` out of `ncta` for `nseq` sequences of `nc` chunks -> out = {sequence, first position, chunks,
// carried-in state, carried-out state}; returns 0 past the CTA's last segment.  For tests; needs no GPU.
extern "C" int mpSsdWalkPartition(int cta, int ncta, int nseq, int nc, int idx, int* out) {
  WalkSeg sg;
  if (ncta <= 0 || ncta > nseq || nc <= 0 || cta < 0 || cta >= ncta || idx < 0) return 0;
  if (!walk_segment(cta, ncta, nseq, nc, idx, sg)) return 0;
  out[0] = sg.seq; out[1] = sg.p0; out[2] = sg.n; out[3] = sg.cin; out[4] = sg.cout;
  return 1;
}

// ---------------------------------------------------------------------------
// Interface to the launchers in ssd.cu.
// ---------------------------------------------------------------------------
bool mp_ssd_walk_supported(int L, int H, int P, int N, int G) {
  return P == WP && N == WN && L % WQ == 0 && L > 0 && G > 0 && H % G == 0 && getenv("MP_SSD_NO_WALK") == nullptr;
}

void mp_ssd_walk_cumsum(const float* dt, const float* A, float* cum, float* dtt, float* colf_c, float* colf_a, int B, int L, int H,
                        int* carry_flags, int n_flags, cudaStream_t st) {
  ssd_walk_cumsum_kernel<false><<<B * H * (L / WQ), WQ, 0, st>>>(dt, A, cum, dtt, colf_c, colf_a, L, H, carry_flags, n_flags, nullptr, 0, nullptr,
                                                                 nullptr, nullptr);
  MP_LAUNCH_CHECK();
}

// The same from the raw projection output and A_log (see the kernel); dt_out and A_out are what the reverse pass takes.
void mp_ssd_walk_cumsum_raw(const __half* raw, size_t raw_pitch, const float* bias, const float* A_log, float* dt_out, float* A_out, float* cum,
                            float* dtt, float* colf_c, int B, int L, int H, int* carry_flags, int n_flags, cudaStream_t st) {
  ssd_walk_cumsum_kernel<true><<<B * H * (L / WQ), WQ, 0, st>>>(nullptr, A_log, cum, dtt, colf_c, nullptr, L, H, carry_flags, n_flags, raw, raw_pitch,
                                                                bias, dt_out, A_out);
  MP_LAUNCH_CHECK();
}

// One walk.  q, k: [B*L, G*128]; v, z, out: [B*L, H*64]; cum, dtt, colf (of the walk's direction): [B, H, L] from mp_ssd_walk_cumsum.
void mp_ssd_walk(int anti, const __half* q, const __half* k, const __half* v, const float* cum, const float* dtt, const float* colf, __half* out,
                 const __half* z,
                 float* dot_out, __half* hs_out, float* carry, int* carry_flag, int max_ctas, int B, int L, int H, int G, uint32_t* status,
                 cudaStream_t st) {
  WalkArgs g;
  g.B = B; g.L = L; g.H = H; g.G = G; g.nc = L / WQ;
  g.cum = cum; g.dtt = dtt; g.colf = colf; g.out = out; g.z = z; g.dot_out = dot_out; g.hs_out = hs_out; g.status = status;
  g.carry = carry; g.carry_flag = carry_flag;
  // One CTA per SM slot it may use, every CTA the same number of chunks; never more CTAs than sequences, so that a CTA's
  // range is at least one sequence long (see walk_segment).  MP_SSD_WALK_PER_SEQUENCE: one CTA per sequence, no hand-off.
  int grid = B * H;
  if (max_ctas > 0 && max_ctas < grid && getenv("MP_SSD_WALK_PER_SEQUENCE") == nullptr) grid = max_ctas;
  const size_t rows = static_cast<size_t>(B) * L;
  const CUtensorMap mq = walk_map(q, rows, static_cast<size_t>(G) * WN), mk = walk_map(k, rows, static_cast<size_t>(G) * WN);
  const CUtensorMap mv = walk_map(v, rows, static_cast<size_t>(H) * WP);
  const CUtensorMap mh = hs_out != nullptr ? walk_map(hs_out, static_cast<size_t>(B) * H * g.nc * WN, WP) : mv;
  auto launch = [&](auto kernel) {
    MP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES));
    kernel<<<grid, W_THREADS, W_SMEM_BYTES, st>>>(mq, mk, mv, mh, g);
  };
  const bool dot = z != nullptr && dot_out != nullptr;
  if (!dot) { g.z = nullptr; g.dot_out = nullptr; }
  if (anti) {
    if (dot) launch(ssd_walk_kernel<1, true>); else launch(ssd_walk_kernel<1, false>);
  } else {
    if (dot) launch(ssd_walk_kernel<0, true>); else launch(ssd_walk_kernel<0, false>);
  }
  MP_LAUNCH_CHECK();
}

// gB, gC [B*L, G*128] from gy, x [B*L, H*64], Bm, Cm [B*L, G*128] and the states left by the two walks
// (hs_causal, hs_anti: [B, H, L/128][128][64]).
void mp_ssd_group_grads(const __half* gy, const __half* x, const __half* Bm, const __half* Cm, const __half* hs_causal, const __half* hs_anti,
                        const float* cum, const float* dtt, const float* colf_c, __half* gB, __half* gC, int B, int L, int H, int G,
                        uint32_t* status, cudaStream_t st) {
  GroupArgs g;
  g.B = B; g.L = L; g.H = H; g.G = G; g.nc = L / WQ;
  g.cum = cum; g.dtt = dtt; g.colf = colf_c; g.status = status;
  const size_t rows = static_cast<size_t>(B) * L;
  const size_t srows = static_cast<size_t>(B) * H * g.nc * WN;
  const CUtensorMap mgy = walk_map(gy, rows, static_cast<size_t>(H) * WP), mx = walk_map(x, rows, static_cast<size_t>(H) * WP);
  const CUtensorMap mhc = walk_map(hs_causal, srows, WP), mha = walk_map(hs_anti, srows, WP);
  const CUtensorMap mb = walk_map(Bm, rows, static_cast<size_t>(G) * WN), mc = walk_map(Cm, rows, static_cast<size_t>(G) * WN);
  const CUtensorMap mgb = walk_map(gB, rows, static_cast<size_t>(G) * WN), mgc = walk_map(gC, rows, static_cast<size_t>(G) * WN);
  MP_CUDA_CHECK(cudaFuncSetAttribute(ssd_group_grads_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GG_SMEM_BYTES));
  ssd_group_grads_kernel<<<B * g.nc * G, W_THREADS, GG_SMEM_BYTES, st>>>(mgy, mx, mhc, mha, mb, mc, mgb, mgc, g);
  MP_LAUNCH_CHECK();
}
