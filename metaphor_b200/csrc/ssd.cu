// Mamba-2 SSD (state-space dual) chunked scan, forward and reverse, r16 storage
// with fp32 accumulation.  No kernel for it exists in the reference; the op is
// defined by the recurrence (per batch b, head h, group g(h)):
//     S_t = exp(dt_t A_h) S_{t-1} + dt_t B_t x_t^T,    y_t = C_t^T S_t .
//
// Everything here is one operator evaluated chunk by chunk (chunk length Q):
//     out_i = r_i * sum_j mask(i,j) * decay(i,j) * c_j * <q_i, k_j> * v_j
//   causal      : j <= i, decay = exp(cum_i - cum_j), c_j = dt_j, r_i = 1
//   anti-causal : j >= i, decay = exp(cum_j - cum_i), c_j = 1,    r_i = dt_i
// with cum the inclusive prefix sum of dt*A.  The forward pass is the causal
// operator with (q,k,v) = (C,B,x); the reverse pass is three more instances
//     gx = anti  (q,k,v) = (B, C, gy)
//     gC = causal(q,k,v) = (gy, x, B)  summed over the heads of a group
//     gB = anti  (q,k,v) = (x, gy, C)  summed over the heads of a group
// and gdt, gA follow from u_t = <gy_t, y_t>, v_t = <gx_t, x_t>:
//     g_a[k] = sum_{t >= k} (u_t - v_t),  gdt_k = v_k/dt_k + A_h g_a[k],  gA_h = sum dt_k g_a[k].
//
// One instance = four tensor-core phases (tcgen05.mma, operands by TMA into
// 128-byte-swizzled shared memory, fp32 accumulators in TMEM):
//   scores  G   = q k^T per chunk                       (Q x Q, K = dk), r16
//   states  S_c = k^T diag(w) v per chunk               (dk x dv, K = Q), fp32
//   scan    H_c : inter-chunk recurrence over S_c       (element-wise, r16 out)
//   output  out = (G o F) v + diag(f) q H_c             (Q x dv, K = Q and dk)
// The decay / mask / dt factors F, f, w are applied to an operand tile in
// shared memory by the four epilogue warps between the TMA arrival and the MMA
// (the same place the r32 contraction kernel splits its operands).
#include "mp_tcgen05.cuh"

#include <cuda.h>
#include <mutex>

namespace {

#ifndef SSD_XF
#define SSD_XF 2   // chunks per iteration of the (rolled) transform loops: compact code, two loads in flight
#endif
constexpr int SSD_THREADS = 192;  // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: transform + epilogue
constexpr int SSD_MAX_STAGES = 4;
constexpr int TILE_BYTES = 128 * 128;  // one operand tile: 128 rows x 128 B, or two 64x64 MN-major boxes
constexpr int BOX_BYTES = 64 * 128;    // MN-major box: 64 k-rows x 64 elements
enum { MODE_SCORES = 0, MODE_STATES = 1, MODE_OUTPUT = 2 };

struct SsdArgs {
  int B, L, H, G, Q, nc;
  int dk, dv;             // inner-product width and value width (64 or 128)
  int anti;               // 0 causal, 1 anti-causal
  int q_head, k_head, v_head;   // 1: the tensor's column block is indexed by head, 0: by group
  int scores_head;        // scores kept per head (1) or per group (0)
  int out_head;           // output per head (1) or per group, summed over the group's heads (0)
  int state_t;            // states stored transposed: [dv x dk] (dk contiguous)
  const float* cum;       // [B, H, nc, Q] inclusive prefix sum of dt*A inside the chunk
  const float* dtt;       // [B, H, nc, Q] dt
  int stages;             // pipeline depth (2..4)
  int stage_bytes;        // A tile (16 KB) + the largest B tile of this launch
  int tmem_cols;          // accumulator columns to allocate (power of two >= tile width)
  __half* g_out;          // SCORES: [(b, c, unit) * Q + i][Q]
  float* s_out;           // STATES: [(b, h, c)][128][d2]
  __half* o_out;          // OUTPUT: row b*L + t, column unit*dv + j (may be null)
  int o_pitch;
  const __half* z;        // OUTPUT: optional row-dot partner, same indexing as o_out
  int z_pitch;
  float* dot_out;         // [B, H, L]
  float* part_out;        // OUTPUT per group: fp32 partial sums [split][B*L][G*dv] (the heads of a group are
  int head_splits;        //   divided over head_splits CTAs and folded afterwards); null / 1 otherwise
  uint32_t* status;
};

__device__ __forceinline__ float ssd_exp(float x) { return __expf(x); }

// ---------------------------------------------------------------------------
// dt*A prefix sums per chunk and dt in [B,H,L] order.  One CTA per (b, h, c).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ssd_cumsum_kernel(const float* __restrict__ dt, const float* __restrict__ A,
                                                         float* __restrict__ cum, float* __restrict__ dtt, int B, int L,
                                                         int H, int Q) {
  __shared__ float warp_tot[8];
  const int nc = L / Q;
  const int c = blockIdx.x % nc, h = (blockIdx.x / nc) % H, b = blockIdx.x / (nc * H);
  const int t = threadIdx.x;
  float a = 0.f, d = 0.f;
  if (t < Q) {
    d = dt[(static_cast<size_t>(b) * L + c * Q + t) * H + h];
    a = d * A[h];
  }
  float v = a;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, off);
    if ((t & 31) >= off) v += n;
  }
  if ((t & 31) == 31) warp_tot[t >> 5] = v;
  __syncthreads();
  float base = 0.f;
  for (int w = 0; w < (t >> 5); ++w) base += warp_tot[w];
  if (t < Q) {
    const size_t o = (static_cast<size_t>(b) * H + h) * L + c * Q + t;
    cum[o] = v + base;
    dtt[o] = d;
  }
}

// ---------------------------------------------------------------------------
// Inter-chunk recurrence.  S: fp32 [B,H,nc,E]; Hs: r16 [B,H,nc,E] = the state a
// chunk receives from its predecessors (causal) or successors (anti-causal).
//   causal: Hs[0] = 0, Hs[c+1] = D_c Hs[c] + S_c      anti: Hs[nc-1] = 0, Hs[c] = S_{c+1} + D_{c+1} Hs[c+1]
// with D_c = exp(cum of the chunk's last step).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ssd_scan_kernel(const float* __restrict__ S, __half* __restrict__ Hs,
                                                       const float* __restrict__ cum, int nc, int Q, int E, int anti) {
  const int bh = blockIdx.y;
  const int e = blockIdx.x * 256 + threadIdx.x;
  if (e >= E) return;
  const float* s = S + static_cast<size_t>(bh) * nc * E + e;
  __half* hs = Hs + static_cast<size_t>(bh) * nc * E + e;
  const float* cl = cum + static_cast<size_t>(bh) * nc * Q + (Q - 1);
  float st = 0.f;
  if (!anti) {
    for (int c = 0; c < nc; ++c) {
      hs[static_cast<size_t>(c) * E] = __float2half_rn(st);
      st = ssd_exp(cl[static_cast<size_t>(c) * Q]) * st + s[static_cast<size_t>(c) * E];
    }
  } else {
    for (int c = nc - 1; c >= 0; --c) {
      hs[static_cast<size_t>(c) * E] = __float2half_rn(st);
      st = ssd_exp(cl[static_cast<size_t>(c) * Q]) * st + s[static_cast<size_t>(c) * E];
    }
  }
}

// ---------------------------------------------------------------------------
// The tensor-core kernel (three modes).
// ---------------------------------------------------------------------------
struct Item {
  int head;   // head whose decay / dt factors apply
  int off;    // OUTPUT: 0 = in-chunk block (scores x values), 1 = carried-state block (q x state)
  int kb;     // 64-wide k-block index
};

template <int MODE>
__device__ __forceinline__ int ssd_num_items(const SsdArgs& g, int mt, int c, int nheads) {
  if (MODE == MODE_SCORES) return g.dk / 64;
  if (MODE == MODE_STATES) return g.Q / 64;
  const int kq = g.Q / 64;
  const int n_diag = g.anti ? (kq - 2 * mt) : (2 * mt + 2);
  const bool has_state = g.anti ? (c < g.nc - 1) : (c > 0);
  const int n_off = has_state ? g.dk / 64 : 0;
  return nheads * (n_diag + n_off);
}

template <int MODE>
__device__ __forceinline__ Item ssd_item(const SsdArgs& g, int it, int mt, int c, int head0) {
  Item r;
  r.head = head0; r.off = 0; r.kb = it;
  if (MODE == MODE_OUTPUT) {
    const int kq = g.Q / 64;
    const int n_diag = g.anti ? (kq - 2 * mt) : (2 * mt + 2);
    const bool has_state = g.anti ? (c < g.nc - 1) : (c > 0);
    const int per = n_diag + (has_state ? g.dk / 64 : 0);
    const int hh = g.out_head ? 0 : it / per, w = g.out_head ? it : it % per;   // one head per CTA: no division
    r.head = head0 + hh;
    if (w < n_diag) { r.off = 0; r.kb = g.anti ? (2 * mt + w) : w; }
    else { r.off = 1; r.kb = w - n_diag; }
  }
  return r;
}

// Column factors of the chunk's Q steps for the head whose cum / dt are in shared memory:
//   causal: colf_j = exp(cum_ref - cum_j) dt_j, ref = last column of j's 64-column k-block
//   anti  : colf_j = exp(cum_j - cum_ref),      ref = first column of the k-block
// (never above one).  Called by the 128 transform threads.
__device__ __forceinline__ void ssd_fill_colf(const SsdArgs& g, const float* cm, const float* dd, float* colf, int et) {
  for (int t = et; t < g.Q; t += 128) {
    const int ref = g.anti ? (t & ~63) : (t | 63);
    colf[t] = g.anti ? ssd_exp(cm[t] - cm[ref]) : ssd_exp(cm[ref] - cm[t]) * dd[t];
  }
}

template <int MODE>
__global__ void __launch_bounds__(SSD_THREADS, 4) ssd_mma_kernel(const __grid_constant__ CUtensorMap map_a0,
                                                                const __grid_constant__ CUtensorMap map_b0,
                                                                const __grid_constant__ CUtensorMap map_a1,
                                                                const __grid_constant__ CUtensorMap map_b1,
                                                                const SsdArgs g) {
  extern __shared__ unsigned char ssd_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ssd_smem_raw) + 1023) & ~uintptr_t(1023));
  const int STAGES = g.stages, STAGE_BYTES = g.stage_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* ready = full + SSD_MAX_STAGES;
  uint64_t* empty = ready + SSD_MAX_STAGES;
  uint64_t* acc_full = empty + SSD_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_cum = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);  // [Q] of the head being transformed
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hpg = g.H / g.G;

  // ---- which tile is this CTA ------------------------------------------------
  // blockIdx.z enumerates (b, c, unit); unit = head or group depending on mode.
  int units;
  if (MODE == MODE_SCORES) units = g.scores_head ? g.H : g.G;
  else if (MODE == MODE_STATES) units = g.H;
  else units = g.out_head ? g.H : g.G;
  const int unit = blockIdx.z % units;
  const int c = (blockIdx.z / units) % g.nc;
  const int b = blockIdx.z / (units * g.nc);
  const int mt = blockIdx.y, nt = blockIdx.x;
  const int r0 = b * g.L + c * g.Q;  // first time row of the chunk in the [B*L, ...] tensors

  if (MODE == MODE_SCORES) {
    // tiles entirely outside the mask are never read by the consumer
    if ((!g.anti && nt > mt) || (g.anti && nt < mt)) return;
  }
  int head0, nheads;
  if (MODE == MODE_SCORES) { head0 = g.scores_head ? unit : unit * hpg; nheads = 1; }
  else if (MODE == MODE_STATES) { head0 = unit; nheads = 1; }
  else {
    const int hps = g.out_head ? 1 : hpg / g.head_splits;   // heads per CTA
    head0 = g.out_head ? unit : unit * hpg + static_cast<int>(blockIdx.x) * hps;
    nheads = hps;
  }
  float* s_dt = s_cum + g.Q;
  float* s_colf = s_dt + g.Q;   // [Q] column factors, each 64-column k-block relative to its own reference column
  const int n_items = ssd_num_items<MODE>(g, mt, c, nheads);
  const int tile_n = MODE == MODE_SCORES ? 128 : (MODE == MODE_STATES ? (g.dk == 128 ? g.dv : g.dk) : g.dv);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(ready + s, 128); mbar_init(empty + s, 1); }
    mbar_init(acc_full, 1);
    *abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, g.tmem_cols);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_acc = *tmem_slot;

  // column block of a [rows, heads-or-groups * width] tensor for a head
  auto colblk = [&](int per_head, int head, int width) { return (per_head ? head : head / hpg) * width; };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t phase = 0;
      for (int it = 0; it < n_items; ++it) {
        const Item w = ssd_item<MODE>(g, it, mt, c, head0);
        if (!mbar_wait_abortable(empty + s, phase ^ 1u, g.status, abort)) break;
        unsigned char* sa = smem + s * STAGE_BYTES;
        unsigned char* sb = sa + TILE_BYTES;
        if (MODE == MODE_SCORES) {
          mbar_arrive_expect_tx(full + s, 2 * TILE_BYTES);
          tma_load_2d(sa, &map_a0, colblk(g.q_head, w.head, g.dk) + w.kb * 64, r0 + mt * 128, full + s);
          tma_load_2d(sb, &map_b0, colblk(g.k_head, w.head, g.dk) + w.kb * 64, r0 + nt * 128, full + s);
        } else if (MODE == MODE_STATES) {
          // A = X1^T (128 wide, MN-major: two 64x64 boxes), B = X2 (tile_n wide, MN-major)
          const bool kfirst = g.dk == 128;   // X1 = k, X2 = v; otherwise X1 = v, X2 = k (transposed state)
          const int c1 = kfirst ? colblk(g.k_head, w.head, g.dk) : colblk(g.v_head, w.head, g.dv);
          const int c2 = kfirst ? colblk(g.v_head, w.head, g.dv) : colblk(g.k_head, w.head, g.dk);
          const CUtensorMap* m1 = kfirst ? &map_a0 : &map_b0;   // a0 = k tensor, b0 = v tensor
          const CUtensorMap* m2 = kfirst ? &map_b0 : &map_a0;
          mbar_arrive_expect_tx(full + s, 2 * BOX_BYTES + (tile_n / 64) * BOX_BYTES);
          for (int j = 0; j < 2; ++j) tma_load_2d(sa + j * BOX_BYTES, m1, c1 + j * 64, r0 + w.kb * 64, full + s);
          for (int j = 0; j < tile_n / 64; ++j) tma_load_2d(sb + j * BOX_BYTES, m2, c2 + j * 64, r0 + w.kb * 64, full + s);
        } else {
          if (!w.off) {
            // A = scores tile (K-major 128 x 64), B = value rows of the k-block (MN-major boxes)
            const int su = g.scores_head ? w.head : w.head / hpg;
            const int sunits = g.scores_head ? g.H : g.G;
            mbar_arrive_expect_tx(full + s, TILE_BYTES + (g.dv / 64) * BOX_BYTES);
            tma_load_2d(sa, &map_a0, w.kb * 64, ((b * g.nc + c) * sunits + su) * g.Q + mt * 128, full + s);
            for (int j = 0; j < g.dv / 64; ++j)
              tma_load_2d(sb + j * BOX_BYTES, &map_b0, colblk(g.v_head, w.head, g.dv) + j * 64, r0 + w.kb * 64, full + s);
          } else {
            // A = q tile (K-major 128 x 64 of dk), B = carried state of (b, head, c)
            const int srow = ((b * g.H + w.head) * g.nc + c) * 128;   // states are [128][d2] blocks
            mbar_arrive_expect_tx(full + s, TILE_BYTES + (g.state_t ? TILE_BYTES : (g.dv / 64) * BOX_BYTES));
            tma_load_2d(sa, &map_a1, colblk(g.q_head, w.head, g.dk) + w.kb * 64, r0 + mt * 128, full + s);
            if (g.state_t) {
              tma_load_2d(sb, &map_b1, w.kb * 64, srow, full + s);   // [dv = 128 rows][64 of dk], K-major
            } else {
              for (int j = 0; j < g.dv / 64; ++j) tma_load_2d(sb + j * BOX_BYTES, &map_b1, j * 64, srow + w.kb * 64, full + s);
            }
          }
        }
        if (++s == STAGES) { s = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int s = 0; uint32_t phase = 0; bool ok = true;
      for (int it = 0; it < n_items; ++it) {
        const Item w = ssd_item<MODE>(g, it, mt, c, head0);
        uint64_t* wait_on = MODE == MODE_SCORES ? (full + s) : (ready + s);
        if (!mbar_wait_abortable(wait_on, phase, g.status, abort)) { ok = false; break; }
        tcgen05_fence_after_sync();
        const uint32_t sa = mp_smem_u32(smem + s * STAGE_BYTES), sb = sa + TILE_BYTES;
        const bool a_mn = MODE == MODE_STATES;
        const bool b_mn = MODE == MODE_STATES || (MODE == MODE_OUTPUT && !(w.off && g.state_t));
        const uint32_t idesc = umma_instr_desc(UMMA_FMT_F16, a_mn ? 1u : 0u, b_mn ? 1u : 0u, 128, tile_n);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {   // 64-wide k-block = 4 x K16
          const uint64_t ad = a_mn ? umma_smem_desc(sa + ks * 16 * 128, BOX_BYTES, 1024) : umma_smem_desc(sa + ks * 32, 16, 1024);
          const uint64_t bd = b_mn ? umma_smem_desc(sb + ks * 16 * 128, BOX_BYTES, 1024) : umma_smem_desc(sb + ks * 32, 16, 1024);
          umma<false>(tmem_acc, ad, bd, idesc, (it | ks) != 0 ? 1u : 0u);
        }
        umma_commit(empty + s);
        if (++s == STAGES) { s = 0; phase ^= 1u; }
      }
      if (ok && n_items > 0) umma_commit(acc_full);
    }
  } else {
    // ---------------- operand transforms, then the epilogue --------------------
    const int et = threadIdx.x - 64;  // 0..127 = accumulator row
    if (MODE != MODE_SCORES) {
      int s = 0; uint32_t phase = 0;
      int cur_head = -1;
      for (int it = 0; it < n_items; ++it) {
        const Item w = ssd_item<MODE>(g, it, mt, c, head0);
        if (w.head != cur_head) {
          // (next) head: bring in its decay / dt factors; only these four warps read them, and the
          // TMA producer is already fetching tiles meanwhile
          if (cur_head >= 0) named_bar_sync(1, 128);
          for (int t = et; t < g.Q; t += 128) {
            const size_t o = (static_cast<size_t>(b) * g.H + w.head) * g.L + c * g.Q + t;
            s_cum[t] = g.cum[o];
            s_dt[t] = g.dtt[o];
          }
          named_bar_sync(1, 128);
          if (MODE == MODE_OUTPUT) { ssd_fill_colf(g, s_cum, s_dt, s_colf, et); named_bar_sync(1, 128); }
          cur_head = w.head;
        }
        if (!mbar_wait_abortable(full + s, phase, g.status, abort)) break;
        unsigned char* sa = smem + s * STAGE_BYTES;
        unsigned char* sb = sa + TILE_BYTES;
        const float* cm = s_cum;
        const float* dd = s_dt;
        if (MODE == MODE_STATES) {
          // scale k-row t of the B tile by w_t
          const float last = cm[g.Q - 1];
          for (int r = et; r < (tile_n / 64) * 64; r += 128) {
            const int t = w.kb * 64 + (r & 63);
            const float wt = g.anti ? ssd_exp(cm[t]) : ssd_exp(last - cm[t]) * dd[t];   // <= 1
            const __half2 wt2 = __float2half2_rn(wt);
            unsigned char* row = sb + (r >> 6) * BOX_BYTES + (r & 63) * 128;
#pragma unroll 1
            for (int qb = 0; qb < 8; qb += SSD_XF) {
              uint4 v[SSD_XF];
#pragma unroll
              for (int q = 0; q < SSD_XF; ++q) v[q] = *reinterpret_cast<uint4*>(row + (((qb + q) ^ (r & 7)) << 4));   // conflict-free
#pragma unroll
              for (int q = 0; q < SSD_XF; ++q) {
                __half2* h2 = reinterpret_cast<__half2*>(&v[q]);
#pragma unroll
                for (int e = 0; e < 4; ++e) h2[e] = __hmul2(h2[e], wt2);
              }
#pragma unroll
              for (int q = 0; q < SSD_XF; ++q) *reinterpret_cast<uint4*>(row + (((qb + q) ^ (r & 7)) << 4)) = v[q];
            }
          }
        } else {
          // row i of the K-major A tile (128 B): element j of the k-block sits in 16-byte chunk (j/8) ^ (i%8)
          const int i = mt * 128 + et;
          unsigned char* row = sa + et * 128;
          const float ci = cm[i];
          if (!w.off) {
            // F_ij = mask * exp(+-(cum_i - cum_j)) * (dt_j | dt_i) is split into a column factor
            // shared by the CTA and a row factor per thread, both relative to a reference
            // column of this k-block chosen so that the column factors never exceed one:
            //   causal: ref = last column,  colf_j = exp(cum_ref - cum_j) dt_j,  rowf_i = exp(cum_i - cum_ref)
            //   anti  : ref = first column, colf_j = exp(cum_j - cum_ref),       rowf_i = exp(cum_ref - cum_i) dt_i
            // (one exp per column and per row instead of one per element).  Rows inside the
            // k-block can have a positive row exponent; beyond 60 they take the direct form.
            const int jref = g.anti ? w.kb * 64 : w.kb * 64 + 63;
            const float cref = cm[jref];
            const float rarg = g.anti ? cref - ci : ci - cref;
            const bool direct = rarg > 60.f;
            const float rowf = direct ? 0.f : (g.anti ? ssd_exp(rarg) * dd[i] : ssd_exp(rarg));
            const float* colf = s_colf + w.kb * 64;
            const int sw = et & 7;
            const int iloc = i - w.kb * 64;              // this row relative to the first column of the k-block
            const int wlo = iloc - lane, whi = wlo + 31; // the warp's 32 consecutive rows
            if (__any_sync(0xffffffffu, direct)) {
              // rare: some row of the warp cannot use the factorised form
#pragma unroll 1
              for (int jc = 0; jc < 8; ++jc) {
                uint4 v = *reinterpret_cast<uint4*>(row + ((jc ^ sw) << 4));
                __half2* h2 = reinterpret_cast<__half2*>(&v);
                float cf[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const int jl = jc * 8 + e, j = w.kb * 64 + jl;
                  float f = direct ? (g.anti ? ssd_exp(cm[j] - ci) * dd[i] : ssd_exp(ci - cm[j]) * dd[j]) : colf[jl] * rowf;
                  if (g.anti ? (jl < iloc) : (jl > iloc)) f = 0.f;
                  cf[e] = f;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f = __half22float2(h2[e]);
                  h2[e] = __floats2half2_rn(f.x * cf[2 * e], f.y * cf[2 * e + 1]);
                }
                *reinterpret_cast<uint4*>(row + ((jc ^ sw) << 4)) = v;
              }
            } else {
              // Logical chunk jc (columns 8 jc .. 8 jc + 7) sits at physical chunk jc ^ (row % 8): the eight
              // rows of a quarter-warp touch eight different chunks, so the accesses are conflict-free and
              // the column factors are the same for the whole warp.  Four chunks at a time, loads first
              // (the tile is rewritten in place, which keeps the compiler from hoisting loads over stores).
#pragma unroll 1
              for (int qb = 0; qb < 8; qb += SSD_XF) {
                uint4 v[SSD_XF];
#pragma unroll
                for (int q = 0; q < SSD_XF; ++q) v[q] = *reinterpret_cast<uint4*>(row + (((qb + q) ^ sw) << 4));
#pragma unroll
                for (int q = 0; q < SSD_XF; ++q) {
                  const int jl = (qb + q) * 8;
                  // mask class of this chunk for the warp's rows (warp-uniform)
                  const bool all_zero = g.anti ? (jl + 7 < wlo) : (jl > whi);
                  const bool all_keep = g.anti ? (jl >= whi) : (jl + 7 <= wlo);
                  if (all_zero) {
                    v[q] = make_uint4(0u, 0u, 0u, 0u);
                  } else {
                    const float4 c0 = *reinterpret_cast<const float4*>(colf + jl);
                    const float4 c1 = *reinterpret_cast<const float4*>(colf + jl + 4);
                    float cf[8] = {c0.x * rowf, c0.y * rowf, c0.z * rowf, c0.w * rowf,
                                   c1.x * rowf, c1.y * rowf, c1.z * rowf, c1.w * rowf};
                    if (!all_keep) {
#pragma unroll
                      for (int e = 0; e < 8; ++e)
                        if (g.anti ? (jl + e < iloc) : (jl + e > iloc)) cf[e] = 0.f;
                    }
                    // the factor is formed in fp32 and rounded once; the product is a packed half multiply
                    __half2* h2 = reinterpret_cast<__half2*>(&v[q]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) h2[e] = __hmul2(h2[e], __floats2half2_rn(cf[2 * e], cf[2 * e + 1]));
                  }
                }
#pragma unroll
                for (int q = 0; q < SSD_XF; ++q) *reinterpret_cast<uint4*>(row + (((qb + q) ^ sw) << 4)) = v[q];
              }
            }
          } else {
            const float fi = g.anti ? ssd_exp(cm[g.Q - 1] - ci) * dd[i] : ssd_exp(ci);   // <= 1
            const __half2 fi2 = __float2half2_rn(fi);
#pragma unroll 1
            for (int qb = 0; qb < 8; qb += SSD_XF) {
              uint4 v[SSD_XF];
#pragma unroll
              for (int q = 0; q < SSD_XF; ++q) v[q] = *reinterpret_cast<uint4*>(row + (((qb + q) ^ (et & 7)) << 4));
#pragma unroll
              for (int q = 0; q < SSD_XF; ++q) {
                __half2* h2 = reinterpret_cast<__half2*>(&v[q]);
#pragma unroll
                for (int e = 0; e < 4; ++e) h2[e] = __hmul2(h2[e], fi2);
              }
#pragma unroll
              for (int q = 0; q < SSD_XF; ++q) *reinterpret_cast<uint4*>(row + (((qb + q) ^ (et & 7)) << 4)) = v[q];
            }
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(ready + s);
        if (++s == STAGES) { s = 0; phase ^= 1u; }
      }
    }
    const bool acc_ready = n_items > 0 ? mbar_wait_abortable(acc_full, 0, g.status, abort) : true;
    __syncwarp();
    if (acc_ready) {
      // The accumulator leaves through shared memory: every thread owns one row in TMEM, which as a
      // direct store would touch 32 different lines per instruction.  The pipeline stages are idle once
      // acc_full has fired, so the warp parks its 32 rows there (16-byte chunks XOR-swizzled by row,
      // conflict-free) and then writes them out with whole rows per instruction.
      tcgen05_fence_after_sync();
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;   // accumulator row of this thread
      const bool f32_out = MODE == MODE_STATES || (MODE == MODE_OUTPUT && g.part_out != nullptr);
      const int RB = tile_n * (f32_out ? 4 : 2);   // bytes of one staged row
      unsigned char* stg_row = smem + row * RB;
      const int cpr = RB >> 4;             // 16-byte chunks per row: 8, 16 or 32
      const int rpi = 32 / cpr;            // rows moved per warp instruction
      const int cc = lane % cpr;
      // Row dots <z, out> use the fp32 accumulator (u - v cancels downstream, so the rounded output
      // is not accurate enough): the z tile is parked behind the output tile with coalesced loads.
      const bool with_dot = MODE == MODE_OUTPUT && g.z != nullptr;
      unsigned char* zst = smem + 128 * RB;
      if (with_dot) {
#pragma unroll 4
        for (int rr = 0; rr < 32; rr += rpi) {
          const int lrow = quarter * 32 + rr + lane / cpr;
          const size_t trow = static_cast<size_t>(r0 + mt * 128 + lrow);
          *reinterpret_cast<uint4*>(zst + lrow * RB + ((cc ^ (lrow & 7)) << 4)) =
              *reinterpret_cast<const uint4*>(g.z + trow * g.z_pitch + unit * g.dv + cc * 8);
        }
        __syncwarp();
      }
      float dot = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < tile_n; c0 += 32) {
        uint32_t v[32];
        if (n_items > 0) {
          tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (f32_out) {
#pragma unroll
          for (int p = 0; p < 8; ++p)
            *reinterpret_cast<uint4*>(stg_row + (((c0 / 4 + p) ^ (row & 7)) << 4)) = make_uint4(v[p * 4], v[p * 4 + 1], v[p * 4 + 2], v[p * 4 + 3]);
        } else {
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __half2 h = __floats2half2_rn(__uint_as_float(v[p * 8 + 2 * e]), __uint_as_float(v[p * 8 + 2 * e + 1]));
              ow[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(stg_row + (((c0 / 8 + p) ^ (row & 7)) << 4)) = o;
            if (with_dot) {
              const uint4 zv = *reinterpret_cast<const uint4*>(zst + row * RB + (((c0 / 8 + p) ^ (row & 7)) << 4));
              const __half2* z2 = reinterpret_cast<const __half2*>(&zv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 zf = __half22float2(z2[e]);
                dot += zf.x * __uint_as_float(v[p * 8 + 2 * e]) + zf.y * __uint_as_float(v[p * 8 + 2 * e + 1]);
              }
            }
          }
        }
      }
      if (with_dot && g.dot_out != nullptr)
        g.dot_out[(static_cast<size_t>(b) * g.H + unit) * g.L + c * g.Q + mt * 128 + row] = dot;
      __syncwarp();
#pragma unroll 1
      for (int rr = 0; rr < 32; rr += rpi) {
        const int lrow = quarter * 32 + rr + lane / cpr;
        const uint4 val = *reinterpret_cast<const uint4*>(smem + lrow * RB + ((cc ^ (lrow & 7)) << 4));
        if (MODE == MODE_SCORES) {
          const int su = g.scores_head ? g.H : g.G;
          __half* dst = g.g_out + (static_cast<size_t>((b * g.nc + c) * su + unit) * g.Q + mt * 128 + lrow) * g.Q + nt * 128;
          *reinterpret_cast<uint4*>(dst + cc * 8) = val;
        } else if (MODE == MODE_STATES) {
          float* dst = g.s_out + (static_cast<size_t>((b * g.H + unit) * g.nc + c) * 128 + lrow) * tile_n;
          *reinterpret_cast<uint4*>(dst + cc * 4) = val;
        } else {
          const size_t trow = static_cast<size_t>(r0 + mt * 128 + lrow);
          if (g.part_out != nullptr) {
            float* dst = g.part_out + (static_cast<size_t>(blockIdx.x) * g.B * g.L + trow) * g.o_pitch + unit * g.dv;
            *reinterpret_cast<uint4*>(dst + cc * 4) = val;
          } else if (g.o_out != nullptr) {
            *reinterpret_cast<uint4*>(g.o_out + trow * g.o_pitch + unit * g.dv + cc * 8) = val;
          }
        }
      }
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_acc, g.tmem_cols);
}

// ---------------------------------------------------------------------------
// gdt, gA from u = <gy, y>, v = <gx, x> (both [B,H,L]).  With g_a_t the gradient of the loss with respect to
// dt_t A_h:  g_a_t = g_a_{t+1} + u_t - v_t,  gdt_t = v_t / dt_t + A_h g_a_t,  gA_h = sum_t dt_t g_a_t.
// u_t - v_t cancels and carries the rounding noise of two different operator instances, so a suffix sum over
// the whole sequence random-walks (measured: gA off by 5 % at 8192 steps).  The sum is therefore pinned at every
// chunk boundary to a value that has no such noise,
//     g_a at the first step of chunk c+1 = < state chunk c receives from its successors (anti-causal scan),
//                                            state chunk c+1 receives from its predecessors (causal scan) >,
// only summed inside a chunk, and the residual between the two pins of a chunk is spread linearly over its steps.
// ---------------------------------------------------------------------------
// pin[b,h,c] = < Hs_anti[b,h,c], Hs_causal[b,h,c+1] >  (0 for the last chunk); one CTA per (b, h, c)
__global__ void __launch_bounds__(256) ssd_boundary_dot_kernel(const __half* __restrict__ hs_anti, const __half* __restrict__ hs_causal,
                                                               float* __restrict__ pin, int nc, int E) {
  __shared__ float red[8];
  const int c = blockIdx.x % nc;
  const size_t bh = blockIdx.x / nc;
  float acc = 0.f;
  if (c + 1 < nc) {
    const __half2* a = reinterpret_cast<const __half2*>(hs_anti + (bh * nc + c) * static_cast<size_t>(E));
    const __half2* f = reinterpret_cast<const __half2*>(hs_causal + (bh * nc + c + 1) * static_cast<size_t>(E));
    for (int i = threadIdx.x; i < E / 2; i += 256) {
      const float2 x = __half22float2(a[i]), y = __half22float2(f[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  acc = warp_reduce<SumOp>(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    pin[blockIdx.x] = t;
  }
}

// One CTA per (b, h); one thread per step of a chunk (Q <= 256), chunks walked from the last to the first.
// `halves` = 2: u and v are the sums of two arrays, the second `B*H*L` elements after the first.
// With `raw` (the projection's raw step sizes, r16, pitched) the reverse of dt = softplus(raw + bias[h]) is applied on the
// way out: graw = gdt * sigmoid(raw + bias) (r16, pitched), gbias[h] += its sum (the arithmetic of launch_softplus_bias_reverse).
__device__ __forceinline__ float ssd_sigmoid(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return r;
}
__global__ void __launch_bounds__(256) ssd_scalar_grads_kernel(const float* __restrict__ u, const float* __restrict__ v,
                                                               const float* __restrict__ dtt, const float* __restrict__ A,
                                                               const float* __restrict__ pin, float* __restrict__ gdt,
                                                               float* __restrict__ gA_part, int B, int L, int H, int Q, int halves,
                                                               const __half* __restrict__ raw = nullptr, size_t raw_pitch = 0,
                                                               const float* __restrict__ bias = nullptr, __half* __restrict__ graw = nullptr,
                                                               size_t graw_pitch = 0, float* __restrict__ gbias = nullptr) {
  __shared__ float warp_tot[8];
  __shared__ float total_s;
  __shared__ float ga_red[8];
  __shared__ float gb_red[8];
  float gb_acc = 0.f;
  const int h = blockIdx.x % H, b = blockIdx.x / H;
  const size_t base = (static_cast<size_t>(b) * H + h) * L;
  const int nc = L / Q;
  const float Ah = A[h];
  float ga_acc = 0.f;
  for (int c = nc - 1; c >= 0; --c) {
    const int j = static_cast<int>(threadIdx.x);           // thread 0 holds the latest step of the chunk
    const int t = c * Q + (Q - 1 - j);
    const bool in = j < Q;
    const size_t hs = static_cast<size_t>(B) * H * L;
    float ut = 0.f, vt = 0.f;
    if (in) {
      ut = u[base + t]; vt = v[base + t];
      if (halves == 2) { ut += u[hs + base + t]; vt += v[hs + base + t]; }
    }
    const float d = ut - vt;
    float s = d;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, s, off);
      if ((threadIdx.x & 31) >= off) s += n;
    }
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = s;
    __syncthreads();
    float wb = 0.f;
    for (int w = 0; w < static_cast<int>(threadIdx.x >> 5); ++w) wb += warp_tot[w];
    const float within = s + wb;                            // sum over the chunk's steps t' >= t
    if (j == Q - 1) total_s = within;                       // the whole chunk
    __syncthreads();
    const float right = pin[(static_cast<size_t>(b) * H + h) * nc + c];          // g_a just after the chunk
    float resid = 0.f;
    if (c > 0) resid = pin[(static_cast<size_t>(b) * H + h) * nc + c - 1] - (right + total_s);   // what the first step should reach
    if (in) {
      const float ga = right + within + resid * (static_cast<float>(j + 1) / static_cast<float>(Q));
      const float dtv = dtt[base + t];
      const float gd = vt / dtv + Ah * ga;
      const size_t row = static_cast<size_t>(b) * L + t;
      gdt[row * H + h] = gd;
      ga_acc += dtv * ga;
      if (raw != nullptr) {
        const float gr = gd * ssd_sigmoid(__half2float(raw[row * raw_pitch + h]) + bias[h]);
        graw[row * graw_pitch + h] = __float2half_rn(gr);
        gb_acc += gr;
      }
    }
    __syncthreads();
  }
  ga_acc = warp_reduce<SumOp>(ga_acc);
  gb_acc = warp_reduce<SumOp>(gb_acc);
  if ((threadIdx.x & 31) == 0) { ga_red[threadIdx.x >> 5] = ga_acc; gb_red[threadIdx.x >> 5] = gb_acc; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f, tb = 0.f;
    for (int w = 0; w < 8; ++w) { t += ga_red[w]; tb += gb_red[w]; }
    gA_part[blockIdx.x] = t;
    if (raw != nullptr && gbias != nullptr) atomicAdd(gbias + h, tb);
  }
}

// out[i] = sum_s part[s][i] rounded to r16 (fold of the per-group partial outputs), 8 elements per thread
__global__ void __launch_bounds__(256) ssd_fold_parts_kernel(const float* __restrict__ part, __half* __restrict__ out, size_t n,
                                                             int splits) {
  const size_t i = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  if (i >= n) return;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int sidx = 0; sidx < splits; ++sidx) {
    const float4 a = *reinterpret_cast<const float4*>(part + sidx * n + i);
    const float4 b = *reinterpret_cast<const float4*>(part + sidx * n + i + 4);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  st_pack(out + i, 0, pack<__half>(acc));
}

// gA[h] = sum over the batch; with A_log's gradient wanted (A = -exp(A_log), so dA / dA_log = A): gA_log[h] += gA[h] * A[h]
__global__ void ssd_sum_batches_kernel(const float* __restrict__ part, float* __restrict__ gA, int B, int H,
                                       const float* __restrict__ A = nullptr, float* __restrict__ gA_log = nullptr) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int b = 0; b < B; ++b) s += part[b * H + h];
  gA[h] = s;
  if (gA_log != nullptr) gA_log[h] += s * A[h];
}

// ---------------------------------------------------------------------------
// Host side.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn ssd_encode_tiled() {
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

// r16 matrix [rows, cols] (row-major, pitch = cols), box {64, box_rows}, 128-byte swizzle
CUtensorMap ssd_map(const void* base, size_t rows, size_t cols, uint32_t box_rows) {
  CUtensorMap m;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * sizeof(__half)};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t es[2] = {1, 1};
  MP_CU_CHECK(ssd_encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return m;
}

struct SsdDims { int B, L, H, P, N, G, Q, nc; };

// CTAs that share the heads of one group when an output is summed over them (gB, gC): with one CTA per
// group and tile only B * L / 128 * G CTAs would exist, each walking all the group's heads in sequence.
// The split count (a divisor of the heads per group, at most 32) minimises
//   waves of resident CTAs x (k-blocks per CTA + a fixed cost per CTA)
// with three CTAs of these launches resident per SM (68 KB of shared memory each).
// SM count of the current device; 148 (a B200) where no device can be queried, so that scratch sizes can be computed
// on a machine without a GPU.
int ssd_sm_count() {
  int device = 0, n = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    return 148;
  }
  return n;
}

int ssd_head_splits(const SsdDims& d, int sm_count) {
  const int hpg = d.H / d.G;
  const long base = 2L * d.B * d.nc * d.G * (d.Q / 128) / 2 * 1;   // tiles of one split: B * nc * G * (Q / 128)
  const long slots = static_cast<long>(sm_count > 0 ? sm_count : 148) * 3;
  int best = 1;
  long best_cost = -1;
  for (int sp = 1; sp <= hpg && sp <= 32; ++sp) {
    if (hpg % sp != 0) continue;
    const long waves = (base * sp + slots - 1) / slots;
    const long cost = waves * (static_cast<long>(hpg / sp) * 5 + 2);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = sp; }
  }
  return best;
}

// Scratch layout (bytes, 256-aligned sections).
struct SsdScratch {
  float* cum; float* dtt; __half* scores; float* states; __half* hs; float* u; float* v; float* ga_part; float* parts; float* pin;
  // reverse: the four operator instances run side by side, each with its own scores / states / partials
  __half* scores_op[4]; float* states_op[4]; __half* hs_op[4]; float* parts_op[4];
  size_t total;
};
SsdScratch ssd_carve(void* base, const SsdDims& d, bool reverse) {
  SsdScratch s;
  size_t off = 0;
  auto take = [&](size_t bytes) { void* p = base ? static_cast<unsigned char*>(base) + off : nullptr; off += (bytes + 255) & ~size_t(255); return p; };
  const size_t bhl = static_cast<size_t>(d.B) * d.H * d.L;
  s.cum = static_cast<float*>(take(bhl * 4));
  s.dtt = static_cast<float*>(take(bhl * 4));
  const size_t st = static_cast<size_t>(d.B) * d.H * d.nc * 128 * 128;   // upper bound on dk*dv
  const size_t group_scores = static_cast<size_t>(d.B) * d.nc * d.G * d.Q * d.Q * 2;
  const size_t head_scores = static_cast<size_t>(d.B) * d.nc * d.H * d.Q * d.Q * 2;   // gB / gC keep per-head scores
  const size_t parts_bytes = static_cast<size_t>(ssd_head_splits(d, ssd_sm_count())) * d.B * d.L * d.G * d.N * 4;
  for (int op = 0; op < (reverse ? 4 : 1); ++op) {
    const bool per_head = reverse && op >= 2;   // operators 2, 3 = gC, gB
    s.scores_op[op] = static_cast<__half*>(take(per_head ? head_scores : group_scores));
    s.states_op[op] = static_cast<float*>(take(st * 4));
    s.hs_op[op] = static_cast<__half*>(take(st * 2));
    s.parts_op[op] = static_cast<float*>(take(per_head ? parts_bytes : 0));
  }
  s.scores = s.scores_op[0]; s.states = s.states_op[0]; s.hs = s.hs_op[0]; s.parts = s.parts_op[0];
  s.u = static_cast<float*>(take(reverse ? bhl * 4 : 0));
  s.v = static_cast<float*>(take(reverse ? bhl * 4 : 0));
  s.ga_part = static_cast<float*>(take(reverse ? static_cast<size_t>(d.B) * d.H * 4 : 0));
  s.pin = static_cast<float*>(take(reverse ? static_cast<size_t>(d.B) * d.H * d.nc * 4 : 0));
  s.total = off;
  return s;
}

struct Roles {
  const __half* q; int q_head;   // [B*L, units*dk]
  const __half* k; int k_head;
  const __half* v; int v_head;   // [B*L, units*dv]
  int dk, dv, anti, scores_head, out_head;
  __half* out; const __half* z; float* dot;
};

template <int MODE>
void ssd_launch(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1, const CUtensorMap& b1, const SsdArgs& g,
                dim3 grid, size_t smem, cudaStream_t st) {
  MP_CUDA_CHECK(cudaFuncSetAttribute(ssd_mma_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  ssd_mma_kernel<MODE><<<grid, SSD_THREADS, smem, st>>>(a0, b0, a1, b1, g);
  MP_LAUNCH_CHECK();
}

// One instance of the chunked operator (scores -> states -> scan -> output).
// `sub` (may be null): a second stream on which the scores kernel runs beside the states + scan chain; `fork`
// and `join` are the events that order it against `st`.
void ssd_operator(const SsdDims& d, const Roles& r, const SsdScratch& sc, uint32_t* status, cudaStream_t st,
                  cudaStream_t sub = nullptr, cudaEvent_t fork = nullptr, cudaEvent_t join = nullptr) {
  SsdArgs g;
  g.B = d.B; g.L = d.L; g.H = d.H; g.G = d.G; g.Q = d.Q; g.nc = d.nc;
  g.dk = r.dk; g.dv = r.dv; g.anti = r.anti;
  g.q_head = r.q_head; g.k_head = r.k_head; g.v_head = r.v_head;
  g.scores_head = r.scores_head; g.out_head = r.out_head;
  g.state_t = r.dk == 128 ? 0 : 1;
  g.cum = sc.cum; g.dtt = sc.dtt;
  g.g_out = sc.scores; g.s_out = sc.states;
  g.o_out = r.out; g.o_pitch = (r.out_head ? d.H : d.G) * r.dv;
  g.z = r.z; g.z_pitch = g.o_pitch; g.dot_out = r.dot;
  g.status = status;
  g.part_out = nullptr; g.head_splits = 1;
  const size_t rows = static_cast<size_t>(d.B) * d.L;
  const size_t qcols = static_cast<size_t>(r.q_head ? d.H : d.G) * r.dk;
  const size_t kcols = static_cast<size_t>(r.k_head ? d.H : d.G) * r.dk;
  const size_t vcols = static_cast<size_t>(r.v_head ? d.H : d.G) * r.dv;
  // Shared memory per CTA is kept near 50-70 KB so that three or four CTAs share an SM: every CTA has
  // only a handful of k-blocks, so latency is hidden across CTAs rather than by a deep pipeline.
  auto configure = [&](int b_tile_bytes, int tile_cols, int stages = 2) {
    g.stage_bytes = TILE_BYTES + b_tile_bytes;
    g.stages = stages;
    g.tmem_cols = tile_cols <= 32 ? 32 : (tile_cols <= 64 ? 64 : 128);
    return static_cast<size_t>(g.stages) * g.stage_bytes + 1024 + 256 + 3 * d.Q * 4;
  };
  const int sunits = r.scores_head ? d.H : d.G;
  const int d2 = r.dk == 128 ? r.dv : r.dk;   // columns of a stored state block ([128][d2])

  // scores: q (K-major 128-row boxes) x k^T
  {
    const CUtensorMap mq = ssd_map(r.q, rows, qcols, 128), mk = ssd_map(r.k, rows, kcols, 128);
    const dim3 grid(d.Q / 128, d.Q / 128, d.B * d.nc * sunits);
    // one k-block per tile when dk = 64 (per-head scores): a single stage, so that four CTAs fit an SM
    const size_t smem = configure(TILE_BYTES, 128, r.dk / 64 == 1 ? 1 : 2);
    if (sub != nullptr) {
      MP_CUDA_CHECK(cudaEventRecord(fork, st));
      MP_CUDA_CHECK(cudaStreamWaitEvent(sub, fork, 0));
      ssd_launch<MODE_SCORES>(mq, mk, mq, mk, g, grid, smem, sub);
      MP_CUDA_CHECK(cudaEventRecord(join, sub));
    } else {
      ssd_launch<MODE_SCORES>(mq, mk, mq, mk, g, grid, smem, st);
    }
  }
  // chunk states: MN-major 64x64 boxes of k and v
  {
    const CUtensorMap mk = ssd_map(r.k, rows, kcols, 64), mv = ssd_map(r.v, rows, vcols, 64);
    const dim3 grid(1, 1, d.B * d.nc * d.H);
    const size_t smem = configure((d2 / 64) * BOX_BYTES, d2);
    ssd_launch<MODE_STATES>(mk, mv, mk, mv, g, grid, smem, st);
  }
  {
    const int E = 128 * d2;
    const dim3 grid((E + 255) / 256, d.B * d.H);
    ssd_scan_kernel<<<grid, 256, 0, st>>>(sc.states, sc.hs, sc.cum, d.nc, d.Q, E, r.anti);
    MP_LAUNCH_CHECK();
  }
  // output
  if (sub != nullptr) MP_CUDA_CHECK(cudaStreamWaitEvent(st, join, 0));
  {
    const CUtensorMap ms = ssd_map(sc.scores, static_cast<size_t>(d.B) * d.nc * sunits * d.Q, d.Q, 128);
    const CUtensorMap mv = ssd_map(r.v, rows, vcols, 64);
    const CUtensorMap mq = ssd_map(r.q, rows, qcols, 128);
    const size_t srows = static_cast<size_t>(d.B) * d.H * d.nc * 128;
    const CUtensorMap mh = g.state_t ? ssd_map(sc.hs, srows, d2, 128) : ssd_map(sc.hs, srows, d2, 64);
    const int units = r.out_head ? d.H : d.G;
    const int splits = r.out_head ? 1 : ssd_head_splits(d, ssd_sm_count());
    g.head_splits = splits;
    g.part_out = splits > 1 ? sc.parts : nullptr;
    const dim3 grid(splits, d.Q / 128, d.B * d.nc * units);
    const size_t smem = configure(g.state_t ? TILE_BYTES : (r.dv / 64) * BOX_BYTES, r.dv);
    ssd_launch<MODE_OUTPUT>(ms, mv, mq, mh, g, grid, smem, st);
    if (splits > 1) {
      const size_t n = static_cast<size_t>(d.B) * d.L * d.G * r.dv;
      ssd_fold_parts_kernel<<<static_cast<unsigned>((n / 8 + 255) / 256), 256, 0, st>>>(sc.parts, r.out, n, splits);
      MP_LAUNCH_CHECK();
    }
    g.head_splits = 1; g.part_out = nullptr;
  }
}

// Shapes the tensor-core path covers; everything else takes the sequential-recurrence kernels of ssd_generic.cu.
bool ssd_tensor_path(const SsdDims& d) {
  if (d.G <= 0 || d.H % d.G != 0) MP_FATAL("ssd_scan: heads %d not divisible by groups %d", d.H, d.G);
  return d.N == 128 && (d.P == 64 || d.P == 128) && (d.Q == 128 || d.Q == 256) && d.L % d.Q == 0 &&
         getenv("MP_SSD_FORCE_GENERIC") == nullptr;
}

SsdDims ssd_dims(len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk) {
  SsdDims d;
  d.B = static_cast<int>(batch); d.L = static_cast<int>(seqlen); d.H = static_cast<int>(heads);
  d.P = static_cast<int>(headdim); d.N = static_cast<int>(dstate); d.G = static_cast<int>(ngroups);
  d.Q = static_cast<int>(chunk); d.nc = d.Q > 0 ? d.L / d.Q : 0;
  return d;
}

}  // namespace

extern "C" len_t mpSsdScanGenericScratchBytes(uint32_t dtype_key, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate,
                                              len_t ngroups, uint32_t reverse);
void mp_ssd_generic_forward_r16(const void* x, const void* dt, const void* A, const void* B, const void* C, void* y, len_t batch, len_t seqlen,
                                len_t heads, len_t headdim, len_t dstate, len_t ngroups, StreamContext ctx);
void mp_ssd_generic_reverse_r16(const void* x, const void* dt, const void* A, const void* B, const void* C, const void* gy, void* gx, void* gdt,
                                void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim,
                                len_t dstate, len_t ngroups, StreamContext ctx);

// chunk-walk kernels (ssd_walk.cu)
bool mp_ssd_walk_supported(int L, int H, int P, int N, int G);
void mp_ssd_walk_cumsum(const float* dt, const float* A, float* cum, float* dtt, float* colf_c, float* colf_a, int B, int L, int H,
                        int* carry_flags, int n_flags, cudaStream_t st);
void mp_ssd_walk_cumsum_raw(const __half* raw, size_t raw_pitch, const float* bias, const float* A_log, float* dt_out, float* A_out, float* cum,
                            float* dtt, float* colf_c, int B, int L, int H, int* carry_flags, int n_flags, cudaStream_t st);
void mp_ssd_walk(int anti, const __half* q, const __half* k, const __half* v, const float* cum, const float* dtt, const float* colf, __half* out,
                 const __half* z, float* dot_out, __half* hs_out, float* carry, int* carry_flag, int max_ctas, int B, int L, int H, int G,
                 uint32_t* status, cudaStream_t st);

void mp_ssd_group_grads(const __half* gy, const __half* x, const __half* Bm, const __half* Cm, const __half* hs_causal, const __half* hs_anti,
                        const float* cum, const float* dtt, const float* colf_c, __half* gB, __half* gC, int B, int L, int H, int G,
                        uint32_t* status, cudaStream_t st);

namespace {
// Scratch of the walk path: prefix sums and dt in [B,H,L] order; for the reverse also the states every 128-step
// chunk receives from its predecessors and from its successors (r16 [B,H,L/128][128][64]).
struct WalkScratch { float* cum; float* dtt; float* colf_c; float* colf_a; __half* hs_causal; __half* hs_anti; float* pin; float* u; float* v; float* ga_part; float* carry_c; float* carry_a; int* flags; size_t total; };
WalkScratch walk_carve(void* base, const SsdDims& d, bool reverse, size_t off0) {
  WalkScratch w;
  size_t off = off0;
  auto take = [&](size_t bytes) { void* p = base ? static_cast<unsigned char*>(base) + off : nullptr; off += (bytes + 255) & ~size_t(255); return p; };
  const size_t bhl = static_cast<size_t>(d.B) * d.H * d.L;
  w.cum = static_cast<float*>(take(bhl * 4));
  w.dtt = static_cast<float*>(take(bhl * 4));
  w.colf_c = static_cast<float*>(take(bhl * 4));
  w.colf_a = static_cast<float*>(take(reverse ? bhl * 4 : 0));
  const size_t st = static_cast<size_t>(d.B) * d.H * (d.L / 128) * 128 * 64 * 2;
  w.hs_causal = static_cast<__half*>(take(reverse ? st : 0));
  w.hs_anti = static_cast<__half*>(take(reverse ? st : 0));
  w.pin = static_cast<float*>(take(reverse ? static_cast<size_t>(d.B) * d.H * (d.L / 128) * 4 : 0));
  w.u = static_cast<float*>(take(reverse ? 2 * bhl * 4 : 0));     // one array per half of the columns
  w.v = static_cast<float*>(take(reverse ? 2 * bhl * 4 : 0));
  w.ga_part = static_cast<float*>(take(reverse ? static_cast<size_t>(d.B) * d.H * 4 : 0));
  // states handed from CTA to CTA inside a walk (fp32 [128][64] per sequence and walk) and their arrival counters
  const size_t carry = static_cast<size_t>(d.B) * d.H * 128 * 64 * 4;
  w.carry_c = static_cast<float*>(take(carry));
  w.carry_a = static_cast<float*>(take(reverse ? carry : 0));
  w.flags = static_cast<int*>(take(2 * static_cast<size_t>(d.B) * d.H * 4));
  w.total = off;
  return w;
}
}  // namespace

// r16 storage (for r32 / r64 see mpSsdScanGenericScratchBytes)
extern "C" len_t mpSsdScanScratchBytes(len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups,
                                       len_t chunk, uint32_t reverse) {
  const SsdDims d = ssd_dims(batch, seqlen, heads, headdim, dstate, ngroups, chunk);
  if (batch == 0 || seqlen == 0 || heads == 0) return 256;
  if (!ssd_tensor_path(d)) return mpSsdScanGenericScratchBytes(0, batch, seqlen, heads, headdim, dstate, ngroups, reverse);
  if (mp_ssd_walk_supported(d.L, d.H, d.P, d.N, d.G)) {
    if (reverse != 0) return walk_carve(nullptr, d, true, 0).total;
    // (the three-phase forward, an A/B switch, needs its own larger scratch: ask with the switch set)
    return getenv("MP_SSD_LEGACY_FORWARD") == nullptr ? walk_carve(nullptr, d, false, 0).total : ssd_carve(nullptr, d, false).total;
  }
  return ssd_carve(nullptr, d, reverse != 0).total;
}

// y = SSD(x, dt, A, B, C).  x, y: [batch, seqlen, heads, headdim] r16; dt: [batch, seqlen, heads] r32 (after
// softplus); A: [heads] r32 (negative); B, C: [batch, seqlen, ngroups, dstate] r16.
extern "C" void launch_ssd_scan_r16(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm, void* y,
                                    void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate,
                                    len_t ngroups, len_t chunk, StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  const SsdDims d = ssd_dims(batch, seqlen, heads, headdim, dstate, ngroups, chunk);
  if (!ssd_tensor_path(d)) {
    mp_ssd_generic_forward_r16(x, dt, A, Bm, Cm, y, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
    return;
  }
  if (scratch == nullptr) MP_FATAL("ssd_scan: scratch must not be NULL");
  MpStreamState* state = mp_state(ctx);
  cudaStream_t st = mp_stream(ctx);
  // The chunk walk (no chunk state in global memory) where it applies; MP_SSD_LEGACY_FORWARD selects the three-phase
  // path (scores, chunk states, scan, output as separate kernels), which also serves head size 128.
  if (mp_ssd_walk_supported(d.L, d.H, d.P, d.N, d.G) && getenv("MP_SSD_LEGACY_FORWARD") == nullptr) {
    const WalkScratch w = walk_carve(scratch, d, false, 0);
    mp_ssd_walk_cumsum(static_cast<const float*>(dt), static_cast<const float*>(A), w.cum, w.dtt, w.colf_c, nullptr, d.B, d.L, d.H, w.flags,
                       2 * d.B * d.H, st);
    mp_ssd_walk(0, static_cast<const __half*>(Cm), static_cast<const __half*>(Bm), static_cast<const __half*>(x), w.cum, w.dtt, w.colf_c,
                static_cast<__half*>(y), nullptr, nullptr, nullptr, w.carry_c, w.flags, state->sm_count, d.B, d.L, d.H, d.G, state->status_dev,
                st);
    return;
  }
  const SsdScratch sc = ssd_carve(scratch, d, false);
  ssd_cumsum_kernel<<<d.B * d.H * d.nc, 256, 0, st>>>(static_cast<const float*>(dt), static_cast<const float*>(A), sc.cum, sc.dtt,
                                                     d.B, d.L, d.H, d.Q);
  MP_LAUNCH_CHECK();
  Roles r;
  r.q = static_cast<const __half*>(Cm); r.q_head = 0;
  r.k = static_cast<const __half*>(Bm); r.k_head = 0;
  r.v = static_cast<const __half*>(x); r.v_head = 1;
  r.dk = d.N; r.dv = d.P; r.anti = 0; r.scores_head = 0; r.out_head = 1;
  r.out = static_cast<__half*>(y); r.z = nullptr; r.dot = nullptr;
  if (getenv("MP_SSD_SERIAL") == nullptr) {
    mp_aux_init(state);
    ssd_operator(d, r, sc, state->status_dev, st, state->aux_stream[3], state->aux_sub_fork[0], state->aux_join[3]);
  } else {
    ssd_operator(d, r, sc, state->status_dev, st);
  }
}

// Forward scan from the projection's raw outputs: dt = softplus(dt_raw + dt_bias[h]) and A = -exp(A_log[h]) are formed
// inside the prefix-sum kernel of the chunk walk (two launches less per call) and left in dt_out [batch, seqlen, heads]
// and A_out [heads] for launch_ssd_scan_reverse.  Elsewhere: launch_softplus_bias, launch_neg_exp, launch_ssd_scan.
extern "C" void launch_softplus_bias_r16(const void*, len_t, const void*, void*, len_t, len_t, StreamContext);
extern "C" void launch_softplus_bias_r32(const void*, len_t, const void*, void*, len_t, len_t, StreamContext);
extern "C" void launch_softplus_bias_r64(const void*, len_t, const void*, void*, len_t, len_t, StreamContext);
extern "C" void launch_neg_exp_r32(const void*, void*, len_t, StreamContext);
extern "C" void launch_neg_exp_r64(const void*, void*, len_t, StreamContext);
extern "C" void launch_ssd_scan_r32(const void*, const void*, const void*, const void*, const void*, void*, void*, len_t, len_t, len_t, len_t, len_t,
                                    len_t, len_t, StreamContext);
extern "C" void launch_ssd_scan_r64(const void*, const void*, const void*, const void*, const void*, void*, void*, len_t, len_t, len_t, len_t, len_t,
                                    len_t, len_t, StreamContext);

extern "C" void launch_ssd_scan_raw_r16(const void* x, const void* dt_raw, len_t dt_pitch, const void* dt_bias, const void* A_log, const void* Bm,
                                        const void* Cm, void* y, void* dt_out, void* A_out, void* scratch, len_t batch, len_t seqlen, len_t heads,
                                        len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  const SsdDims d = ssd_dims(batch, seqlen, heads, headdim, dstate, ngroups, chunk);
  if (ssd_tensor_path(d) && mp_ssd_walk_supported(d.L, d.H, d.P, d.N, d.G) && getenv("MP_SSD_LEGACY_FORWARD") == nullptr) {
    if (scratch == nullptr) MP_FATAL("ssd_scan_raw: scratch must not be NULL");
    MpStreamState* state = mp_state(ctx);
    cudaStream_t st = mp_stream(ctx);
    const WalkScratch w = walk_carve(scratch, d, false, 0);
    mp_ssd_walk_cumsum_raw(static_cast<const __half*>(dt_raw), dt_pitch, static_cast<const float*>(dt_bias), static_cast<const float*>(A_log),
                           static_cast<float*>(dt_out), static_cast<float*>(A_out), w.cum, w.dtt, w.colf_c, d.B, d.L, d.H, w.flags, 2 * d.B * d.H, st);
    mp_ssd_walk(0, static_cast<const __half*>(Cm), static_cast<const __half*>(Bm), static_cast<const __half*>(x), w.cum, w.dtt, w.colf_c,
                static_cast<__half*>(y), nullptr, nullptr, nullptr, w.carry_c, w.flags, state->sm_count, d.B, d.L, d.H, d.G, state->status_dev,
                st);
    return;
  }
  launch_softplus_bias_r16(dt_raw, dt_pitch, dt_bias, dt_out, batch * seqlen, heads, ctx);
  launch_neg_exp_r32(A_log, A_out, heads, ctx);
  launch_ssd_scan_r16(x, dt_out, A_out, Bm, Cm, y, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx);
}
extern "C" void launch_ssd_scan_raw_r32(const void* x, const void* dt_raw, len_t dt_pitch, const void* dt_bias, const void* A_log, const void* Bm,
                                        const void* Cm, void* y, void* dt_out, void* A_out, void* scratch, len_t batch, len_t seqlen, len_t heads,
                                        len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  launch_softplus_bias_r32(dt_raw, dt_pitch, dt_bias, dt_out, batch * seqlen, heads, ctx);
  launch_neg_exp_r32(A_log, A_out, heads, ctx);
  launch_ssd_scan_r32(x, dt_out, A_out, Bm, Cm, y, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx);
}
extern "C" void launch_ssd_scan_raw_r64(const void* x, const void* dt_raw, len_t dt_pitch, const void* dt_bias, const void* A_log, const void* Bm,
                                        const void* Cm, void* y, void* dt_out, void* A_out, void* scratch, len_t batch, len_t seqlen, len_t heads,
                                        len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  launch_softplus_bias_r64(dt_raw, dt_pitch, dt_bias, dt_out, batch * seqlen, heads, ctx);
  launch_neg_exp_r64(A_log, A_out, heads, ctx);
  launch_ssd_scan_r64(x, dt_out, A_out, Bm, Cm, y, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx);
}

// Gradients of a loss with upstream gradient gy (same shape as y); every output is overwritten.
// gx: like x; gdt: like dt (r32); gA: [heads] r32; gB, gC: like B, C.
namespace {
struct RawSide { const __half* raw; size_t raw_pitch; const float* bias; __half* graw; size_t graw_pitch; float* gbias; float* gA_log; };
}
static bool ssd_scan_reverse_r16_impl(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm, const void* gy, void* gx,
                                      void* gdt, void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads,
                                      len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx, const RawSide* rs);

extern "C" void launch_ssd_scan_reverse_r16(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm,
                                            const void* gy, void* gx, void* gdt, void* gA, void* gB, void* gC, void* scratch,
                                            len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups,
                                            len_t chunk, StreamContext ctx) {
  ssd_scan_reverse_r16_impl(x, dt, A, Bm, Cm, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx,
                            nullptr);
}

// Returns true when the raw-side gradients (rs) were produced inside the scan's own kernels.
static bool ssd_scan_reverse_r16_impl(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm, const void* gy, void* gx,
                                      void* gdt, void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads,
                                      len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx, const RawSide* rs) {
  if (batch == 0 || seqlen == 0 || heads == 0) return true;
  const SsdDims d = ssd_dims(batch, seqlen, heads, headdim, dstate, ngroups, chunk);
  if (!ssd_tensor_path(d)) {
    mp_ssd_generic_reverse_r16(x, dt, A, Bm, Cm, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
    return false;
  }
  if (scratch == nullptr) MP_FATAL("ssd_scan_reverse: scratch must not be NULL");
  MpStreamState* state = mp_state(ctx);
  cudaStream_t st = mp_stream(ctx);
  const __half* xh = static_cast<const __half*>(x);
  const __half* bh = static_cast<const __half*>(Bm);
  const __half* ch = static_cast<const __half*>(Cm);
  const __half* gyh = static_cast<const __half*>(gy);
  if (mp_ssd_walk_supported(d.L, d.H, d.P, d.N, d.G)) {
    // Two chunk walks side by side (anti-causal: gx and the row dots <gx, x>; causal: the row dots <gy, y>), both
    // leaving the states every 128-step chunk receives; then gB / gC from those states, and gdt / gA.
    const WalkScratch w = walk_carve(scratch, d, true, 0);
    const bool side = getenv("MP_SSD_SERIAL") == nullptr;
    cudaStream_t lane1 = st;
    mp_ssd_walk_cumsum(static_cast<const float*>(dt), static_cast<const float*>(A), w.cum, w.dtt, w.colf_c, w.colf_a, d.B, d.L, d.H, w.flags,
                       2 * d.B * d.H, st);
    // side by side each walk takes half of the SMs (a CTA fills an SM), one after the other all of them
    const int walk_ctas = side ? state->sm_count / 2 : state->sm_count;
    if (side) {
      mp_aux_init(state);
      lane1 = state->aux_stream[0];
      MP_CUDA_CHECK(cudaEventRecord(state->aux_fork, st));
      MP_CUDA_CHECK(cudaStreamWaitEvent(lane1, state->aux_fork, 0));
    }
    mp_ssd_walk(1, bh, ch, gyh, w.cum, w.dtt, w.colf_a, static_cast<__half*>(gx), xh, w.v, w.hs_anti, w.carry_a, w.flags + d.B * d.H, walk_ctas,
                d.B, d.L, d.H, d.G, state->status_dev, st);
    mp_ssd_walk(0, ch, bh, xh, w.cum, w.dtt, w.colf_c, nullptr, gyh, w.u, w.hs_causal, w.carry_c, w.flags, walk_ctas, d.B, d.L, d.H, d.G,
                state->status_dev, lane1);
    if (side) {
      MP_CUDA_CHECK(cudaEventRecord(state->aux_join[0], lane1));
      MP_CUDA_CHECK(cudaStreamWaitEvent(st, state->aux_join[0], 0));
      // gdt / gA need both walks (u, v, states) but not gB / gC: they run beside the group-gradient kernel
      MP_CUDA_CHECK(cudaEventRecord(state->aux_sub_fork[0], st));
      MP_CUDA_CHECK(cudaStreamWaitEvent(lane1, state->aux_sub_fork[0], 0));
    }
    mp_ssd_group_grads(gyh, xh, bh, ch, w.hs_causal, w.hs_anti, w.cum, w.dtt, w.colf_c, static_cast<__half*>(gB), static_cast<__half*>(gC),
                       d.B, d.L, d.H, d.G, state->status_dev, st);
    const int wnc = d.L / 128;
    ssd_boundary_dot_kernel<<<d.B * d.H * wnc, 256, 0, lane1>>>(w.hs_anti, w.hs_causal, w.pin, wnc, d.N * d.P);
    MP_LAUNCH_CHECK();
    if (rs != nullptr)
      ssd_scalar_grads_kernel<<<d.B * d.H, 256, 0, lane1>>>(w.u, w.v, w.dtt, static_cast<const float*>(A), w.pin, static_cast<float*>(gdt), w.ga_part,
                                                           d.B, d.L, d.H, 128, 2, rs->raw, rs->raw_pitch, rs->bias, rs->graw, rs->graw_pitch,
                                                           rs->gbias);
    else
      ssd_scalar_grads_kernel<<<d.B * d.H, 256, 0, lane1>>>(w.u, w.v, w.dtt, static_cast<const float*>(A), w.pin, static_cast<float*>(gdt), w.ga_part,
                                                           d.B, d.L, d.H, 128, 2);
    MP_LAUNCH_CHECK();
    ssd_sum_batches_kernel<<<(d.H + 127) / 128, 128, 0, lane1>>>(w.ga_part, static_cast<float*>(gA), d.B, d.H, static_cast<const float*>(A),
                                                                 rs != nullptr ? rs->gA_log : nullptr);
    MP_LAUNCH_CHECK();
    if (side) {
      MP_CUDA_CHECK(cudaEventRecord(state->aux_join[1], lane1));
      MP_CUDA_CHECK(cudaStreamWaitEvent(st, state->aux_join[1], 0));
    }
    return true;
  }
  const SsdScratch sc = ssd_carve(scratch, d, true);
  ssd_cumsum_kernel<<<d.B * d.H * d.nc, 256, 0, st>>>(static_cast<const float*>(dt), static_cast<const float*>(A), sc.cum, sc.dtt,
                                                     d.B, d.L, d.H, d.Q);
  MP_LAUNCH_CHECK();
  // The four operator instances are independent of one another: each runs on its own stream (forked from and
  // joined back into the caller's stream, which also works under stream capture) with its own scratch set, so
  // that one chain's kernels fill the SM slots another chain's last wave leaves idle.
  const bool side_by_side = getenv("MP_SSD_SERIAL") == nullptr;
  cudaStream_t lanes[4] = {st, st, st, st};
  if (side_by_side) {
    mp_aux_init(state);
    MP_CUDA_CHECK(cudaEventRecord(state->aux_fork, st));
    for (int i = 0; i < 3; ++i) {
      MP_CUDA_CHECK(cudaStreamWaitEvent(state->aux_stream[i], state->aux_fork, 0));
      lanes[i + 1] = state->aux_stream[i];
    }
  }
  auto scratch_of = [&](int op) {
    SsdScratch o = sc;
    o.scores = sc.scores_op[op]; o.states = sc.states_op[op]; o.hs = sc.hs_op[op]; o.parts = sc.parts_op[op];
    return o;
  };
  Roles r;
  // gx and v_t = <gx_t, x_t>   (the caller's stream)
  r.q = bh; r.q_head = 0; r.k = ch; r.k_head = 0; r.v = gyh; r.v_head = 1;
  r.dk = d.N; r.dv = d.P; r.anti = 1; r.scores_head = 0; r.out_head = 1;
  r.out = static_cast<__half*>(gx); r.z = xh; r.dot = sc.v;
  auto run_op = [&](int op) {
    if (side_by_side) ssd_operator(d, r, scratch_of(op), state->status_dev, lanes[op], state->aux_stream[3 + op],
                                   state->aux_sub_fork[op], state->aux_join[3 + op]);
    else ssd_operator(d, r, scratch_of(op), state->status_dev, lanes[op]);
  };
  run_op(0);
  // u_t = <gy_t, y_t>: the forward operator with the row dot as its only output
  r.q = ch; r.q_head = 0; r.k = bh; r.k_head = 0; r.v = xh; r.v_head = 1;
  r.dk = d.N; r.dv = d.P; r.anti = 0; r.scores_head = 0; r.out_head = 1;
  r.out = nullptr; r.z = gyh; r.dot = sc.u;
  run_op(1);
  // gC (summed over the heads of each group)
  r.q = gyh; r.q_head = 1; r.k = xh; r.k_head = 1; r.v = bh; r.v_head = 0;
  r.dk = d.P; r.dv = d.N; r.anti = 0; r.scores_head = 1; r.out_head = 0;
  r.out = static_cast<__half*>(gC); r.z = nullptr; r.dot = nullptr;
  run_op(2);
  // gB
  r.q = xh; r.q_head = 1; r.k = gyh; r.k_head = 1; r.v = ch; r.v_head = 0;
  r.dk = d.P; r.dv = d.N; r.anti = 1; r.scores_head = 1; r.out_head = 0;
  r.out = static_cast<__half*>(gB); r.z = nullptr; r.dot = nullptr;
  run_op(3);
  if (side_by_side) {
    for (int i = 0; i < 3; ++i) {
      MP_CUDA_CHECK(cudaEventRecord(state->aux_join[i], state->aux_stream[i]));
      MP_CUDA_CHECK(cudaStreamWaitEvent(st, state->aux_join[i], 0));
    }
  }
  // gdt, gA
  // (operator 0 = gx: anti-causal states of C gy^T; operator 1 = u: causal states of B x^T; both [B,H,nc][N][P])
    ssd_boundary_dot_kernel<<<d.B * d.H * d.nc, 256, 0, st>>>(sc.hs_op[0], sc.hs_op[1], sc.pin, d.nc, d.N * d.P);
    MP_LAUNCH_CHECK();
    ssd_scalar_grads_kernel<<<d.B * d.H, 256, 0, st>>>(sc.u, sc.v, sc.dtt, static_cast<const float*>(A), sc.pin, static_cast<float*>(gdt),
                                                      sc.ga_part, d.B, d.L, d.H, d.Q, 1);
    MP_LAUNCH_CHECK();
  ssd_sum_batches_kernel<<<(d.H + 127) / 128, 128, 0, st>>>(sc.ga_part, static_cast<float*>(gA), d.B, d.H);
  MP_LAUNCH_CHECK();
  return false;
}

// launch_ssd_scan_reverse plus the reverses of dt = softplus(dt_raw + dt_bias[h]) and A = -exp(A_log[h]):
//   gdt_raw = gdt * sigmoid(dt_raw + dt_bias) (T, pitched), gdt_bias[h] += its sum, gA_log[h] += gA[h] * A[h]
// inside the scan's scalar-gradient kernels where the chunk walk runs (two launches less per call), else as
// launch_softplus_bias_reverse and launch_hadamard_reverse after launch_ssd_scan_reverse.  gdt and gA are written as well.
extern "C" void launch_softplus_bias_reverse_r16(const void*, len_t, const void*, const void*, void*, len_t, void*, len_t, len_t, StreamContext);
extern "C" void launch_softplus_bias_reverse_r32(const void*, len_t, const void*, const void*, void*, len_t, void*, len_t, len_t, StreamContext);
extern "C" void launch_softplus_bias_reverse_r64(const void*, len_t, const void*, const void*, void*, len_t, void*, len_t, len_t, StreamContext);
extern "C" void launch_hadamard_reverse_r32(const void*, const void*, void*, len_t, StreamContext);
extern "C" void launch_hadamard_reverse_r64(const void*, const void*, void*, len_t, StreamContext);
extern "C" void launch_ssd_scan_reverse_r32(const void*, const void*, const void*, const void*, const void*, const void*, void*, void*, void*, void*,
                                            void*, void*, len_t, len_t, len_t, len_t, len_t, len_t, len_t, StreamContext);
extern "C" void launch_ssd_scan_reverse_r64(const void*, const void*, const void*, const void*, const void*, const void*, void*, void*, void*, void*,
                                            void*, void*, len_t, len_t, len_t, len_t, len_t, len_t, len_t, StreamContext);

extern "C" void launch_ssd_scan_reverse_raw_r16(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm, const void* gy,
                                                const void* dt_raw, len_t dt_pitch, const void* dt_bias, void* gx, void* gdt, void* gA,
                                                void* gdt_raw, len_t gdt_raw_pitch, void* gdt_bias, void* gA_log, void* gB, void* gC, void* scratch,
                                                len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk,
                                                StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  RawSide rs{static_cast<const __half*>(dt_raw), dt_pitch, static_cast<const float*>(dt_bias), static_cast<__half*>(gdt_raw), gdt_raw_pitch,
             static_cast<float*>(gdt_bias), static_cast<float*>(gA_log)};
  if (ssd_scan_reverse_r16_impl(x, dt, A, Bm, Cm, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx, &rs))
    return;
  launch_softplus_bias_reverse_r16(dt_raw, dt_pitch, dt_bias, gdt, gdt_raw, gdt_raw_pitch, gdt_bias, batch * seqlen, heads, ctx);
  if (gA_log != nullptr) launch_hadamard_reverse_r32(gA, A, gA_log, heads, ctx);
}
extern "C" void launch_ssd_scan_reverse_raw_r32(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm, const void* gy,
                                                const void* dt_raw, len_t dt_pitch, const void* dt_bias, void* gx, void* gdt, void* gA,
                                                void* gdt_raw, len_t gdt_raw_pitch, void* gdt_bias, void* gA_log, void* gB, void* gC, void* scratch,
                                                len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk,
                                                StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  launch_ssd_scan_reverse_r32(x, dt, A, Bm, Cm, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx);
  launch_softplus_bias_reverse_r32(dt_raw, dt_pitch, dt_bias, gdt, gdt_raw, gdt_raw_pitch, gdt_bias, batch * seqlen, heads, ctx);
  if (gA_log != nullptr) launch_hadamard_reverse_r32(gA, A, gA_log, heads, ctx);
}
extern "C" void launch_ssd_scan_reverse_raw_r64(const void* x, const void* dt, const void* A, const void* Bm, const void* Cm, const void* gy,
                                                const void* dt_raw, len_t dt_pitch, const void* dt_bias, void* gx, void* gdt, void* gA,
                                                void* gdt_raw, len_t gdt_raw_pitch, void* gdt_bias, void* gA_log, void* gB, void* gC, void* scratch,
                                                len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk,
                                                StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  launch_ssd_scan_reverse_r64(x, dt, A, Bm, Cm, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, chunk, ctx);
  launch_softplus_bias_reverse_r64(dt_raw, dt_pitch, dt_bias, gdt, gdt_raw, gdt_raw_pitch, gdt_bias, batch * seqlen, heads, ctx);
  if (gA_log != nullptr) launch_hadamard_reverse_r64(gA, A, gA_log, heads, ctx);
}
