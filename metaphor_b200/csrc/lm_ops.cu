// Operators that sit between the contractions, the RMSNorm and the SSD scan in a
// Mamba-2 language-model step: token embedding, depthwise causal convolution +
// SiLU, softplus of the step sizes, D-skip + SiLU gate, cross-entropy (loss and
// logit gradient in one kernel) and precision conversion between r16 working
// copies and r32 master buffers.  The reference has none of these (its loss
// layer is a sketch, src/ops/loss.zig:60-237); they follow its launcher
// conventions: inputs, scalars, outputs, sizes, StreamContext last.
//
// All of them are HBM-bound: every tensor is read once and written once with
// 16-byte accesses; small parameter gradients (conv taps, biases, D) are reduced
// inside the CTA and added with one atomic per CTA and element.  Parameter
// gradients and per-head parameters are kept in the accumulator type (r32 for
// r16 / r32 tensors, r64 for r64).
#include "mp_async.cuh"

namespace {

template <typename T, int V>
struct alignas(sizeof(T) * V) VecT { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_vec(const T* p, typename Acc<T>::type* out) {
  const VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(p);
#pragma unroll
  for (int e = 0; e < V; ++e) out[e] = mp_up(x.v[e]);
}
template <typename T, int V>
__device__ __forceinline__ void store_vec(T* p, const typename Acc<T>::type* in) {
  VecT<T, V> x;
#pragma unroll
  for (int e = 0; e < V; ++e) x.v[e] = mp_down<T>(in[e]);
  *reinterpret_cast<VecT<T, V>*>(p) = x;
}

// ex2 + rcp on the special-function unit, four instructions: an IEEE division costs ten, and the non-flushing forms
// behind __expf / __fdividef add range fix-ups that the conv and gate kernels, which are bound by instruction issue,
// pay per element.  Saturates correctly: x -> -inf gives ex2 = +inf, rcp = 0; x -> +inf gives ex2 = 0, rcp = 1.
__device__ __forceinline__ float sigmoid_a(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return r;
}
__device__ __forceinline__ double sigmoid_a(double x) { return 1.0 / (1.0 + exp(-x)); }
__device__ __forceinline__ float exp_a(float x) { return __expf(x); }
__device__ __forceinline__ double exp_a(double x) { return exp(x); }
__device__ __forceinline__ float log_a(float x) { return __logf(x); }
__device__ __forceinline__ double log_a(double x) { return log(x); }
__device__ __forceinline__ float log1p_a(float x) { return log1pf(x); }
__device__ __forceinline__ double log1p_a(double x) { return log1p(x); }

// true when V-wide accesses at base + k * pitch (+ multiples of V) are aligned
template <typename T>
bool vec_ok(const void* p, size_t pitch, size_t width) {
  constexpr size_t PN = Pack<T>::N;
  return mp_aligned16(p) && pitch % PN == 0 && width % PN == 0;
}

// ---------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]; ids outside [0, vocab) give a zero row
// ---------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(256) embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                                        T* __restrict__ out, size_t n, size_t dim, size_t vocab) {
  const size_t per_row = dim / V;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n * per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / per_row, p = i % per_row;
    const long long id = ids[t];
    VecT<T, V> x;
    if (id >= 0 && static_cast<size_t>(id) < vocab) {
      x = *reinterpret_cast<const VecT<T, V>*>(table + static_cast<size_t>(id) * dim + p * V);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) x.v[e] = mp_down<T>(0);
    }
    *reinterpret_cast<VecT<T, V>*>(out + t * dim + p * V) = x;
  }
}

// gtable[ids[t], :] += gy[t, :]   (accumulator-typed table gradient, atomics)
template <typename T>
__global__ void __launch_bounds__(256) embedding_reverse_kernel(const int* __restrict__ ids, const T* __restrict__ gy,
                                                                typename Acc<T>::type* __restrict__ gtable, size_t n,
                                                                size_t dim, size_t vocab) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n * dim;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / dim, j = i % dim;
    const long long id = ids[t];
    if (id >= 0 && static_cast<size_t>(id) < vocab) atomicAdd(gtable + static_cast<size_t>(id) * dim + j, mp_up(gy[i]));
  }
}

// The V x W taps (and V biases) of a thread's channels are contiguous in memory: fetch them with the
// widest aligned vector loads (element-wise loads at a 2 * V * W byte lane stride cost one sector each).
template <typename T, int N>
__device__ __forceinline__ void load_contiguous(const T* p, typename Acc<T>::type* out) {
  constexpr int MAXV = 16 / sizeof(T);
  constexpr int LOW = N & (-N);                     // largest power of two dividing N
  constexpr int CH = LOW < MAXV ? LOW : MAXV;
  if ((reinterpret_cast<uintptr_t>(p) & (CH * sizeof(T) - 1)) == 0) {
#pragma unroll
    for (int i = 0; i < N; i += CH) load_vec<T, CH>(p + i, out + i);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = mp_up(p[i]);
  }
}

// ---------------------------------------------------------------------------
// depthwise causal convolution + SiLU over [batch, len, channels] (pitched rows)
//   pre[b,l,c] = bias[c] + sum_k w[c,k] x[b, l - W + 1 + k, c]   (x = 0 before the sequence)
//   y = pre * sigmoid(pre)
// A thread owns CONV_LT consecutive steps of V channels and loads the CONV_LT + W - 1
// inputs it needs up front (independent loads; neighbouring threads share them through
// L1 / L2).  CTA = 32 channel groups x CONV_TY time lanes.
// ---------------------------------------------------------------------------
constexpr int CONV_LT = 4;
constexpr int CONV_TY = 8;
constexpr int CONV_NB = 4;   // reverse: time blocks walked by one CTA (fewer atomics on the tap gradients)

template <typename T, int V, int W>
__global__ void __launch_bounds__(32 * CONV_TY) conv1d_silu_kernel(const T* __restrict__ x, size_t xp, const T* __restrict__ w,
                                                                  const T* __restrict__ bias, T* __restrict__ y, size_t yp,
                                                                  int L, int C) {
  using A = typename Acc<T>::type;
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * V;
  const int l0 = (blockIdx.y * CONV_TY + threadIdx.y) * CONV_LT;
  if (c0 >= C || l0 >= L) return;
  const size_t b = blockIdx.z;
  const T* xb = x + b * L * xp + c0;
  T* yb = y + b * L * yp + c0;
  A xw[CONV_LT + W - 1][V];
#pragma unroll
  for (int j = 0; j < CONV_LT + W - 1; ++j) {
    const int l = l0 - (W - 1) + j;
    if (l >= 0 && l < L) load_vec<T, V>(xb + static_cast<size_t>(l) * xp, xw[j]);
    else {
#pragma unroll
      for (int e = 0; e < V; ++e) xw[j][e] = A(0);
    }
  }
  A wk[W][V], bs[V], wflat[V * W];
  load_contiguous<T, V * W>(w + static_cast<size_t>(c0) * W, wflat);
  if (bias != nullptr) load_contiguous<T, V>(bias + c0, bs);
#pragma unroll
  for (int e = 0; e < V; ++e) {
    if (bias == nullptr) bs[e] = A(0);
#pragma unroll
    for (int k = 0; k < W; ++k) wk[k][e] = wflat[e * W + k];
  }
#pragma unroll
  for (int j = 0; j < CONV_LT; ++j) {
    if (l0 + j < L) {
      A r[V];
#pragma unroll
      for (int e = 0; e < V; ++e) {
        A acc = bs[e];
#pragma unroll
        for (int k = 0; k < W; ++k) acc += wk[k][e] * xw[j + k][e];
        r[e] = acc * sigmoid_a(acc);
      }
      store_vec<T, V>(yb + static_cast<size_t>(l0 + j) * yp, r);
    }
  }
}

// Reverse: dpre = gy * s * (1 + pre * (1 - s)) with pre recomputed;
//   gx[l] = sum_k w[k] dpre[l + W - 1 - k];  gw[c,k] += sum_l dpre[l] x[l - W + 1 + k];  gbias[c] += sum_l dpre[l]
// A thread owns CONV_LT steps; the W - 1 values of dpre after them come from the next time lane of
// the CTA through shared memory (the last lane recomputes them).
template <typename T, int V, int W>
__global__ void __launch_bounds__(32 * CONV_TY) conv1d_silu_reverse_kernel(const T* __restrict__ x, size_t xp,
                                                                          const T* __restrict__ w, const T* __restrict__ bias,
                                                                          const T* __restrict__ gy, size_t gyp,
                                                                          T* __restrict__ gx, size_t gxp,
                                                                          typename Acc<T>::type* __restrict__ gw,
                                                                          typename Acc<T>::type* __restrict__ gbias, int L,
                                                                          int C) {
  using A = typename Acc<T>::type;
  constexpr int H = W - 1;                   // look-ahead steps
  constexpr int ND = CONV_LT + H;            // dpre values a thread needs
  __shared__ A red[CONV_TY][32][V * (W + 1) + 1];
  __shared__ A halo[CONV_TY][H][32][V];      // first H dpre of every time lane
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int c0 = (blockIdx.x * 32 + tx) * V;
  const bool live_c = c0 < C;
  const bool last_lane = ty == CONV_TY - 1;
  A gwk[W][V], gbs[V], wk[W][V], bs[V], wflat[V * W];
#pragma unroll
  for (int i = 0; i < V * W; ++i) wflat[i] = A(0);
#pragma unroll
  for (int e = 0; e < V; ++e) bs[e] = A(0);
  if (live_c) {
    load_contiguous<T, V * W>(w + static_cast<size_t>(c0) * W, wflat);
    if (bias != nullptr) load_contiguous<T, V>(bias + c0, bs);
  }
#pragma unroll
  for (int e = 0; e < V; ++e) {
    gbs[e] = A(0);
#pragma unroll
    for (int k = 0; k < W; ++k) { gwk[k][e] = A(0); wk[k][e] = wflat[e * W + k]; }
  }
  const size_t b = blockIdx.z;
  const T* xb = x + b * L * xp + c0;
  const T* gyb = gy + b * L * gyp + c0;
  T* gxb = gx + b * L * gxp + c0;
  auto dpre_of = [&](const A (*xwin)[V], const A* g, A* out) {   // xwin[k] = x[l - W + 1 + k]
#pragma unroll
    for (int e = 0; e < V; ++e) {
      A pre = bs[e];
#pragma unroll
      for (int k = 0; k < W; ++k) pre += wk[k][e] * xwin[k][e];
      const A sg = sigmoid_a(pre);
      out[e] = g[e] * sg * (A(1) + pre * (A(1) - sg));
    }
  };
#pragma unroll 1
  for (int nb = 0; nb < CONV_NB; ++nb) {
    const int l0 = ((blockIdx.y * CONV_NB + nb) * CONV_TY + ty) * CONV_LT;
    const bool live = live_c && l0 < L;
    A xw[CONV_LT + 2 * H][V], dp[ND][V];
#pragma unroll
    for (int j = 0; j < ND; ++j)
#pragma unroll
      for (int e = 0; e < V; ++e) dp[j][e] = A(0);
    if (live) {
      const int nx = last_lane ? CONV_LT + 2 * H : CONV_LT + H;   // the last lane also recomputes the look-ahead
#pragma unroll
      for (int j = 0; j < CONV_LT + 2 * H; ++j) {
        const int l = l0 - H + j;
        if (j < nx && l >= 0 && l < L) load_vec<T, V>(xb + static_cast<size_t>(l) * xp, xw[j]);
        else {
#pragma unroll
          for (int e = 0; e < V; ++e) xw[j][e] = A(0);
        }
      }
      const int ng = last_lane ? ND : CONV_LT;
#pragma unroll
      for (int j = 0; j < ND; ++j)
        if (j < ng && l0 + j < L) load_vec<T, V>(gyb + static_cast<size_t>(l0 + j) * gyp, dp[j]);   // gy for now
#pragma unroll
      for (int j = 0; j < CONV_LT; ++j) {
        dpre_of(&xw[j], dp[j], dp[j]);      // zero beyond the sequence (gy stayed zero there)
#pragma unroll
        for (int e = 0; e < V; ++e) {
          gbs[e] += dp[j][e];
#pragma unroll
          for (int k = 0; k < W; ++k) gwk[k][e] += dp[j][e] * xw[j + k][e];
        }
      }
      if (last_lane) {
#pragma unroll
        for (int j = CONV_LT; j < ND; ++j) dpre_of(&xw[j], dp[j], dp[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < H; ++j)
#pragma unroll
      for (int e = 0; e < V; ++e) halo[ty][j][tx][e] = dp[j][e];
    __syncthreads();
    if (!last_lane) {
#pragma unroll
      for (int j = 0; j < H; ++j)
#pragma unroll
        for (int e = 0; e < V; ++e) dp[CONV_LT + j][e] = halo[ty + 1][j][tx][e];
    }
    __syncthreads();
    if (live) {
#pragma unroll
      for (int m = 0; m < CONV_LT; ++m) {
        if (l0 + m < L) {
          A r[V];
#pragma unroll
          for (int e = 0; e < V; ++e) {
            A acc = A(0);
#pragma unroll
            for (int k = 0; k < W; ++k) acc += wk[k][e] * dp[m + W - 1 - k][e];
            r[e] = acc;
          }
          store_vec<T, V>(gxb + static_cast<size_t>(l0 + m) * gxp, r);
        }
      }
    }
  }
  // fold the time lanes of the CTA, then one atomic per (channel, tap)
#pragma unroll
  for (int e = 0; e < V; ++e) {
#pragma unroll
    for (int k = 0; k < W; ++k) red[ty][tx][e * (W + 1) + k] = gwk[k][e];
    red[ty][tx][e * (W + 1) + W] = gbs[e];
  }
  __syncthreads();
  if (ty == 0 && live_c) {
#pragma unroll
    for (int e = 0; e < V; ++e) {
#pragma unroll
      for (int k = 0; k <= W; ++k) {
        A sum = A(0);
#pragma unroll
        for (int t2 = 0; t2 < CONV_TY; ++t2) sum += red[t2][tx][e * (W + 1) + k];
        if (k < W) atomicAdd(gw + static_cast<size_t>(c0 + e) * W + k, sum);
        else if (gbias != nullptr) atomicAdd(gbias + c0 + e, sum);
      }
    }
  }
}

// Reverse for r16 rows that allow 16-byte accesses: a CTA stages a tile of 64 channels x 64 steps (plus the
// W - 1 steps before it of x and after it of gy) in shared memory with 16-byte loads, then every thread walks
// 16 steps of one channel with the windows of x and dpre in registers (one shared-memory read of x and of gy per
// step, no barrier inside the walk), and the gx tile leaves through shared memory with 16-byte stores.  The
// W - 1 look-ahead values of dpre are recomputed by the lane that needs them.  Tap / bias gradients accumulate
// in registers over the CTA's time tiles and end in one atomic per (CTA, channel, tap).
constexpr int CT_C = 64;            // channels per tile
constexpr int CT_L = 64;            // steps per tile
constexpr int CT_LANES = 4;         // time lanes: 128 threads = 32 channel PAIRS x 4 lanes (one warp per lane)
constexpr int CT_STEPS = CT_L / CT_LANES;
constexpr int CT_THREADS = (CT_C / 2) * CT_LANES;
// A thread owns two neighbouring channels: one 4-byte shared-memory access, one packed conversion and one packed
// store serve two elements (with a channel per thread and 2-byte accesses both kernels were bound by instruction
// issue at 35 / 59 instructions per element).

// 16-byte asynchronous global -> shared copies (LDGSTS); `valid == false` writes 16 zero bytes without touching global memory.
__device__ __forceinline__ void cp_async_16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(mp_smem_u32(smem_dst)), "l"(gmem_src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The channels of one convolution may be cut into up to CONV_MAX_SEGS consecutive segments whose outputs
// (forward: y; reverse: the incoming gy) live in buffers of their own: one launch then serves what would be
// one launch per segment (x / B / C of a Mamba-2 block share one convolution over neighbouring columns).
constexpr int CONV_MAX_SEGS = 4;
struct ConvSegs {
  int nseg;
  int blk_begin[CONV_MAX_SEGS + 1];   // first channel block (of CT_C channels) of every segment
  int ch_begin[CONV_MAX_SEGS];        // first channel
  int ch_count[CONV_MAX_SEGS];        // channels (a multiple of 8)
  const void* ptr[CONV_MAX_SEGS];     // the segment's own buffer (y resp. gy), channel 0 of the segment at column 0
  unsigned long long pitch[CONV_MAX_SEGS];
  // reverse only: a second upstream term per segment, gy_total = gy + scale[channel / skip_group] * skip (or nullptr)
  const void* skip_ptr[CONV_MAX_SEGS];
  unsigned long long skip_pitch[CONV_MAX_SEGS];
  const float* skip_scale[CONV_MAX_SEGS];
  int skip_group;
};
__device__ __forceinline__ int conv_segment_of(const ConvSegs& sg, int block) {
  int s = 0;
#pragma unroll
  for (int i = 1; i < CONV_MAX_SEGS; ++i)
    if (i < sg.nseg && block >= sg.blk_begin[i]) s = i;
  return s;
}

// Forward with the same staging: x tile (+ W - 1 rows before it) in, y tile out, 16 steps of two channels per thread.
template <int W>
__global__ void __launch_bounds__(CT_THREADS) conv1d_silu_tiled_kernel(const __half* __restrict__ x, size_t xp, const __half* __restrict__ w,
                                                                       const __half* __restrict__ bias, const ConvSegs sg, int L,
                                                                       int tiles_per_cta) {
  constexpr int H = W - 1;
  __shared__ __align__(16) __half xs[2][CT_L + H][CT_C];    // two tiles in turn; row r = step l0 - H + r
  __shared__ __align__(16) __half ys[CT_L][CT_C];
  const int tid = threadIdx.x;
  const int c = (tid % (CT_C / 2)) * 2, lane = tid / (CT_C / 2);
  const int seg = conv_segment_of(sg, blockIdx.x);
  const int local = (blockIdx.x - sg.blk_begin[seg]) * CT_C;   // first channel of the tile inside its segment
  const int cbase = sg.ch_begin[seg] + local;                  // ... and in x / w / bias
  const int C = sg.ch_begin[seg] + sg.ch_count[seg];           // channels past the segment's end belong to the next tile row
  const bool live_c = cbase + c < C;                           // (channel counts are multiples of 8: a pair is live or dead as one)
  const size_t b = blockIdx.z;
  const size_t yp = sg.pitch[seg];
  const __half* xb = x + b * L * xp + cbase;
  __half* yb = static_cast<__half*>(const_cast<void*>(sg.ptr[seg])) + b * L * yp + local;
  float wk[2][W], bs[2] = {0.f, 0.f};
#pragma unroll
  for (int e = 0; e < 2; ++e) {
#pragma unroll
    for (int k = 0; k < W; ++k) wk[e][k] = live_c ? __half2float(w[static_cast<size_t>(cbase + c + e) * W + k]) : 0.f;
    if (live_c && bias != nullptr) bs[e] = __half2float(bias[cbase + c + e]);
  }
  constexpr int PPR = CT_C / 8;
  const int packs_live = min(PPR, (C - cbase) / 8);
  // tile t + 1 is fetched (asynchronous copies, zero-filled outside the sequence / the segment) while tile t is computed
  auto stage = [&](int t) {
    const int l0 = (blockIdx.y * tiles_per_cta + t) * CT_L;
    for (int v = tid; v < (CT_L + H) * PPR; v += CT_THREADS) {
      const int r = v / PPR, pk = v % PPR;
      const int l = l0 - H + r;
      const bool ok = l >= 0 && l < L && pk < packs_live;
      cp_async_16_zfill(&xs[t & 1][r][pk * 8], ok ? xb + static_cast<size_t>(l) * xp + pk * 8 : xb, ok);
    }
    cp_async_commit();
  };
  stage(0);
  for (int t = 0; t < tiles_per_cta; ++t) {
    const int l0 = (blockIdx.y * tiles_per_cta + t) * CT_L;
    if (l0 >= L) break;
    const bool more = t + 1 < tiles_per_cta && l0 + CT_L < L;
    if (more) { stage(t + 1); cp_async_wait<1>(); } else cp_async_wait<0>();
    __syncthreads();
    {
      const __half (*xt)[CT_C] = xs[t & 1];
      const int s0 = lane * CT_STEPS;
      float2 xw[W];
#pragma unroll
      for (int k = 0; k < H; ++k) xw[k + 1] = __half22float2(*reinterpret_cast<const __half2*>(&xt[s0 + k][c]));
#pragma unroll
      for (int j = 0; j < CT_STEPS; ++j) {
#pragma unroll
        for (int k = 0; k < H; ++k) xw[k] = xw[k + 1];
        xw[H] = __half22float2(*reinterpret_cast<const __half2*>(&xt[s0 + j + H][c]));
        float p0 = bs[0], p1 = bs[1];
#pragma unroll
        for (int k = 0; k < W; ++k) { p0 += wk[0][k] * xw[k].x; p1 += wk[1][k] * xw[k].y; }
        *reinterpret_cast<__half2*>(&ys[s0 + j][c]) = __floats2half2_rn(p0 * sigmoid_a(p0), p1 * sigmoid_a(p1));
      }
    }
    __syncthreads();
    for (int v = tid; v < CT_L * PPR; v += CT_THREADS) {
      const int r = v / PPR, pk = v % PPR;
      const int l = l0 + r;
      if (l < L && pk < packs_live) *reinterpret_cast<uint4*>(yb + static_cast<size_t>(l) * yp + pk * 8) = *reinterpret_cast<const uint4*>(&ys[r][pk * 8]);
    }
  }
}

// SKIP: segments may carry a second upstream term (ConvSegs::skip_*), staged beside gy.  That variant stages ONE time
// tile at a time (the third tile would otherwise cost a quarter of the resident warps, and the kernel is bound by
// instruction issue and latency, not by bytes in flight: other CTAs of the SM cover a CTA's load phase).
template <int W, bool SKIP>
__global__ void __launch_bounds__(CT_THREADS) conv1d_silu_reverse_tiled_kernel(const __half* __restrict__ x, size_t xp,
                                                                               const __half* __restrict__ w, const __half* __restrict__ bias,
                                                                               const ConvSegs sg, __half* __restrict__ gx, size_t gxp,
                                                                               float* __restrict__ gw, float* __restrict__ gbias, int L,
                                                                               int tiles_per_cta) {
  constexpr int H = W - 1;
  constexpr int NBUF = SKIP ? 1 : 2;
  extern __shared__ __align__(16) unsigned char conv_rev_smem[];
  typedef __half (*TileX)[CT_L + 2 * H][CT_C];
  typedef __half (*TileG)[CT_L + H][CT_C];
  TileX xs = reinterpret_cast<TileX>(conv_rev_smem);                                   // [NBUF]: row r = step l0 - H + r
  TileG gys = reinterpret_cast<TileG>(conv_rev_smem + sizeof(__half) * NBUF * (CT_L + 2 * H) * CT_C);   // [NBUF]: row r = step l0 + r
  __half (*gxs)[CT_C] = reinterpret_cast<__half (*)[CT_C]>(reinterpret_cast<unsigned char*>(gys) + sizeof(__half) * NBUF * (CT_L + H) * CT_C);
  float (*red)[CT_C][W + 1] = reinterpret_cast<float (*)[CT_C][W + 1]>(reinterpret_cast<unsigned char*>(gxs) + sizeof(__half) * CT_L * CT_C);
  TileG g2s = reinterpret_cast<TileG>(reinterpret_cast<unsigned char*>(red) + sizeof(float) * CT_LANES * CT_C * (W + 1));   // [1], SKIP only
  const int tid = threadIdx.x;
  const int c = (tid % (CT_C / 2)) * 2, lane = tid / (CT_C / 2);
  const int seg = conv_segment_of(sg, blockIdx.x);
  const int local = (blockIdx.x - sg.blk_begin[seg]) * CT_C;
  const int cbase = sg.ch_begin[seg] + local;
  const int C = sg.ch_begin[seg] + sg.ch_count[seg];
  const bool live_c = cbase + c < C;
  const size_t b = blockIdx.z;
  const size_t gyp = sg.pitch[seg];
  const __half* xb = x + b * L * xp + cbase;
  const __half* gyb = static_cast<const __half*>(sg.ptr[seg]) + b * L * gyp + local;
  __half* gxb = gx + b * L * gxp + cbase;
  const bool skip = SKIP && sg.skip_ptr[seg] != nullptr;
  const size_t g2p = SKIP ? sg.skip_pitch[seg] : 0;
  const __half* g2b = skip ? static_cast<const __half*>(sg.skip_ptr[seg]) + b * L * g2p + local : nullptr;
  float sk[2] = {0.f, 0.f};   // the skip term's factor for this thread's two channels
  if (skip && cbase + c < C) {
    sk[0] = sg.skip_scale[seg][(local + c) / sg.skip_group];
    sk[1] = sg.skip_scale[seg][(local + c + 1) / sg.skip_group];
  }
  float wk[2][W], bs[2] = {0.f, 0.f}, gwk[2][W], gbs[2] = {0.f, 0.f};
#pragma unroll
  for (int e = 0; e < 2; ++e) {
#pragma unroll
    for (int k = 0; k < W; ++k) { wk[e][k] = live_c ? __half2float(w[static_cast<size_t>(cbase + c + e) * W + k]) : 0.f; gwk[e][k] = 0.f; }
    if (live_c && bias != nullptr) bs[e] = __half2float(bias[cbase + c + e]);
  }
  constexpr int PPR = CT_C / 8;   // 16-byte packs per tile row
  const int packs_live = min(PPR, (C - cbase) / 8);   // C is a multiple of 8 on this path

  // ---- stage x and gy of tile t (zero outside the sequence and beyond the last channel) with asynchronous copies:
  //      tile t + 1 is in flight while tile t is walked ----
  auto stage = [&](int t) {
    const int l0 = (blockIdx.y * tiles_per_cta + t) * CT_L;
    for (int v = tid; v < (CT_L + 2 * H) * PPR; v += CT_THREADS) {
      const int r = v / PPR, pk = v % PPR;
      const int l = l0 - H + r;
      const bool ok = l >= 0 && l < L && pk < packs_live;
      cp_async_16_zfill(&xs[t % NBUF][r][pk * 8], ok ? xb + static_cast<size_t>(l) * xp + pk * 8 : xb, ok);
    }
    for (int v = tid; v < (CT_L + H) * PPR; v += CT_THREADS) {
      const int r = v / PPR, pk = v % PPR;
      const int l = l0 + r;
      const bool ok = l < L && pk < packs_live;
      cp_async_16_zfill(&gys[t % NBUF][r][pk * 8], ok ? gyb + static_cast<size_t>(l) * gyp + pk * 8 : gyb, ok);
      if (SKIP && skip) cp_async_16_zfill(&g2s[0][r][pk * 8], ok ? g2b + static_cast<size_t>(l) * g2p + pk * 8 : g2b, ok);
    }
    cp_async_commit();
  };
  stage(0);
  for (int t = 0; t < tiles_per_cta; ++t) {
    const int l0 = (blockIdx.y * tiles_per_cta + t) * CT_L;
    if (l0 >= L) break;
    const bool more = t + 1 < tiles_per_cta && l0 + CT_L < L;
    if (NBUF == 2) {
      if (more) { stage(t + 1); cp_async_wait<1>(); } else cp_async_wait<0>();
    } else {
      if (t > 0) { __syncthreads(); stage(t); }   // every thread is past the previous tile's walk
      cp_async_wait<0>();
    }
    __syncthreads();
    // ---- walk CT_STEPS (+ H look-ahead) steps of two channels ----
    {
      const __half (*xt)[CT_C] = xs[t % NBUF];
      const __half (*gt)[CT_C] = gys[t % NBUF];
      const __half (*g2t)[CT_C] = g2s[0];
      const int s0 = lane * CT_STEPS;
      float2 xw[W], d[W];   // xw[k] = x at step s + k - H (tile row s + k); d[k] = dpre at step s - k
#pragma unroll
      for (int k = 0; k < W; ++k) d[k] = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < H; ++k) xw[k + 1] = __half22float2(*reinterpret_cast<const __half2*>(&xt[s0 + k][c]));
#pragma unroll
      for (int j = 0; j < CT_STEPS + H; ++j) {
        const int s = s0 + j;
#pragma unroll
        for (int k = 0; k < H; ++k) xw[k] = xw[k + 1];
        xw[H] = __half22float2(*reinterpret_cast<const __half2*>(&xt[s + H][c]));
        float p0 = bs[0], p1 = bs[1];
#pragma unroll
        for (int k = 0; k < W; ++k) { p0 += wk[0][k] * xw[k].x; p1 += wk[1][k] * xw[k].y; }
        const float g0 = sigmoid_a(p0), g1 = sigmoid_a(p1);
        float2 gyv = __half22float2(*reinterpret_cast<const __half2*>(&gt[s][c]));
        if (SKIP && skip) {
          const float2 g2v = __half22float2(*reinterpret_cast<const __half2*>(&g2t[s][c]));
          gyv.x += sk[0] * g2v.x; gyv.y += sk[1] * g2v.y;
        }
        const float2 dp = make_float2(gyv.x * g0 * (1.f + p0 * (1.f - g0)), gyv.y * g1 * (1.f + p1 * (1.f - g1)));
#pragma unroll
        for (int k = H; k > 0; --k) d[k] = d[k - 1];
        d[0] = dp;
        if (j < CT_STEPS) {   // own steps only: the look-ahead belongs to the next lane / tile
          gbs[0] += dp.x; gbs[1] += dp.y;
#pragma unroll
          for (int k = 0; k < W; ++k) { gwk[0][k] += dp.x * xw[k].x; gwk[1][k] += dp.y * xw[k].y; }
        }
        if (j >= H) {         // gx at step s - H = sum_k w[k] dpre[s - k]
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int k = 0; k < W; ++k) { a0 += wk[0][k] * d[k].x; a1 += wk[1][k] * d[k].y; }
          *reinterpret_cast<__half2*>(&gxs[s - H][c]) = __floats2half2_rn(a0, a1);
        }
      }
    }
    __syncthreads();
    // ---- gx tile -> global ----
    for (int v = tid; v < CT_L * PPR; v += CT_THREADS) {
      const int r = v / PPR, pk = v % PPR;
      const int l = l0 + r;
      if (l < L && pk < packs_live) *reinterpret_cast<uint4*>(gxb + static_cast<size_t>(l) * gxp + pk * 8) = *reinterpret_cast<const uint4*>(&gxs[r][pk * 8]);
    }
    // the staging of tile t + 2 (issued in the next trip) overwrites this tile's buffers: all threads are past the walk;
    // gxs is rewritten after the next barrier pair, so no further barrier is needed here
  }
  // ---- fold the time lanes, one atomic per (channel, tap) ----
#pragma unroll
  for (int e = 0; e < 2; ++e) {
#pragma unroll
    for (int k = 0; k < W; ++k) red[lane][c + e][k] = gwk[e][k];
    red[lane][c + e][W] = gbs[e];
  }
  __syncthreads();
  for (int i = tid; i < CT_C * (W + 1); i += CT_THREADS) {
    const int ch = i / (W + 1), k = i % (W + 1);
    if (cbase + ch < C) {
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < CT_LANES; ++q) sum += red[q][ch][k];
      if (k < W) atomicAdd(gw + static_cast<size_t>(cbase + ch) * W + k, sum);
      else if (gbias != nullptr) atomicAdd(gbias + cbase + ch, sum);
    }
  }
}

// ---------------------------------------------------------------------------
// dt = softplus(raw + bias[h]) (accumulator-typed output), raw pitched [rows, H]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) softplus_bias_kernel(const T* __restrict__ raw, size_t rp,
                                                            const typename Acc<T>::type* __restrict__ bias,
                                                            typename Acc<T>::type* __restrict__ out, size_t rows, int H) {
  using A = typename Acc<T>::type;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < rows * H;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / H;
    const int h = static_cast<int>(i % H);
    const A v = mp_up(raw[r * rp + h]) + bias[h];
    out[i] = v > A(20) ? v : log1p_a(exp_a(v));
  }
}

// graw = gdt * sigmoid(raw + bias);  gbias[h] += sum_rows graw
template <typename T>
__global__ void __launch_bounds__(256) softplus_bias_reverse_kernel(const T* __restrict__ raw, size_t rp,
                                                                    const typename Acc<T>::type* __restrict__ bias,
                                                                    const typename Acc<T>::type* __restrict__ gdt,
                                                                    T* __restrict__ graw, size_t gp,
                                                                    typename Acc<T>::type* __restrict__ gbias, size_t rows,
                                                                    int H) {
  using A = typename Acc<T>::type;
  extern __shared__ unsigned char sp_smem[];
  A* bins = reinterpret_cast<A*>(sp_smem);
  for (int h = threadIdx.x; h < H; h += blockDim.x) bins[h] = A(0);
  __syncthreads();
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < rows * H;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / H;
    const int h = static_cast<int>(i % H);
    const A v = mp_up(raw[r * rp + h]) + bias[h];
    const A g = gdt[i] * sigmoid_a(v);
    graw[r * gp + h] = mp_down<T>(g);
    atomicAdd(bins + h, g);
  }
  __syncthreads();
  if (gbias != nullptr)
    for (int h = threadIdx.x; h < H; h += blockDim.x) atomicAdd(gbias + h, bins[h]);
}

// The same for H <= 256 heads without a shared-memory atomic per element: thread (rr, h) keeps head h for all its
// rows rr, rr + RR, ... and sums in a register; the RR sums of a head meet in shared memory, one global atomic per
// (CTA, head).  (24 bins shared by 256 threads serialised the per-element atomics: 17 us for 0.8 MB.)
template <typename T>
__global__ void __launch_bounds__(256) softplus_bias_reverse_heads_kernel(const T* __restrict__ raw, size_t rp,
                                                                          const typename Acc<T>::type* __restrict__ bias,
                                                                          const typename Acc<T>::type* __restrict__ gdt,
                                                                          T* __restrict__ graw, size_t gp,
                                                                          typename Acc<T>::type* __restrict__ gbias, size_t rows,
                                                                          int H, int RR) {
  using A = typename Acc<T>::type;
  __shared__ A part[256];
  const int tid = threadIdx.x;
  const int rr = tid / H, h = tid - rr * H;
  A sum = A(0);
  if (rr < RR) {
    const A b = bias[h];
    for (size_t r = static_cast<size_t>(blockIdx.x) * RR + rr; r < rows; r += static_cast<size_t>(gridDim.x) * RR) {
      const A v = mp_up(raw[r * rp + h]) + b;
      const A g = gdt[r * H + h] * sigmoid_a(v);
      graw[r * gp + h] = mp_down<T>(g);
      sum += g;
    }
  }
  part[tid] = sum;
  __syncthreads();
  if (gbias != nullptr && tid < H) {
    A t = A(0);
    for (int q = 0; q < RR; ++q) t += part[q * H + tid];
    atomicAdd(gbias + tid, t);
  }
}

// ---------------------------------------------------------------------------
// skip + gate around the scan: u = (y + D[h] x) * silu(z);  rows x (H * P), z pitched
// ---------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(256) ssd_gate_kernel(const T* __restrict__ y, const T* __restrict__ x,
                                                       const typename Acc<T>::type* __restrict__ D, const T* __restrict__ z,
                                                       size_t zp, T* __restrict__ u, size_t rows, int H, int P) {
  using A = typename Acc<T>::type;
  const size_t width = static_cast<size_t>(H) * P, per_row = width / V;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < rows * per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / per_row, c = (i % per_row) * V;
    A yv[V], xv[V], zv[V], o[V];
    load_vec<T, V>(y + r * width + c, yv);
    load_vec<T, V>(x + r * width + c, xv);
    load_vec<T, V>(z + r * zp + c, zv);
    const A d = D != nullptr ? D[c / P] : A(0);
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = (yv[e] + d * xv[e]) * zv[e] * sigmoid_a(zv[e]);
    store_vec<T, V>(u + r * width + c, o);
  }
}

// gy = gu * silu(z);  gz = gu * (y + D x) * (s + z s (1 - s));  gD[h] += sum gy * x
template <typename T, int V>
__global__ void __launch_bounds__(256) ssd_gate_reverse_kernel(const T* __restrict__ y, const T* __restrict__ x,
                                                               const typename Acc<T>::type* __restrict__ D,
                                                               const T* __restrict__ z, size_t zp, const T* __restrict__ gu,
                                                               T* __restrict__ gy, T* __restrict__ gz, size_t gzp,
                                                               typename Acc<T>::type* __restrict__ gD, size_t rows, int H,
                                                               int P) {
  using A = typename Acc<T>::type;
  extern __shared__ unsigned char gate_smem[];
  A* bins = reinterpret_cast<A*>(gate_smem);
  for (int h = threadIdx.x; h < H; h += blockDim.x) bins[h] = A(0);
  __syncthreads();
  const size_t width = static_cast<size_t>(H) * P, per_row = width / V;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < rows * per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / per_row, c = (i % per_row) * V;
    A yv[V], xv[V], zv[V], gv[V], oy[V], oz[V];
    load_vec<T, V>(y + r * width + c, yv);
    load_vec<T, V>(x + r * width + c, xv);
    load_vec<T, V>(z + r * zp + c, zv);
    load_vec<T, V>(gu + r * width + c, gv);
    const int h = static_cast<int>(c / P);
    const A d = D != nullptr ? D[h] : A(0);
    A part = A(0);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const A s = sigmoid_a(zv[e]);
      oy[e] = gv[e] * zv[e] * s;
      oz[e] = gv[e] * (yv[e] + d * xv[e]) * (s + zv[e] * s * (A(1) - s));
      part += oy[e] * xv[e];
    }
    store_vec<T, V>(gy + r * width + c, oy);
    store_vec<T, V>(gz + r * gzp + c, oz);
    if (gD != nullptr) atomicAdd(bins + h, part);
  }
  __syncthreads();
  if (gD != nullptr)
    for (int h = threadIdx.x; h < H; h += blockDim.x) atomicAdd(gD + h, bins[h]);
}

// ---------------------------------------------------------------------------
// Gate + RMSNorm in one pass (the block's "gated norm"): with u = (y + D[h] x) * silu(z),
//   out = u * rstd * gain,  rstd = 1 / sqrt(mean_j u_j^2 + eps)
// u is never written: the reverse recomputes it from y, x and z.  One warp per row; with NP > 0 the row's
// packs stay in registers between the reduction and the output pass (NP packs of V elements per lane, row
// width = 32 * NP * V), with NP = 0 the second pass reads the row again (any width, V = 1 for unaligned rows).
// ---------------------------------------------------------------------------
constexpr int GN_THREADS = 256;   // 8 rows in flight per CTA

template <typename PackT>
__device__ __forceinline__ void gn_opaque(PackT& v) {
  if constexpr (sizeof(PackT) % 4 == 0) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(PackT) / 4); ++i) asm volatile("" : "+r"(w[i]));
  }
}

template <typename T, int V>
__device__ __forceinline__ void gn_load3(const T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ z, size_t off, size_t zoff,
                                         typename Acc<T>::type* yv, typename Acc<T>::type* xv, typename Acc<T>::type* zv) {
  load_vec<T, V>(y + off, yv);
  load_vec<T, V>(x + off, xv);
  load_vec<T, V>(z + zoff, zv);
}

template <typename T, int V, int NP>
__global__ void __launch_bounds__(GN_THREADS) gate_rmsnorm_kernel(const T* __restrict__ y, const T* __restrict__ x,
                                                                  const typename Acc<T>::type* __restrict__ D, const T* __restrict__ z,
                                                                  size_t zp, const T* __restrict__ gain, typename Acc<T>::type eps,
                                                                  T* __restrict__ out, typename Acc<T>::type* __restrict__ rstd,
                                                                  size_t rows, int H, int P) {
  using A = typename Acc<T>::type;
  const int lane = threadIdx.x & 31;
  const size_t width = static_cast<size_t>(H) * P;
  const int packs = NP > 0 ? NP : static_cast<int>((width / V + 31) / 32);
  const size_t warps = static_cast<size_t>(gridDim.x) * (GN_THREADS / 32);
  for (size_t r = blockIdx.x * static_cast<size_t>(GN_THREADS / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
    A u[NP > 0 ? NP : 1][V];
    A sum = A(0);
#pragma unroll
    for (int p = 0; p < packs; ++p) {
      const size_t c = (static_cast<size_t>(p) * 32 + lane) * V;
      if (NP > 0 || c < width) {
        A yv[V], xv[V], zv[V];
        gn_load3<T, V>(y, x, z, r * width + c, r * zp + c, yv, xv, zv);
        const A d = D != nullptr ? D[c / P] : A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const A t = (yv[e] + d * xv[e]) * zv[e] * sigmoid_a(zv[e]);
          if (NP > 0) u[NP > 0 ? p : 0][e] = t;
          sum += t * t;
        }
      }
    }
    sum = warp_reduce<SumOp>(sum);
    const A rs = A(1) / sqrt(sum / static_cast<A>(width) + eps);
    if (lane == 0 && rstd != nullptr) rstd[r] = rs;
#pragma unroll
    for (int p = 0; p < packs; ++p) {
      const size_t c = (static_cast<size_t>(p) * 32 + lane) * V;
      if (NP > 0 || c < width) {
        A gv[V], o[V];
        load_vec<T, V>(gain + c, gv);
        if (NP > 0) {
#pragma unroll
          for (int e = 0; e < V; ++e) o[e] = u[NP > 0 ? p : 0][e] * rs * gv[e];
        } else {
          A yv[V], xv[V], zv[V];
          gn_load3<T, V>(y, x, z, r * width + c, r * zp + c, yv, xv, zv);
          const A d = D != nullptr ? D[c / P] : A(0);
#pragma unroll
          for (int e = 0; e < V; ++e) o[e] = (yv[e] + d * xv[e]) * zv[e] * sigmoid_a(zv[e]) * rs * gv[e];
        }
        store_vec<T, V>(out + r * width + c, o);
      }
    }
  }
}

// Reverse of the gated norm.  Per row, with u as above, xh = u * rstd, gxh = gout * gain, m = mean_j gxh_j xh_j:
//   gu = rstd * (gxh - xh * m);  gy = gu * silu(z);  gz = gu * (y + D x) * silu'(z);  gD[h] += sum gy * x
//   ggain_j = sum over rows of gout_j * xh_j: every CTA leaves one partial row in `partial` (folded afterwards).
// The per-column and per-head sums of a lane's packs are kept in registers over all rows of the warp (NP > 0)
// or added to shared memory row by row (NP = 0).  Shared memory: width + H accumulators.
template <typename T, int V, int NP>
__global__ void __launch_bounds__(GN_THREADS) gate_rmsnorm_reverse_kernel(
    const T* __restrict__ y, const T* __restrict__ x, const typename Acc<T>::type* __restrict__ D, const T* __restrict__ z, size_t zp,
    const T* __restrict__ gain, const typename Acc<T>::type* __restrict__ rstd, const T* __restrict__ gout, T* __restrict__ gy,
    T* __restrict__ gz, size_t gzp, typename Acc<T>::type* __restrict__ gD, typename Acc<T>::type* __restrict__ partial, size_t rows,
    int H, int P) {
  using A = typename Acc<T>::type;
  extern __shared__ unsigned char gn_smem[];
  A* cols = reinterpret_cast<A*>(gn_smem);
  const size_t width = static_cast<size_t>(H) * P;
  A* bins = cols + width;
  for (size_t i = threadIdx.x; i < width + H; i += GN_THREADS) cols[i] = A(0);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int packs = NP > 0 ? NP : static_cast<int>((width / V + 31) / 32);
  const size_t warps = static_cast<size_t>(gridDim.x) * (GN_THREADS / 32);
  A gacc[NP > 0 ? NP : 1][V];
  A dacc[NP > 0 ? NP : 1];
#pragma unroll
  for (int p = 0; p < (NP > 0 ? NP : 1); ++p) {
    dacc[p] = A(0);
#pragma unroll
    for (int e = 0; e < V; ++e) gacc[p][e] = A(0);
  }
  for (size_t r = blockIdx.x * static_cast<size_t>(GN_THREADS / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
    const A rs = rstd[r];
    // pass 1: dot = sum gxh * xh, and the gain-gradient terms; the raw packs stay in registers for pass 2
    VecT<T, V> ry[NP > 0 ? NP : 1], rx[NP > 0 ? NP : 1], rz[NP > 0 ? NP : 1], rg[NP > 0 ? NP : 1];
    A dot = A(0);
    if (NP > 0) {
#pragma unroll
      for (int p = 0; p < NP; ++p) {   // all loads of the row first
        const size_t c = (static_cast<size_t>(p) * 32 + lane) * V;
        ry[p] = *reinterpret_cast<const VecT<T, V>*>(y + r * width + c);
        rx[p] = *reinterpret_cast<const VecT<T, V>*>(x + r * width + c);
        rz[p] = *reinterpret_cast<const VecT<T, V>*>(z + r * zp + c);
        rg[p] = *reinterpret_cast<const VecT<T, V>*>(gout + r * width + c);
      }
    }
#pragma unroll
    for (int p = 0; p < packs; ++p) {
      const size_t c = (static_cast<size_t>(p) * 32 + lane) * V;
      if (NP > 0 || c < width) {
        const int q = NP > 0 ? p : 0;
        if (NP == 0) {
          ry[0] = *reinterpret_cast<const VecT<T, V>*>(y + r * width + c);
          rx[0] = *reinterpret_cast<const VecT<T, V>*>(x + r * width + c);
          rz[0] = *reinterpret_cast<const VecT<T, V>*>(z + r * zp + c);
          rg[0] = *reinterpret_cast<const VecT<T, V>*>(gout + r * width + c);
        }
        A gn[V];
        load_vec<T, V>(gain + c, gn);
        const A d = D != nullptr ? D[c / P] : A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const A zz = mp_up(rz[q].v[e]), gv = mp_up(rg[q].v[e]);
          const A xh = (mp_up(ry[q].v[e]) + d * mp_up(rx[q].v[e])) * zz * sigmoid_a(zz) * rs;
          dot += gv * gn[e] * xh;
          if (NP > 0) gacc[q][e] += gv * xh;
          else atomicAdd(cols + c + e, gv * xh);
        }
      }
    }
    dot = warp_reduce<SumOp>(dot);
    const A m = dot / static_cast<A>(width);
    if (NP > 0) {
      // pass 2 decodes the packs again: without this fence the compiler keeps pass 1's converted values alive
      // (four times the registers of the packs) and spills
#pragma unroll
      for (int p = 0; p < (NP > 0 ? NP : 1); ++p) { gn_opaque(ry[p]); gn_opaque(rx[p]); gn_opaque(rz[p]); gn_opaque(rg[p]); }
    }
#pragma unroll
    for (int p = 0; p < packs; ++p) {
      const size_t c = (static_cast<size_t>(p) * 32 + lane) * V;
      if (NP > 0 || c < width) {
        const int q = NP > 0 ? p : 0;
        if (NP == 0) {
          ry[0] = *reinterpret_cast<const VecT<T, V>*>(y + r * width + c);
          rx[0] = *reinterpret_cast<const VecT<T, V>*>(x + r * width + c);
          rz[0] = *reinterpret_cast<const VecT<T, V>*>(z + r * zp + c);
          rg[0] = *reinterpret_cast<const VecT<T, V>*>(gout + r * width + c);
        }
        A gn[V], oy[V], oz[V];
        load_vec<T, V>(gain + c, gn);
        const A d = D != nullptr ? D[c / P] : A(0);
        A part = A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const A zz = mp_up(rz[q].v[e]), xv = mp_up(rx[q].v[e]);
          const A s = sigmoid_a(zz);
          const A ww = mp_up(ry[q].v[e]) + d * xv;
          const A xh = ww * zz * s * rs;
          const A gu = rs * (mp_up(rg[q].v[e]) * gn[e] - xh * m);
          oy[e] = gu * zz * s;
          oz[e] = gu * ww * (s + zz * s * (A(1) - s));
          part += oy[e] * xv;
        }
        if (NP > 0) dacc[q] += part;
        else if (gD != nullptr) atomicAdd(bins + c / P, part);
        store_vec<T, V>(gy + r * width + c, oy);
        store_vec<T, V>(gz + r * gzp + c, oz);
      }
    }
  }
  if (NP > 0) {
#pragma unroll
    for (int p = 0; p < (NP > 0 ? NP : 1); ++p) {
      const size_t c = (static_cast<size_t>(p) * 32 + lane) * V;
#pragma unroll
      for (int e = 0; e < V; ++e) atomicAdd(cols + c + e, gacc[p][e]);
      if (gD != nullptr) atomicAdd(bins + c / P, dacc[p]);
    }
  }
  __syncthreads();
  for (size_t i = threadIdx.x; i < width; i += GN_THREADS) partial[blockIdx.x * width + i] = cols[i];
  if (gD != nullptr)
    for (int h = threadIdx.x; h < H; h += GN_THREADS) atomicAdd(gD + h, bins[h]);
}

// r16 rows of 512 * NP elements: TWO warps per row (half the registers per lane, twice the warps in flight: the
// one-warp kernels above run 8 - 16 warps per SM and wait on their own loads), the row sums meet in shared memory
// behind a 64-thread named barrier.  Pack p of warp w of the pair covers columns ((2 p + w) * 32 + lane) * 8 ...
__device__ __forceinline__ void gn_pair_sync(int pair) { asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory"); }

template <int NP>
__global__ void __launch_bounds__(GN_THREADS) gate_rmsnorm_h2_kernel(const __half* __restrict__ y, const __half* __restrict__ x,
                                                                     const float* __restrict__ D, const __half* __restrict__ z, size_t zp,
                                                                     const __half* __restrict__ gain, float eps, __half* __restrict__ out,
                                                                     float* __restrict__ rstd, size_t rows, int P) {
  __shared__ float slot[2][GN_THREADS / 64][2];
  constexpr size_t width = static_cast<size_t>(NP) * 512;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, pair = warp >> 1, wsub = warp & 1;
  const size_t pairs = static_cast<size_t>(gridDim.x) * (GN_THREADS / 64);
  int parity = 0;
  for (size_t r = blockIdx.x * static_cast<size_t>(GN_THREADS / 64) + pair; r < rows; r += pairs, parity ^= 1) {
    uint4 ry[NP], rx[NP], rz[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
      ry[p] = *reinterpret_cast<const uint4*>(y + r * width + c);
      rx[p] = *reinterpret_cast<const uint4*>(x + r * width + c);
      rz[p] = *reinterpret_cast<const uint4*>(z + r * zp + c);
    }
    float t[NP][8];
    float sum = 0.f;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
      const float d = D != nullptr ? D[c / P] : 0.f;
      const __half2* hy = reinterpret_cast<const __half2*>(&ry[p]);
      const __half2* hx = reinterpret_cast<const __half2*>(&rx[p]);
      const __half2* hz = reinterpret_cast<const __half2*>(&rz[p]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fy = __half22float2(hy[q]), fx = __half22float2(hx[q]), fz = __half22float2(hz[q]);
        t[p][2 * q] = (fy.x + d * fx.x) * fz.x * sigmoid_a(fz.x);
        t[p][2 * q + 1] = (fy.y + d * fx.y) * fz.y * sigmoid_a(fz.y);
        sum += t[p][2 * q] * t[p][2 * q] + t[p][2 * q + 1] * t[p][2 * q + 1];
      }
    }
    sum = warp_reduce<SumOp>(sum);
    if (lane == 0) slot[parity][pair][wsub] = sum;
    gn_pair_sync(pair);
    sum = slot[parity][pair][0] + slot[parity][pair][1];
    const float rs = rsqrtf(sum * (1.f / static_cast<float>(width)) + eps);
    if (lane == 0 && wsub == 0 && rstd != nullptr) rstd[r] = rs;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
      const uint4 rg = *reinterpret_cast<const uint4*>(gain + c);
      const __half2* hg = reinterpret_cast<const __half2*>(&rg);
      uint4 o;
      __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fg = __half22float2(hg[q]);
        ho[q] = __floats2half2_rn(t[p][2 * q] * rs * fg.x, t[p][2 * q + 1] * rs * fg.y);
      }
      *reinterpret_cast<uint4*>(out + r * width + c) = o;
    }
  }
}

// Reverse, same layout.  The outputs are linear in the row mean m, which is only known after the row has been read:
//   gy = a1 - m b1,  gz = a2 - m b2,  with a1 = rstd gxh zs, b1 = rstd xh zs, a2 = rstd gxh w ds, b2 = rstd xh w ds
// (w = y + D x, zs = silu(z), ds = silu'(z)).  The first pass leaves a1, b1, a2, b2 as packed halves in registers (the
// size of the raw inputs) and the second pass is two packed multiply-adds per pair of elements instead of a second
// evaluation of the gate.  gD uses sum(gy x) = sum(a1 x) - m sum(b1 x) in fp32.
template <int NP>
__global__ void __launch_bounds__(GN_THREADS) gate_rmsnorm_reverse_h2_kernel(
    const __half* __restrict__ y, const __half* __restrict__ x, const float* __restrict__ D, const __half* __restrict__ z, size_t zp,
    const __half* __restrict__ gain, const float* __restrict__ rstd, const __half* __restrict__ gout, __half* __restrict__ gy,
    __half* __restrict__ gz, size_t gzp, float* __restrict__ gD, float* __restrict__ partial, size_t rows, int H, int P) {
  extern __shared__ unsigned char gn_smem[];
  float* cols = reinterpret_cast<float*>(gn_smem);
  constexpr size_t width = static_cast<size_t>(NP) * 512;
  float* bins = cols + width;
  __shared__ float slot[2][GN_THREADS / 64][2];
  for (size_t i = threadIdx.x; i < width + H; i += GN_THREADS) cols[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, pair = warp >> 1, wsub = warp & 1;
  const size_t pairs = static_cast<size_t>(gridDim.x) * (GN_THREADS / 64);
  float gacc[NP][8], dacc[NP];
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    dacc[p] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) gacc[p][e] = 0.f;
  }
  int parity = 0;
  for (size_t r = blockIdx.x * static_cast<size_t>(GN_THREADS / 64) + pair; r < rows; r += pairs, parity ^= 1) {
    const float rs = rstd[r];
    uint4 ry[NP], rx[NP], rz[NP], rg[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
      ry[p] = *reinterpret_cast<const uint4*>(y + r * width + c);
      rx[p] = *reinterpret_cast<const uint4*>(x + r * width + c);
      rz[p] = *reinterpret_cast<const uint4*>(z + r * zp + c);
      rg[p] = *reinterpret_cast<const uint4*>(gout + r * width + c);
    }
    __half2 a1[NP][4], b1[NP][4], a2[NP][4], b2[NP][4];
    float pa[NP], pb[NP];
    float dot = 0.f;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
      const float d = D != nullptr ? D[c / P] : 0.f;
      const uint4 rn = *reinterpret_cast<const uint4*>(gain + c);
      const __half2* hy = reinterpret_cast<const __half2*>(&ry[p]);
      const __half2* hx = reinterpret_cast<const __half2*>(&rx[p]);
      const __half2* hz = reinterpret_cast<const __half2*>(&rz[p]);
      const __half2* hg = reinterpret_cast<const __half2*>(&rg[p]);
      const __half2* hn = reinterpret_cast<const __half2*>(&rn);
      pa[p] = 0.f;
      pb[p] = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fy = __half22float2(hy[q]), fx = __half22float2(hx[q]), fz = __half22float2(hz[q]);
        const float2 fg = __half22float2(hg[q]), fn = __half22float2(hn[q]);
        float A1[2], B1[2], A2[2], B2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float yy = e ? fy.y : fy.x, xx = e ? fx.y : fx.x, zz = e ? fz.y : fz.x, gg = e ? fg.y : fg.x, nn = e ? fn.y : fn.x;
          const float sg = sigmoid_a(zz);
          const float zs = zz * sg;
          const float w = yy + d * xx;
          const float xh = w * zs * rs;
          const float gxh = gg * nn;
          dot += gxh * xh;
          gacc[p][2 * q + e] += gg * xh;
          const float wds = w * (sg + zs * (1.f - sg));
          const float t1 = rs * gxh, t2 = rs * xh;
          A1[e] = t1 * zs; B1[e] = t2 * zs; A2[e] = t1 * wds; B2[e] = t2 * wds;
          pa[p] += A1[e] * xx;
          pb[p] += B1[e] * xx;
        }
        a1[p][q] = __floats2half2_rn(A1[0], A1[1]);
        b1[p][q] = __floats2half2_rn(B1[0], B1[1]);
        a2[p][q] = __floats2half2_rn(A2[0], A2[1]);
        b2[p][q] = __floats2half2_rn(B2[0], B2[1]);
      }
    }
    dot = warp_reduce<SumOp>(dot);
    if (lane == 0) slot[parity][pair][wsub] = dot;
    gn_pair_sync(pair);
    const float m = (slot[parity][pair][0] + slot[parity][pair][1]) * (1.f / static_cast<float>(width));
    const __half2 nm = __float2half2_rn(-m);
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
      uint4 oy, oz;
      __half2* hy = reinterpret_cast<__half2*>(&oy);
      __half2* hz = reinterpret_cast<__half2*>(&oz);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        hy[q] = __hfma2(nm, b1[p][q], a1[p][q]);
        hz[q] = __hfma2(nm, b2[p][q], a2[p][q]);
      }
      *reinterpret_cast<uint4*>(gy + r * width + c) = oy;
      *reinterpret_cast<uint4*>(gz + r * gzp + c) = oz;
      dacc[p] += pa[p] - m * pb[p];
    }
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const size_t c = (static_cast<size_t>(2 * p + wsub) * 32 + lane) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(cols + c + e, gacc[p][e]);
    if (gD != nullptr) atomicAdd(bins + c / P, dacc[p]);
  }
  __syncthreads();
  for (size_t i = threadIdx.x; i < width; i += GN_THREADS) partial[blockIdx.x * width + i] = cols[i];
  if (gD != nullptr)
    for (int h = threadIdx.x; h < H; h += GN_THREADS) atomicAdd(gD + h, bins[h]);
}

// ggain = alpha * ggain + sum over the CTAs' partial rows (fixed order)
template <typename T>
__global__ void __launch_bounds__(1024) gate_rmsnorm_fold_kernel(const typename Acc<T>::type* __restrict__ partial, int nrows, size_t width,
                                                                 typename Acc<T>::type alpha, T* __restrict__ ggain) {
  using A = typename Acc<T>::type;
  __shared__ A part[32][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;   // 32 columns x 32 row slices: ~10 dependent additions per thread
  const size_t c = blockIdx.x * static_cast<size_t>(32) + cx;
  A sum = A(0);
  if (c < width)
    for (int r = ry; r < nrows; r += 32) sum += partial[static_cast<size_t>(r) * width + c];
  part[ry][cx] = sum;
  __syncthreads();
  if (ry == 0 && c < width) {
    A t = A(0);
#pragma unroll
    for (int q = 0; q < 32; ++q) t += part[q][cx];
    if (alpha != A(0)) t += alpha * mp_up(ggain[c]);
    ggain[c] = mp_down<T>(t);
  }
}

// gx[r, h, :] += D[h] * gy[r, h, :]
template <typename T, int V>
__global__ void __launch_bounds__(256) head_scale_accumulate_kernel(const typename Acc<T>::type* __restrict__ D,
                                                                    const T* __restrict__ gy, T* __restrict__ gx, size_t rows,
                                                                    int H, int P) {
  using A = typename Acc<T>::type;
  const size_t width = static_cast<size_t>(H) * P, per_row = width / V;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < rows * per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t c = (i % per_row) * V;
    A a[V], g[V];
    load_vec<T, V>(gx + i * V, a);
    load_vec<T, V>(gy + i * V, g);
    const A d = D[c / P];
#pragma unroll
    for (int e = 0; e < V; ++e) a[e] += d * g[e];
    store_vec<T, V>(gx + i * V, a);
  }
}

// ---------------------------------------------------------------------------
// cross-entropy over rows of logits [m, n] with integer targets:
//   loss_i = log sum_j exp(x_ij) - x_i,target;  glogits_ij = scale * (softmax_ij - [j == target])
// One CTA per row; the row is parked in shared memory when it fits (one read of
// the logits, one write of the gradient, which may alias the logits).
// ---------------------------------------------------------------------------
constexpr int CE_THREADS = 512;

template <typename T, int V, bool STAGED>
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(const T* logits, const int* __restrict__ targets,
                                                                  typename Acc<T>::type scale,
                                                                  typename Acc<T>::type* __restrict__ loss, T* glogits,
                                                                  size_t n) {
  using A = typename Acc<T>::type;
  extern __shared__ __align__(128) unsigned char ce_smem[];
  __shared__ A red[CE_THREADS / 32];
  __shared__ A bc;
  T* srow = reinterpret_cast<T*>(ce_smem);
  const size_t row = blockIdx.x;
  const T* src = logits + row * n;
  const size_t nv = n / V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto block_reduce = [&](A v, bool is_max) -> A {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const A other = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? (v > other ? v : other) : v + other;
    }
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
      A t = lane < CE_THREADS / 32 ? red[lane] : (is_max ? A(-INFINITY) : A(0));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const A other = __shfl_xor_sync(0xffffffffu, t, o);
        t = is_max ? (t > other ? t : other) : t + other;
      }
      if (lane == 0) bc = t;
    }
    __syncthreads();
    const A r = bc;
    __syncthreads();
    return r;
  };
  A mx = A(-INFINITY);
  for (size_t i = threadIdx.x; i < nv; i += CE_THREADS) {
    const VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(src + i * V);
    if (STAGED) *reinterpret_cast<VecT<T, V>*>(srow + i * V) = x;
#pragma unroll
    for (int e = 0; e < V; ++e) { const A f = mp_up(x.v[e]); mx = f > mx ? f : mx; }
  }
  mx = block_reduce(mx, true);   // (the barriers inside also publish the staged row)
  const T* rd = STAGED ? srow : src;
  const long long tg = targets[row];
  const bool valid = tg >= 0 && static_cast<size_t>(tg) < n;   // other targets: ignored row (zero loss, zero gradient)
  // (global memory still holds the logits here: an aliased gradient is only written in the last pass)
  const A x_target = (threadIdx.x == 0 && valid) ? mp_up(src[tg]) : A(0);
  A sum = A(0);
  for (size_t i = threadIdx.x; i < nv; i += CE_THREADS) {
    const VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(rd + i * V);
    VecT<T, V> ex;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const A t = exp_a(mp_up(x.v[e]) - mx);
      sum += t;
      ex.v[e] = mp_down<T>(t);
    }
    // the parked row now keeps exp(x - max) (at most one, in T): one exponential per element in total
    if (STAGED) *reinterpret_cast<VecT<T, V>*>(srow + i * V) = ex;
  }
  sum = block_reduce(sum, false);
  if (threadIdx.x == 0 && loss != nullptr) loss[row] = valid ? log_a(sum) + mx - x_target : A(0);
  if (glogits != nullptr) {
    const A inv = scale / sum;
    T* dst = glogits + row * n;
    for (size_t i = threadIdx.x; i < nv; i += CE_THREADS) {
      const VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(rd + i * V);
      VecT<T, V> o;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        A gval = A(0);
        if (valid) gval = (STAGED ? mp_up(x.v[e]) : exp_a(mp_up(x.v[e]) - mx)) * inv;
        if (valid && i * V + e == static_cast<size_t>(tg)) gval -= scale;
        o.v[e] = mp_down<T>(gval);
      }
      *reinterpret_cast<VecT<T, V>*>(dst + i * V) = o;
    }
  }
}

// Same computation with the row moved by bulk asynchronous copies: one thread asks for the whole row
// (global -> shared, completion counted on an mbarrier), the CTA makes its passes over shared memory,
// writes the gradient in place there and one thread sends it back (shared -> global).  A CTA then has
// its full row in flight at once instead of what its threads' registers can hold, and two CTAs per SM
// alternate between moving and computing.  Needs rows that are multiples of 16 bytes.
constexpr uint32_t CE_BULK_CHUNK = 32768;

template <typename T, int V>
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_bulk_kernel(const T* logits, const int* __restrict__ targets,
                                                                       typename Acc<T>::type scale,
                                                                       typename Acc<T>::type* __restrict__ loss, T* glogits,
                                                                       size_t n, uint32_t* status) {
  using A = typename Acc<T>::type;
  extern __shared__ __align__(128) unsigned char ce_smem[];
  __shared__ uint64_t bar;
  __shared__ A red[CE_THREADS / 32];
  __shared__ A bc;
  T* srow = reinterpret_cast<T*>(ce_smem);
  const size_t row = blockIdx.x;
  const T* src = logits + row * n;
  const uint32_t row_bytes = static_cast<uint32_t>(n * sizeof(T));
  const size_t nv = n / V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bar, row_bytes);
    for (uint32_t off = 0; off < row_bytes; off += CE_BULK_CHUNK)
      bulk_load_1d(ce_smem + off, reinterpret_cast<const unsigned char*>(src) + off,
                   row_bytes - off < CE_BULK_CHUNK ? row_bytes - off : CE_BULK_CHUNK, &bar);
  }
  const long long tg = targets[row];
  const bool valid = tg >= 0 && static_cast<size_t>(tg) < n;
  if (!mbar_wait(&bar, 0, status)) return;   // bounded; every thread sees the same outcome
  auto block_reduce = [&](A v, bool is_max) -> A {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const A other = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? (v > other ? v : other) : v + other;
    }
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
      A t = lane < CE_THREADS / 32 ? red[lane] : (is_max ? A(-INFINITY) : A(0));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const A other = __shfl_xor_sync(0xffffffffu, t, o);
        t = is_max ? (t > other ? t : other) : t + other;
      }
      if (lane == 0) bc = t;
    }
    __syncthreads();
    const A r = bc;
    __syncthreads();
    return r;
  };
  A mx = A(-INFINITY);
  for (size_t i = threadIdx.x; i < nv; i += CE_THREADS) {
    const VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(srow + i * V);
#pragma unroll
    for (int e = 0; e < V; ++e) { const A f = mp_up(x.v[e]); mx = f > mx ? f : mx; }
  }
  mx = block_reduce(mx, true);
  const A x_target = (threadIdx.x == 0 && valid) ? mp_up(srow[tg]) : A(0);   // read before the row is overwritten
  __syncthreads();
  A sum = A(0);
  for (size_t i = threadIdx.x; i < nv; i += CE_THREADS) {
    VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(srow + i * V);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const A t = exp_a(mp_up(x.v[e]) - mx);
      sum += t;
      x.v[e] = mp_down<T>(t);
    }
    *reinterpret_cast<VecT<T, V>*>(srow + i * V) = x;
  }
  sum = block_reduce(sum, false);
  if (threadIdx.x == 0 && loss != nullptr) loss[row] = valid ? log_a(sum) + mx - x_target : A(0);
  if (glogits == nullptr) return;
  const A inv = scale / sum;
  for (size_t i = threadIdx.x; i < nv; i += CE_THREADS) {
    VecT<T, V> x = *reinterpret_cast<const VecT<T, V>*>(srow + i * V);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      A gval = valid ? mp_up(x.v[e]) * inv : A(0);
      if (valid && i * V + e == static_cast<size_t>(tg)) gval -= scale;
      x.v[e] = mp_down<T>(gval);
    }
    *reinterpret_cast<VecT<T, V>*>(srow + i * V) = x;
  }
  fence_proxy_async_smem();   // generic-proxy writes of the gradient -> visible to the bulk store
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned char* dst = reinterpret_cast<unsigned char*>(glogits + row * n);
    for (uint32_t off = 0; off < row_bytes; off += CE_BULK_CHUNK)
      bulk_store_1d(dst + off, ce_smem + off, row_bytes - off < CE_BULK_CHUNK ? row_bytes - off : CE_BULK_CHUNK);
    bulk_commit();
    bulk_wait_all<0>();       // shared memory must outlive the copy
  }
}

// ---------------------------------------------------------------------------
// small element-wise helpers
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) neg_exp_kernel(const T* __restrict__ src, T* __restrict__ dst, size_t n) {
  using A = typename Acc<T>::type;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = mp_down<T>(-exp_a(static_cast<A>(mp_up(src[i]))));
}

// dst(r32) = src(r16) + beta * dst
template <int V>
__global__ void __launch_bounds__(512) convert_r16_r32_kernel(const __half* __restrict__ src, float* __restrict__ dst, float beta,
                                                              size_t n) {
  const size_t nv = n / V;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float a[V], o[V];
    load_vec<__half, V>(src + i * V, a);
    if (beta != 0.f) {
      load_vec<float, V>(dst + i * V, o);
#pragma unroll
      for (int e = 0; e < V; ++e) a[e] += beta * o[e];
    }
    store_vec<float, V>(dst + i * V, a);
  }
}
template <int V>
__global__ void __launch_bounds__(512) convert_r32_r16_kernel(const float* __restrict__ src, __half* __restrict__ dst, size_t n) {
  const size_t nv = n / V;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float a[V];
    load_vec<float, V>(src + i * V, a);
    store_vec<__half, V>(dst + i * V, a);
  }
}

// Mixed-precision Adam over a flat bucket (see launch_adam_mixed_r32).  The step-dependent bias corrections come
// from device memory, so a captured graph can replay the call for every step.
struct AdamTick { float inv_bc1, inv_bc2; uint32_t step, nonfinite; };
__global__ void adam_tick_kernel(AdamTick* t, float beta1, float beta2) {
  const uint32_t step = t->step + 1;
  t->step = step;
  t->inv_bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  t->inv_bc2 = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
}
template <int V>
__global__ void __launch_bounds__(512) adam_mixed_kernel(float* __restrict__ w32, __half* __restrict__ w16, const float* __restrict__ g32,
                                                         const __half* __restrict__ g16, float* __restrict__ m, float* __restrict__ v,
                                                         float lr, float b1, float b2, float eps, float gscale, AdamTick* tick, size_t n) {
  const float ib1 = tick->inv_bc1, ib2 = tick->inv_bc2;
  const size_t nv = n / V;
  bool bad = false;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float w[V], g[V], mm[V], vv[V], h[V];
    load_vec<float, V>(w32 + i * V, w);
    load_vec<float, V>(g32 + i * V, g);
    load_vec<float, V>(m + i * V, mm);
    load_vec<float, V>(v + i * V, vv);
    if (g16 != nullptr) {
      load_vec<__half, V>(g16 + i * V, h);
#pragma unroll
      for (int e = 0; e < V; ++e) g[e] += h[e];
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float gs = g[e] * gscale;
      if (!isfinite(gs)) { bad = true; continue; }      // an overflowed gradient leaves this element untouched
      mm[e] = b1 * mm[e] + (1.f - b1) * gs;
      vv[e] = b2 * vv[e] + (1.f - b2) * gs * gs;
      w[e] -= lr * (mm[e] * ib1) / (sqrtf(vv[e] * ib2) + eps);
    }
    store_vec<float, V>(w32 + i * V, w);
    store_vec<float, V>(m + i * V, mm);
    store_vec<float, V>(v + i * V, vv);
    store_vec<__half, V>(w16 + i * V, w);
  }
  if (bad) tick->nonfinite = 1u;
}

inline unsigned grid_for(size_t work_items, int threads) {
  const size_t g = (work_items + threads - 1) / threads;
  return static_cast<unsigned>(g < 1 ? 1 : (g > (1u << 30) ? (1u << 30) : g));
}

// ------------------------------- launch bodies ------------------------------
template <typename T>
void embedding_impl(const void* table, const void* ids, void* out, len_t n, len_t dim, len_t vocab, StreamContext ctx) {
  if (n == 0 || dim == 0) return;
  constexpr int PN = Pack<T>::N;
  cudaStream_t st = mp_stream(ctx);
  if (dim % PN == 0 && mp_aligned16(table) && mp_aligned16(out))
    embedding_kernel<T, PN><<<grid_for(n * (dim / PN), 256), 256, 0, st>>>(static_cast<const T*>(table), static_cast<const int*>(ids),
                                                                         static_cast<T*>(out), n, dim, vocab);
  else
    embedding_kernel<T, 1><<<grid_for(n * dim, 256), 256, 0, st>>>(static_cast<const T*>(table), static_cast<const int*>(ids),
                                                                 static_cast<T*>(out), n, dim, vocab);
  MP_LAUNCH_CHECK();
}

template <typename T>
void embedding_reverse_impl(const void* ids, const void* gy, void* gtable, len_t n, len_t dim, len_t vocab, StreamContext ctx) {
  if (n == 0 || dim == 0) return;
  using A = typename Acc<T>::type;
  embedding_reverse_kernel<T><<<grid_for(n * dim, 256), 256, 0, mp_stream(ctx)>>>(static_cast<const int*>(ids), static_cast<const T*>(gy),
                                                                              static_cast<A*>(gtable), n, dim, vocab);
  MP_LAUNCH_CHECK();
}

template <typename T, int V>
void conv_forward_dispatch(const T* x, size_t xp, const T* w, const T* bias, T* y, size_t yp, len_t batch, len_t len, len_t channels,
                           len_t width, cudaStream_t st) {
  const dim3 block(32, CONV_TY);
  const size_t steps_per_cta = static_cast<size_t>(CONV_TY) * CONV_LT;
  const dim3 grid(static_cast<unsigned>((channels / V + 31) / 32), static_cast<unsigned>((len + steps_per_cta - 1) / steps_per_cta),
                  static_cast<unsigned>(batch));
  const int L = static_cast<int>(len), C = static_cast<int>(channels);
  switch (width) {
    case 2: conv1d_silu_kernel<T, V, 2><<<grid, block, 0, st>>>(x, xp, w, bias, y, yp, L, C); break;
    case 3: conv1d_silu_kernel<T, V, 3><<<grid, block, 0, st>>>(x, xp, w, bias, y, yp, L, C); break;
    case 4: conv1d_silu_kernel<T, V, 4><<<grid, block, 0, st>>>(x, xp, w, bias, y, yp, L, C); break;
    default: MP_FATAL("causal_conv1d_silu: kernel width %llu is not supported (2, 3 or 4)", static_cast<unsigned long long>(width));
  }
  MP_LAUNCH_CHECK();
}

template <typename T, int V>
void conv_reverse_dispatch(const T* x, size_t xp, const T* w, const T* bias, const T* gy, size_t gyp, T* gx, size_t gxp,
                           typename Acc<T>::type* gw, typename Acc<T>::type* gbias, len_t batch, len_t len, len_t channels, len_t width,
                           cudaStream_t st) {
  const dim3 block(32, CONV_TY);
  const size_t steps_per_cta = static_cast<size_t>(CONV_TY) * CONV_LT * CONV_NB;
  const dim3 grid(static_cast<unsigned>((channels / V + 31) / 32), static_cast<unsigned>((len + steps_per_cta - 1) / steps_per_cta),
                  static_cast<unsigned>(batch));
  const int L = static_cast<int>(len), C = static_cast<int>(channels);
  switch (width) {
    case 2: conv1d_silu_reverse_kernel<T, V, 2><<<grid, block, 0, st>>>(x, xp, w, bias, gy, gyp, gx, gxp, gw, gbias, L, C); break;
    case 3: conv1d_silu_reverse_kernel<T, V, 3><<<grid, block, 0, st>>>(x, xp, w, bias, gy, gyp, gx, gxp, gw, gbias, L, C); break;
    case 4: conv1d_silu_reverse_kernel<T, V, 4><<<grid, block, 0, st>>>(x, xp, w, bias, gy, gyp, gx, gxp, gw, gbias, L, C); break;
    default: MP_FATAL("causal_conv1d_silu_reverse: kernel width %llu is not supported (2, 3 or 4)", static_cast<unsigned long long>(width));
  }
  MP_LAUNCH_CHECK();
}

// Segment table for the tiled r16 kernels; false when a segment does not allow 16-byte accesses.
static bool conv_make_segs(ConvSegs& sg, const void* const* bufs, const len_t* pitches, const len_t* counts, len_t nseg) {
  if (nseg == 0 || nseg > CONV_MAX_SEGS) return false;
  sg.nseg = static_cast<int>(nseg);
  int blk = 0, ch = 0;
  for (int i = 0; i < sg.nseg; ++i) {
    if (!vec_ok<__half>(bufs[i], pitches[i], counts[i]) || counts[i] == 0) return false;
    sg.blk_begin[i] = blk;
    sg.ch_begin[i] = ch;
    sg.ch_count[i] = static_cast<int>(counts[i]);
    sg.ptr[i] = bufs[i];
    sg.pitch[i] = pitches[i];
    sg.skip_ptr[i] = nullptr; sg.skip_pitch[i] = 0; sg.skip_scale[i] = nullptr;
    blk += static_cast<int>((counts[i] + CT_C - 1) / CT_C);
    ch += static_cast<int>(counts[i]);
  }
  for (int i = sg.nseg; i <= CONV_MAX_SEGS; ++i) sg.blk_begin[i] = blk;
  for (int i = sg.nseg; i < CONV_MAX_SEGS; ++i) { sg.skip_ptr[i] = nullptr; sg.skip_pitch[i] = 0; sg.skip_scale[i] = nullptr; }
  sg.skip_group = 1;
  return true;
}
static dim3 conv_tiled_grid(const ConvSegs& sg, len_t len, len_t batch, int* tiles_per_cta) {
  const size_t ltiles = (len + CT_L - 1) / CT_L;
  size_t per = ltiles >= 2 ? 2 : 1;   // time tiles per CTA (measured best of 1, 2, 4, 8 at 1536 and 128 channels)
  if (const char* e = getenv("MP_CONV_TILES_PER_CTA")) { const long v = strtol(e, nullptr, 10); if (v >= 1 && v <= 64) per = static_cast<size_t>(v); }
  *tiles_per_cta = static_cast<int>(per);
  return dim3(static_cast<unsigned>(sg.blk_begin[sg.nseg]), static_cast<unsigned>((ltiles + per - 1) / per), static_cast<unsigned>(batch));
}
static bool conv_tiles_enabled(len_t width) { return width >= 2 && width <= 4 && !getenv("MP_CONV_NO_TILES"); }
static void conv_tiled_forward(const void* x, len_t x_pitch, const void* w, const void* bias, const ConvSegs& sg, len_t batch, len_t len,
                               len_t width, StreamContext ctx) {
  int tp = 1;
  const dim3 grid = conv_tiled_grid(sg, len, batch, &tp);
  const int L = static_cast<int>(len);
  cudaStream_t st = mp_stream(ctx);
  const __half* xh = static_cast<const __half*>(x); const __half* wh = static_cast<const __half*>(w);
  const __half* bh = static_cast<const __half*>(bias);
  if (width == 4) conv1d_silu_tiled_kernel<4><<<grid, CT_THREADS, 0, st>>>(xh, x_pitch, wh, bh, sg, L, tp);
  else if (width == 3) conv1d_silu_tiled_kernel<3><<<grid, CT_THREADS, 0, st>>>(xh, x_pitch, wh, bh, sg, L, tp);
  else conv1d_silu_tiled_kernel<2><<<grid, CT_THREADS, 0, st>>>(xh, x_pitch, wh, bh, sg, L, tp);
  MP_LAUNCH_CHECK();
}
static void conv_tiled_reverse(const void* x, len_t x_pitch, const void* w, const void* bias, const ConvSegs& sg, void* gx, len_t gx_pitch,
                               void* gw, void* gbias, len_t batch, len_t len, len_t width, StreamContext ctx) {
  int tp = 1;
  const dim3 grid = conv_tiled_grid(sg, len, batch, &tp);
  const int L = static_cast<int>(len);
  cudaStream_t st = mp_stream(ctx);
  const __half* xh = static_cast<const __half*>(x); const __half* wh = static_cast<const __half*>(w);
  const __half* bh = static_cast<const __half*>(bias);
  __half* gxh = static_cast<__half*>(gx);
  float* gwf = static_cast<float*>(gw); float* gbf = static_cast<float*>(gbias);
  bool skip = false;
  for (int i = 0; i < sg.nseg; ++i) skip = skip || sg.skip_ptr[i] != nullptr;
#define CONV_REV(WV, SK)                                                                                                            \
  do {                                                                                                                              \
    constexpr int HV = WV - 1;                                                                                                      \
    constexpr int NB = SK ? 1 : 2;                                                                                                  \
    const size_t smem = sizeof(__half) * (NB * (CT_L + 2 * HV) * CT_C + NB * (CT_L + HV) * CT_C + CT_L * CT_C) +                     \
                        sizeof(float) * CT_LANES * CT_C * (WV + 1) + (SK ? sizeof(__half) * (CT_L + HV) * CT_C : 0);                 \
    if (smem > 48 * 1024)                                                                                                           \
      MP_CUDA_CHECK(cudaFuncSetAttribute(conv1d_silu_reverse_tiled_kernel<WV, SK>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                         static_cast<int>(smem)));                                                                  \
    conv1d_silu_reverse_tiled_kernel<WV, SK><<<grid, CT_THREADS, smem, st>>>(xh, x_pitch, wh, bh, sg, gxh, gx_pitch, gwf, gbf, L, tp); \
  } while (0)
  if (skip) { if (width == 4) CONV_REV(4, true); else if (width == 3) CONV_REV(3, true); else CONV_REV(2, true); }
  else { if (width == 4) CONV_REV(4, false); else if (width == 3) CONV_REV(3, false); else CONV_REV(2, false); }
#undef CONV_REV
  MP_LAUNCH_CHECK();
}

template <typename T>
void causal_conv1d_silu_impl(const void* x, len_t x_pitch, const void* w, const void* bias, void* y, len_t y_pitch, len_t batch,
                             len_t len, len_t channels, len_t width, StreamContext ctx) {
  if (batch == 0 || len == 0 || channels == 0) return;
  constexpr int PN = Pack<T>::N;
  const bool v = vec_ok<T>(x, x_pitch, channels) && vec_ok<T>(y, y_pitch, channels);
  if constexpr (std::is_same<T, __half>::value) {
    ConvSegs sg;
    const void* bufs[1] = {y};
    if (v && conv_tiles_enabled(width) && conv_make_segs(sg, bufs, &y_pitch, &channels, 1)) {
      conv_tiled_forward(x, x_pitch, w, bias, sg, batch, len, width, ctx);
      return;
    }
  }
  if (v) conv_forward_dispatch<T, PN>(static_cast<const T*>(x), x_pitch, static_cast<const T*>(w), static_cast<const T*>(bias), static_cast<T*>(y),
                                      y_pitch, batch, len, channels, width, mp_stream(ctx));
  else conv_forward_dispatch<T, 1>(static_cast<const T*>(x), x_pitch, static_cast<const T*>(w), static_cast<const T*>(bias), static_cast<T*>(y),
                                   y_pitch, batch, len, channels, width, mp_stream(ctx));
}

template <typename T>
void causal_conv1d_silu_reverse_impl(const void* x, len_t x_pitch, const void* w, const void* bias, const void* gy, len_t gy_pitch,
                                     void* gx, len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t channels,
                                     len_t width, StreamContext ctx) {
  if (batch == 0 || len == 0 || channels == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  constexpr int RV = PN > 4 ? 2 : PN;   // at most 4 channels per thread (register footprint)
  const bool v = vec_ok<T>(x, x_pitch, channels) && vec_ok<T>(gy, gy_pitch, channels) && vec_ok<T>(gx, gx_pitch, channels);
  if constexpr (std::is_same<T, __half>::value) {
    ConvSegs sg;
    const void* bufs[1] = {gy};
    if (v && conv_tiles_enabled(width) && conv_make_segs(sg, bufs, &gy_pitch, &channels, 1)) {
      conv_tiled_reverse(x, x_pitch, w, bias, sg, gx, gx_pitch, gw, gbias, batch, len, width, ctx);
      return;
    }
  }
  if (v) conv_reverse_dispatch<T, RV>(static_cast<const T*>(x), x_pitch, static_cast<const T*>(w), static_cast<const T*>(bias),
                                      static_cast<const T*>(gy), gy_pitch, static_cast<T*>(gx), gx_pitch, static_cast<A*>(gw),
                                      static_cast<A*>(gbias), batch, len, channels, width, mp_stream(ctx));
  else conv_reverse_dispatch<T, 1>(static_cast<const T*>(x), x_pitch, static_cast<const T*>(w), static_cast<const T*>(bias),
                                   static_cast<const T*>(gy), gy_pitch, static_cast<T*>(gx), gx_pitch, static_cast<A*>(gw),
                                   static_cast<A*>(gbias), batch, len, channels, width, mp_stream(ctx));
}

// Segmented forms: the convolution covers sum(seg_channels) consecutive channels of x (w, bias, gx, gw, gbias are indexed
// by that channel), segment i writes y (reads gy) in its own buffer ys[i] / gys[i] with pitch pitches[i].  One launch on
// the tiled r16 path, otherwise one launch per segment.
template <typename T>
void causal_conv1d_silu_segments_impl(const void* x, len_t x_pitch, const void* w, const void* bias, void* const* ys, const len_t* y_pitches,
                                      const len_t* seg_channels, len_t nseg, len_t batch, len_t len, len_t width, StreamContext ctx) {
  if (batch == 0 || len == 0 || nseg == 0) return;
  if (ys == nullptr || y_pitches == nullptr || seg_channels == nullptr) MP_FATAL("causal_conv1d_silu_segments: the segment arrays are host arrays of nseg entries");
  len_t total = 0;
  for (len_t i = 0; i < nseg; ++i) total += seg_channels[i];
  if constexpr (std::is_same<T, __half>::value) {
    ConvSegs sg;
    if (vec_ok<T>(x, x_pitch, total) && conv_tiles_enabled(width) &&
        conv_make_segs(sg, const_cast<const void* const*>(ys), y_pitches, seg_channels, nseg)) {
      conv_tiled_forward(x, x_pitch, w, bias, sg, batch, len, width, ctx);
      return;
    }
  }
  len_t c0 = 0;
  for (len_t i = 0; i < nseg; ++i) {
    causal_conv1d_silu_impl<T>(static_cast<const T*>(x) + c0, x_pitch, static_cast<const T*>(w) + c0 * width,
                               bias ? static_cast<const T*>(bias) + c0 : nullptr, ys[i], y_pitches[i], batch, len, seg_channels[i], width, ctx);
    c0 += seg_channels[i];
  }
}
template <typename T>
void causal_conv1d_silu_segments_reverse_impl(const void* x, len_t x_pitch, const void* w, const void* bias, const void* const* gys,
                                              const len_t* gy_pitches, const len_t* seg_channels, len_t nseg, void* gx, len_t gx_pitch,
                                              void* gw, void* gbias, len_t batch, len_t len, len_t width, StreamContext ctx) {
  if (batch == 0 || len == 0 || nseg == 0) return;
  using A = typename Acc<T>::type;
  if (gys == nullptr || gy_pitches == nullptr || seg_channels == nullptr) MP_FATAL("causal_conv1d_silu_segments_reverse: the segment arrays are host arrays of nseg entries");
  len_t total = 0;
  for (len_t i = 0; i < nseg; ++i) total += seg_channels[i];
  if constexpr (std::is_same<T, __half>::value) {
    ConvSegs sg;
    if (vec_ok<T>(x, x_pitch, total) && vec_ok<T>(gx, gx_pitch, total) && conv_tiles_enabled(width) &&
        conv_make_segs(sg, gys, gy_pitches, seg_channels, nseg)) {
      conv_tiled_reverse(x, x_pitch, w, bias, sg, gx, gx_pitch, gw, gbias, batch, len, width, ctx);
      return;
    }
  }
  len_t c0 = 0;
  for (len_t i = 0; i < nseg; ++i) {
    causal_conv1d_silu_reverse_impl<T>(static_cast<const T*>(x) + c0, x_pitch, static_cast<const T*>(w) + c0 * width,
                                       bias ? static_cast<const T*>(bias) + c0 : nullptr, gys[i], gy_pitches[i], static_cast<T*>(gx) + c0, gx_pitch,
                                       static_cast<A*>(gw) + c0 * width, gbias ? static_cast<A*>(gbias) + c0 : nullptr, batch, len,
                                       seg_channels[i], width, ctx);
    c0 += seg_channels[i];
  }
}

template <typename T>
void head_scale_accumulate_impl(const void* D, const void* gy, void* gx, len_t rows, len_t heads, len_t headdim, StreamContext ctx);

// The same with a second upstream term on chosen segments: gy_total = gys[i] + scale_i[channel / group] * skips[i]
// (skips[i] NULL: none).  One launch on the tiled r16 path; elsewhere the term is first added into gys[i] in place
// (the upstream buffers of segments with a skip term are unspecified afterwards).
template <typename T>
void causal_conv1d_silu_segments_reverse_skip_impl(const void* x, len_t x_pitch, const void* w, const void* bias, const void* const* gys,
                                                   const len_t* gy_pitches, const len_t* seg_channels, len_t nseg, const void* const* skips,
                                                   const len_t* skip_pitches, const void* const* skip_scales, len_t skip_group, void* gx,
                                                   len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t width,
                                                   StreamContext ctx) {
  if (batch == 0 || len == 0 || nseg == 0) return;
  if (gys == nullptr || gy_pitches == nullptr || seg_channels == nullptr || skips == nullptr || skip_pitches == nullptr || skip_scales == nullptr ||
      skip_group == 0)
    MP_FATAL("causal_conv1d_silu_segments_reverse_skip: the segment arrays are host arrays of nseg entries, skip_group > 0");
  len_t total = 0;
  for (len_t i = 0; i < nseg; ++i) total += seg_channels[i];
  if constexpr (std::is_same<T, __half>::value) {
    ConvSegs sg;
    bool ok = vec_ok<T>(x, x_pitch, total) && vec_ok<T>(gx, gx_pitch, total) && conv_tiles_enabled(width) &&
              conv_make_segs(sg, gys, gy_pitches, seg_channels, nseg) && skip_group % 2 == 0;
    for (len_t i = 0; ok && i < nseg; ++i)
      if (skips[i] != nullptr) ok = vec_ok<T>(skips[i], skip_pitches[i], seg_channels[i]) && skip_scales[i] != nullptr;
    if (ok) {
      for (len_t i = 0; i < nseg; ++i) {
        sg.skip_ptr[i] = skips[i];
        sg.skip_pitch[i] = skip_pitches[i];
        sg.skip_scale[i] = static_cast<const float*>(skip_scales[i]);
      }
      sg.skip_group = static_cast<int>(skip_group);
      conv_tiled_reverse(x, x_pitch, w, bias, sg, gx, gx_pitch, gw, gbias, batch, len, width, ctx);
      return;
    }
  }
  for (len_t i = 0; i < nseg; ++i) {
    if (skips[i] == nullptr) continue;
    if (gy_pitches[i] != seg_channels[i] || skip_pitches[i] != seg_channels[i] || seg_channels[i] % skip_group != 0)
      MP_FATAL("causal_conv1d_silu_segments_reverse_skip: outside the tiled r16 path a skip term needs densely packed buffers");
    head_scale_accumulate_impl<T>(skip_scales[i], skips[i], const_cast<void*>(gys[i]), batch * len, seg_channels[i] / skip_group, skip_group, ctx);
  }
  causal_conv1d_silu_segments_reverse_impl<T>(x, x_pitch, w, bias, gys, gy_pitches, seg_channels, nseg, gx, gx_pitch, gw, gbias, batch, len, width,
                                              ctx);
}

template <typename T>
void softplus_bias_impl(const void* raw, len_t raw_pitch, const void* bias, void* out, len_t rows, len_t heads, StreamContext ctx) {
  if (rows == 0 || heads == 0) return;
  using A = typename Acc<T>::type;
  softplus_bias_kernel<T><<<grid_for(rows * heads, 256), 256, 0, mp_stream(ctx)>>>(static_cast<const T*>(raw), raw_pitch, static_cast<const A*>(bias),
                                                                               static_cast<A*>(out), rows, static_cast<int>(heads));
  MP_LAUNCH_CHECK();
}

template <typename T>
void softplus_bias_reverse_impl(const void* raw, len_t raw_pitch, const void* bias, const void* gdt, void* graw, len_t graw_pitch,
                                void* gbias, len_t rows, len_t heads, StreamContext ctx) {
  if (rows == 0 || heads == 0) return;
  using A = typename Acc<T>::type;
  if (heads <= 256) {
    const int RR = static_cast<int>(256 / heads);
    size_t ctas = (rows + static_cast<size_t>(RR) * 4 - 1) / (static_cast<size_t>(RR) * 4);   // about four rows per thread
    const size_t cap = static_cast<size_t>(mp_sm_count(ctx)) * 8;
    if (ctas > cap) ctas = cap;
    softplus_bias_reverse_heads_kernel<T><<<static_cast<unsigned>(ctas < 1 ? 1 : ctas), 256, 0, mp_stream(ctx)>>>(
        static_cast<const T*>(raw), raw_pitch, static_cast<const A*>(bias), static_cast<const A*>(gdt), static_cast<T*>(graw), graw_pitch,
        static_cast<A*>(gbias), rows, static_cast<int>(heads), RR);
    MP_LAUNCH_CHECK();
    return;
  }
  // few, fat CTAs: each one ends with `heads` global atomics
  const unsigned grid = grid_for((rows * heads + 15) / 16, 256);
  softplus_bias_reverse_kernel<T><<<grid, 256, heads * sizeof(A), mp_stream(ctx)>>>(
      static_cast<const T*>(raw), raw_pitch, static_cast<const A*>(bias), static_cast<const A*>(gdt), static_cast<T*>(graw), graw_pitch,
      static_cast<A*>(gbias), rows, static_cast<int>(heads));
  MP_LAUNCH_CHECK();
}

template <typename T>
void ssd_gate_impl(const void* y, const void* x, const void* D, const void* z, len_t z_pitch, void* u, len_t rows, len_t heads,
                   len_t headdim, StreamContext ctx) {
  if (rows == 0 || heads == 0 || headdim == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t width = heads * headdim;
  const bool v = headdim % PN == 0 && vec_ok<T>(z, z_pitch, width) && mp_aligned16(y) && mp_aligned16(x) && mp_aligned16(u);
  cudaStream_t st = mp_stream(ctx);
  if (v) ssd_gate_kernel<T, PN><<<grid_for(rows * (width / PN), 256), 256, 0, st>>>(static_cast<const T*>(y), static_cast<const T*>(x), static_cast<const A*>(D),
                                                                                 static_cast<const T*>(z), z_pitch, static_cast<T*>(u), rows,
                                                                                 static_cast<int>(heads), static_cast<int>(headdim));
  else ssd_gate_kernel<T, 1><<<grid_for(rows * width, 256), 256, 0, st>>>(static_cast<const T*>(y), static_cast<const T*>(x), static_cast<const A*>(D),
                                                                        static_cast<const T*>(z), z_pitch, static_cast<T*>(u), rows,
                                                                        static_cast<int>(heads), static_cast<int>(headdim));
  MP_LAUNCH_CHECK();
}

template <typename T>
void ssd_gate_reverse_impl(const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gu, void* gy, void* gz,
                           len_t gz_pitch, void* gD, len_t rows, len_t heads, len_t headdim, StreamContext ctx) {
  if (rows == 0 || heads == 0 || headdim == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t width = heads * headdim;
  const bool v = headdim % PN == 0 && vec_ok<T>(z, z_pitch, width) && vec_ok<T>(gz, gz_pitch, width) && mp_aligned16(y) &&
                 mp_aligned16(x) && mp_aligned16(gu) && mp_aligned16(gy);
  cudaStream_t st = mp_stream(ctx);
  const size_t smem = heads * sizeof(A);
  if (v) ssd_gate_reverse_kernel<T, PN><<<grid_for((rows * (width / PN) + 7) / 8, 256), 256, smem, st>>>(
        static_cast<const T*>(y), static_cast<const T*>(x), static_cast<const A*>(D), static_cast<const T*>(z), z_pitch, static_cast<const T*>(gu),
        static_cast<T*>(gy), static_cast<T*>(gz), gz_pitch, static_cast<A*>(gD), rows, static_cast<int>(heads), static_cast<int>(headdim));
  else ssd_gate_reverse_kernel<T, 1><<<grid_for((rows * width + 7) / 8, 256), 256, smem, st>>>(
        static_cast<const T*>(y), static_cast<const T*>(x), static_cast<const A*>(D), static_cast<const T*>(z), z_pitch, static_cast<const T*>(gu),
        static_cast<T*>(gy), static_cast<T*>(gz), gz_pitch, static_cast<A*>(gD), rows, static_cast<int>(heads), static_cast<int>(headdim));
  MP_LAUNCH_CHECK();
}

inline unsigned gate_rmsnorm_grid(size_t rows, int sms) {
  const size_t want = (rows + GN_THREADS / 32 - 1) / (GN_THREADS / 32);
  const size_t cap = 2 * static_cast<size_t>(sms);   // one partial row of gain gradients per CTA
  return static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap));
}

// packs per lane when the whole row fits the register plan (0: it does not)
template <typename T>
int gate_rmsnorm_packs(size_t width, bool aligned) {
  constexpr size_t PN = Pack<T>::N;
  if (!aligned || width % (32 * PN) != 0) return 0;
  const size_t np = width / (32 * PN);
  return np <= (sizeof(T) == 2 ? 6 : 8) ? static_cast<int>(np) : 0;   // r16 beyond 6 packs: the register plan spills
}

template <typename T>
void ssd_gate_rmsnorm_impl(const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gain, double eps, void* out,
                           void* rstd, len_t rows, len_t heads, len_t headdim, StreamContext ctx) {
  if (rows == 0 || heads == 0 || headdim == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t width = heads * headdim;
  const bool v = headdim % PN == 0 && vec_ok<T>(z, z_pitch, width) && mp_aligned16(y) && mp_aligned16(x) && mp_aligned16(out) && mp_aligned16(gain);
  cudaStream_t st = mp_stream(ctx);
  if constexpr (std::is_same<T, __half>::value) {
    if (v && width % 512 == 0 && width / 512 <= 4 && headdim % 8 == 0 && getenv("MP_GATED_NORM_ONE_WARP") == nullptr) {
      const unsigned g2 = grid_for(rows * 64, GN_THREADS);
#define GN_FWD2(NPV)                                                                                                                 \
  gate_rmsnorm_h2_kernel<NPV><<<g2, GN_THREADS, 0, st>>>(static_cast<const __half*>(y), static_cast<const __half*>(x),               \
                                                         static_cast<const float*>(D), static_cast<const __half*>(z), z_pitch,      \
                                                         static_cast<const __half*>(gain), static_cast<float>(eps),                 \
                                                         static_cast<__half*>(out), static_cast<float*>(rstd), rows, static_cast<int>(headdim))
      switch (width / 512) {
        case 1: GN_FWD2(1); break;
        case 2: GN_FWD2(2); break;
        case 3: GN_FWD2(3); break;
        default: GN_FWD2(4); break;
      }
#undef GN_FWD2
      MP_LAUNCH_CHECK();
      return;
    }
  }
  const unsigned grid = grid_for(rows * 32, GN_THREADS);
#define GN_FWD(VV, NPV)                                                                                                              \
  gate_rmsnorm_kernel<T, VV, NPV><<<grid, GN_THREADS, 0, st>>>(static_cast<const T*>(y), static_cast<const T*>(x), static_cast<const A*>(D), \
                                                               static_cast<const T*>(z), z_pitch, static_cast<const T*>(gain), static_cast<A>(eps), \
                                                               static_cast<T*>(out), static_cast<A*>(rstd), rows, static_cast<int>(heads),   \
                                                               static_cast<int>(headdim))
  switch (gate_rmsnorm_packs<T>(width, v)) {
    case 1: GN_FWD(PN, 1); break;
    case 2: GN_FWD(PN, 2); break;
    case 3: GN_FWD(PN, 3); break;
    case 4: GN_FWD(PN, 4); break;
    case 5: GN_FWD(PN, 5); break;
    case 6: GN_FWD(PN, 6); break;
    case 7: GN_FWD(PN, 7); break;
    case 8: GN_FWD(PN, 8); break;
    default:
      if (v) GN_FWD(PN, 0);
      else GN_FWD(1, 0);
  }
#undef GN_FWD
  MP_LAUNCH_CHECK();
}

template <typename T>
void ssd_gate_rmsnorm_reverse_impl(const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gain, const void* rstd,
                                   const void* gout, void* gy, void* gz, len_t gz_pitch, void* gD, void* ggain, double alpha, void* scratch,
                                   len_t rows, len_t heads, len_t headdim, StreamContext ctx) {
  if (rows == 0 || heads == 0 || headdim == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t width = heads * headdim;
  const bool v = headdim % PN == 0 && vec_ok<T>(z, z_pitch, width) && vec_ok<T>(gz, gz_pitch, width) && mp_aligned16(y) && mp_aligned16(x) &&
                 mp_aligned16(gout) && mp_aligned16(gy) && mp_aligned16(gain);
  cudaStream_t st = mp_stream(ctx);
  const unsigned grid = gate_rmsnorm_grid(rows, mp_sm_count(ctx));
  const size_t smem = (width + heads) * sizeof(A);
  if (smem > 200 * 1024) MP_FATAL("ssd_gate_rmsnorm_reverse: row too wide for the shared-memory accumulators");
  bool launched = false;
  if constexpr (std::is_same<T, __half>::value) {
    if (v && width % 512 == 0 && width / 512 <= 4 && headdim % 8 == 0 && getenv("MP_GATED_NORM_ONE_WARP") == nullptr) {
#define GN_REV2(NPV)                                                                                                                 \
  gate_rmsnorm_reverse_h2_kernel<NPV><<<grid, GN_THREADS, smem, st>>>(                                                               \
      static_cast<const __half*>(y), static_cast<const __half*>(x), static_cast<const float*>(D), static_cast<const __half*>(z), z_pitch, \
      static_cast<const __half*>(gain), static_cast<const float*>(rstd), static_cast<const __half*>(gout), static_cast<__half*>(gy),   \
      static_cast<__half*>(gz), gz_pitch, static_cast<float*>(gD), static_cast<float*>(scratch), rows, static_cast<int>(heads),        \
      static_cast<int>(headdim))
      switch (width / 512) {
        case 1: GN_REV2(1); break;
        case 2: GN_REV2(2); break;
        case 3: GN_REV2(3); break;
        default: GN_REV2(4); break;
      }
#undef GN_REV2
      launched = true;
    }
  }
#define GN_REV(VV, NPV)                                                                                                              \
  do {                                                                                                                               \
    if (smem > 48 * 1024)                                                                                                            \
      MP_CUDA_CHECK(cudaFuncSetAttribute(gate_rmsnorm_reverse_kernel<T, VV, NPV>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                         static_cast<int>(smem)));                                                                   \
    gate_rmsnorm_reverse_kernel<T, VV, NPV><<<grid, GN_THREADS, smem, st>>>(                                                         \
        static_cast<const T*>(y), static_cast<const T*>(x), static_cast<const A*>(D), static_cast<const T*>(z), z_pitch,             \
        static_cast<const T*>(gain), static_cast<const A*>(rstd), static_cast<const T*>(gout), static_cast<T*>(gy), static_cast<T*>(gz), \
        gz_pitch, static_cast<A*>(gD), static_cast<A*>(scratch), rows, static_cast<int>(heads), static_cast<int>(headdim));          \
  } while (0)
  if (!launched) switch (gate_rmsnorm_packs<T>(width, v)) {
    case 1: GN_REV(PN, 1); break;
    case 2: GN_REV(PN, 2); break;
    case 3: GN_REV(PN, 3); break;
    case 4: GN_REV(PN, 4); break;
    case 5: GN_REV(PN, 5); break;
    case 6: GN_REV(PN, 6); break;
    case 7: GN_REV(PN, 7); break;
    case 8: GN_REV(PN, 8); break;
    default:
      if (v) GN_REV(PN, 0);
      else GN_REV(1, 0);
  }
#undef GN_REV
  MP_LAUNCH_CHECK();
  if (ggain != nullptr) {
    gate_rmsnorm_fold_kernel<T><<<static_cast<unsigned>((width + 31) / 32), 1024, 0, st>>>(static_cast<const A*>(scratch), static_cast<int>(grid), width,
                                                                                          static_cast<A>(alpha), static_cast<T*>(ggain));
    MP_LAUNCH_CHECK();
  }
}

template <typename T>
void head_scale_accumulate_impl(const void* D, const void* gy, void* gx, len_t rows, len_t heads, len_t headdim, StreamContext ctx) {
  if (rows == 0 || heads == 0 || headdim == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t width = heads * headdim;
  cudaStream_t st = mp_stream(ctx);
  if (headdim % PN == 0 && mp_aligned16(gy) && mp_aligned16(gx))
    head_scale_accumulate_kernel<T, PN><<<grid_for(rows * (width / PN), 256), 256, 0, st>>>(static_cast<const A*>(D), static_cast<const T*>(gy),
                                                                                        static_cast<T*>(gx), rows, static_cast<int>(heads),
                                                                                        static_cast<int>(headdim));
  else
    head_scale_accumulate_kernel<T, 1><<<grid_for(rows * width, 256), 256, 0, st>>>(static_cast<const A*>(D), static_cast<const T*>(gy), static_cast<T*>(gx),
                                                                                rows, static_cast<int>(heads), static_cast<int>(headdim));
  MP_LAUNCH_CHECK();
}

template <typename T, int V>
void ce_launch(const T* logits, const int* targets, double scale, typename Acc<T>::type* loss, T* glogits, len_t m, len_t n, cudaStream_t st,
               uint32_t* status) {
  using A = typename Acc<T>::type;
  const size_t row_bytes = n * sizeof(T);
  if (status != nullptr && row_bytes <= 100 * 1024 + 4096 && row_bytes % 16 == 0 && n % V == 0 && mp_aligned16(logits) &&
      (glogits == nullptr || mp_aligned16(glogits)) && getenv("MP_CE_NO_BULK") == nullptr) {
    // (two CTAs per SM need the row below ~110 KB)
    MP_CUDA_CHECK(cudaFuncSetAttribute(cross_entropy_bulk_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    cross_entropy_bulk_kernel<T, V><<<static_cast<unsigned>(m), CE_THREADS, (row_bytes + 127) & ~size_t(127), st>>>(
        logits, targets, static_cast<A>(scale), loss, glogits, n, status);
  } else if (row_bytes <= 200 * 1024) {
    MP_CUDA_CHECK(cudaFuncSetAttribute(cross_entropy_kernel<T, V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    cross_entropy_kernel<T, V, true><<<static_cast<unsigned>(m), CE_THREADS, (row_bytes + 15) & ~size_t(15), st>>>(logits, targets, static_cast<A>(scale), loss,
                                                                                                                 glogits, n);
  } else {
    cross_entropy_kernel<T, V, false><<<static_cast<unsigned>(m), CE_THREADS, 0, st>>>(logits, targets, static_cast<A>(scale), loss, glogits, n);
  }
  MP_LAUNCH_CHECK();
}

template <typename T>
void cross_entropy_impl(const void* logits, const void* targets, double scale, void* loss, void* glogits, len_t m, len_t n, StreamContext ctx) {
  if (m == 0 || n == 0) return;
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const bool v = n % PN == 0 && mp_aligned16(logits) && (glogits == nullptr || mp_aligned16(glogits));
  MpStreamState* state = mp_state_or_null(ctx);
  uint32_t* status = state != nullptr ? state->status_dev : nullptr;   // bounded waits report here
  if (v) ce_launch<T, PN>(static_cast<const T*>(logits), static_cast<const int*>(targets), scale, static_cast<A*>(loss), static_cast<T*>(glogits), m, n, mp_stream(ctx), status);
  else ce_launch<T, 1>(static_cast<const T*>(logits), static_cast<const int*>(targets), scale, static_cast<A*>(loss), static_cast<T*>(glogits), m, n, mp_stream(ctx), status);
}

template <typename T>
void neg_exp_impl(const void* src, void* dst, len_t n, StreamContext ctx) {
  if (n == 0) return;
  neg_exp_kernel<T><<<grid_for(n, 256), 256, 0, mp_stream(ctx)>>>(static_cast<const T*>(src), static_cast<T*>(dst), n);
  MP_LAUNCH_CHECK();
}

}  // namespace

MP_STAMP3(embedding, (const void* table, const void* ids, void* out, len_t n, len_t dim, len_t vocab, StreamContext ctx),
          (table, ids, out, n, dim, vocab, ctx))
MP_STAMP3(embedding_reverse, (const void* ids, const void* gy, void* gtable, len_t n, len_t dim, len_t vocab, StreamContext ctx),
          (ids, gy, gtable, n, dim, vocab, ctx))
MP_STAMP3(causal_conv1d_silu,
          (const void* x, len_t x_pitch, const void* w, const void* bias, void* y, len_t y_pitch, len_t batch, len_t len, len_t channels,
           len_t width, StreamContext ctx),
          (x, x_pitch, w, bias, y, y_pitch, batch, len, channels, width, ctx))
MP_STAMP3(causal_conv1d_silu_reverse,
          (const void* x, len_t x_pitch, const void* w, const void* bias, const void* gy, len_t gy_pitch, void* gx, len_t gx_pitch, void* gw,
           void* gbias, len_t batch, len_t len, len_t channels, len_t width, StreamContext ctx),
          (x, x_pitch, w, bias, gy, gy_pitch, gx, gx_pitch, gw, gbias, batch, len, channels, width, ctx))
MP_STAMP3(causal_conv1d_silu_segments,
          (const void* x, len_t x_pitch, const void* w, const void* bias, void* const* ys, const len_t* y_pitches, const len_t* seg_channels,
           len_t nseg, len_t batch, len_t len, len_t width, StreamContext ctx),
          (x, x_pitch, w, bias, ys, y_pitches, seg_channels, nseg, batch, len, width, ctx))
MP_STAMP3(causal_conv1d_silu_segments_reverse,
          (const void* x, len_t x_pitch, const void* w, const void* bias, const void* const* gys, const len_t* gy_pitches,
           const len_t* seg_channels, len_t nseg, void* gx, len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t width,
           StreamContext ctx),
          (x, x_pitch, w, bias, gys, gy_pitches, seg_channels, nseg, gx, gx_pitch, gw, gbias, batch, len, width, ctx))
MP_STAMP3(causal_conv1d_silu_segments_reverse_skip,
          (const void* x, len_t x_pitch, const void* w, const void* bias, const void* const* gys, const len_t* gy_pitches,
           const len_t* seg_channels, len_t nseg, const void* const* skips, const len_t* skip_pitches, const void* const* skip_scales,
           len_t skip_group, void* gx, len_t gx_pitch, void* gw, void* gbias, len_t batch, len_t len, len_t width, StreamContext ctx),
          (x, x_pitch, w, bias, gys, gy_pitches, seg_channels, nseg, skips, skip_pitches, skip_scales, skip_group, gx, gx_pitch, gw, gbias, batch,
           len, width, ctx))
MP_STAMP3(softplus_bias, (const void* raw, len_t raw_pitch, const void* bias, void* out, len_t rows, len_t heads, StreamContext ctx),
          (raw, raw_pitch, bias, out, rows, heads, ctx))
MP_STAMP3(softplus_bias_reverse,
          (const void* raw, len_t raw_pitch, const void* bias, const void* gdt, void* graw, len_t graw_pitch, void* gbias, len_t rows,
           len_t heads, StreamContext ctx),
          (raw, raw_pitch, bias, gdt, graw, graw_pitch, gbias, rows, heads, ctx))
MP_STAMP3(ssd_gate,
          (const void* y, const void* x, const void* D, const void* z, len_t z_pitch, void* u, len_t rows, len_t heads, len_t headdim,
           StreamContext ctx),
          (y, x, D, z, z_pitch, u, rows, heads, headdim, ctx))
MP_STAMP3(ssd_gate_reverse,
          (const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gu, void* gy, void* gz, len_t gz_pitch,
           void* gD, len_t rows, len_t heads, len_t headdim, StreamContext ctx),
          (y, x, D, z, z_pitch, gu, gy, gz, gz_pitch, gD, rows, heads, headdim, ctx))
MP_STAMP3(ssd_gate_rmsnorm,
          (const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gain, double eps, void* out, void* rstd,
           len_t rows, len_t heads, len_t headdim, StreamContext ctx),
          (y, x, D, z, z_pitch, gain, eps, out, rstd, rows, heads, headdim, ctx))
MP_STAMP3(ssd_gate_rmsnorm_reverse,
          (const void* y, const void* x, const void* D, const void* z, len_t z_pitch, const void* gain, const void* rstd, const void* gout,
           void* gy, void* gz, len_t gz_pitch, void* gD, void* ggain, double alpha, void* scratch, len_t rows, len_t heads, len_t headdim,
           StreamContext ctx),
          (y, x, D, z, z_pitch, gain, rstd, gout, gy, gz, gz_pitch, gD, ggain, alpha, scratch, rows, heads, headdim, ctx))
extern "C" len_t mpSsdGateRmsnormReverseScratchBytes(len_t rows, len_t heads, len_t headdim, StreamContext ctx) {
  return static_cast<len_t>(gate_rmsnorm_grid(rows, mp_sm_count(ctx))) * heads * headdim * sizeof(double);
}
MP_STAMP3(head_scale_accumulate, (const void* D, const void* gy, void* gx, len_t rows, len_t heads, len_t headdim, StreamContext ctx),
          (D, gy, gx, rows, heads, headdim, ctx))
MP_STAMP3(cross_entropy,
          (const void* logits, const void* targets, double scale, void* loss, void* glogits, len_t m, len_t n, StreamContext ctx),
          (logits, targets, scale, loss, glogits, m, n, ctx))
MP_STAMP3(neg_exp, (const void* src, void* dst, len_t n, StreamContext ctx), (src, dst, n, ctx))

extern "C" void launch_convert_r16_r32(const void* src, void* dst, double beta, len_t n, StreamContext ctx) {
  if (n == 0) return;
  cudaStream_t st = mp_stream(ctx);
  if (n % 8 == 0 && mp_aligned16(src) && (reinterpret_cast<uintptr_t>(dst) & 31u) == 0)
    convert_r16_r32_kernel<8><<<grid_for(n / 8, 512), 512, 0, st>>>(static_cast<const __half*>(src), static_cast<float*>(dst), static_cast<float>(beta), n);
  else
    convert_r16_r32_kernel<1><<<grid_for(n, 512), 512, 0, st>>>(static_cast<const __half*>(src), static_cast<float*>(dst), static_cast<float>(beta), n);
  MP_LAUNCH_CHECK();
}

extern "C" void launch_convert_r32_r16(const void* src, void* dst, len_t n, StreamContext ctx) {
  if (n == 0) return;
  cudaStream_t st = mp_stream(ctx);
  if (n % 8 == 0 && mp_aligned16(dst) && (reinterpret_cast<uintptr_t>(src) & 31u) == 0)
    convert_r32_r16_kernel<8><<<grid_for(n / 8, 512), 512, 0, st>>>(static_cast<const float*>(src), static_cast<__half*>(dst), n);
  else
    convert_r32_r16_kernel<1><<<grid_for(n, 512), 512, 0, st>>>(static_cast<const float*>(src), static_cast<__half*>(dst), n);
  MP_LAUNCH_CHECK();
}

// ---- mixed-precision optimizer step of the language-model composition ---------------------------------------
// tick: 16 bytes of device memory, zero-filled once by the caller: {1/(1-b1^t), 1/(1-b2^t), t, non-finite flag}.
// launch_adam_tick advances t and refreshes the two corrections; it runs on the stream like any launcher (one
// thread), so a step that is replayed from a captured graph still sees its own step number.
extern "C" void launch_adam_tick(void* tick, double beta1, double beta2, StreamContext ctx) {
  adam_tick_kernel<<<1, 1, 0, mp_stream(ctx)>>>(static_cast<AdamTick*>(tick), static_cast<float>(beta1), static_cast<float>(beta2));
  MP_LAUNCH_CHECK();
}

// One pass over a flat parameter bucket: g = (g32 + g16) * grad_scale (g16 may be NULL), Adam update of the r32 master
// weights and moments with the corrections in `tick`, and the refreshed r16 working copy w16 = round(w32).  Elements
// whose gradient is not finite are left unchanged and the flag in `tick` is set (a static loss scale can overflow).
extern "C" void launch_adam_mixed_r32(void* w32, void* w16, const void* g32, const void* g16, void* m, void* v, double lr, double beta1,
                                      double beta2, double eps, double grad_scale, void* tick, len_t n, StreamContext ctx) {
  if (n == 0) return;
  cudaStream_t st = mp_stream(ctx);
  const bool vec = n % 8 == 0 && mp_aligned16(w16) && (g16 == nullptr || mp_aligned16(g16)) &&
                   ((reinterpret_cast<uintptr_t>(w32) | reinterpret_cast<uintptr_t>(g32) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 31u) == 0;
  if (vec)
    adam_mixed_kernel<8><<<grid_for(n / 8, 512), 512, 0, st>>>(static_cast<float*>(w32), static_cast<__half*>(w16), static_cast<const float*>(g32),
                                                             static_cast<const __half*>(g16), static_cast<float*>(m), static_cast<float*>(v),
                                                             static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
                                                             static_cast<float>(eps), static_cast<float>(grad_scale), static_cast<AdamTick*>(tick), n);
  else
    adam_mixed_kernel<1><<<grid_for(n, 512), 512, 0, st>>>(static_cast<float*>(w32), static_cast<__half*>(w16), static_cast<const float*>(g32),
                                                         static_cast<const __half*>(g16), static_cast<float*>(m), static_cast<float*>(v),
                                                         static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
                                                         static_cast<float>(eps), static_cast<float>(grad_scale), static_cast<AdamTick*>(tick), n);
  MP_LAUNCH_CHECK();
}
