// Sequential-recurrence SSD scan for every storage type and shape (the tensor-core path of ssd.cu covers r16
// with d_state 128, headdim 64 / 128 and chunked sequence lengths; everything else lands here).  One CTA walks
// one (batch, head) sequence in time order with the N x P state distributed over its 256 threads, exactly the
// definition
//     S_t = exp(dt_t A_h) S_{t-1} + dt_t B_t x_t^T,      y_t = C_t^T S_t,      S_{-1} = 0
// and, for the reverse, the adjoint recurrence run backwards in time
//     lam_t = C_t gy_t^T + exp(dt_{t+1} A_h) lam_{t+1}
//     gC_t += S_t gy_t        gx_t = dt_t lam_t^T B_t        gB_t += dt_t lam_t x_t
//     gdt_t = <lam_t, B_t x_t^T> + A_h a_t <lam_t, S_{t-1}>        gA_h += dt_t a_t <lam_t, S_{t-1}>     (a_t = exp(dt_t A_h))
// The reverse keeps a state checkpoint every GEN_QS steps and recomputes the states of one block of GEN_QS steps
// at a time into scratch.  Arithmetic in the accumulator type (r32 for r16 / r32 storage, r64 for r64); dt, A,
// gdt, gA are accumulator-typed for r32 / r64 storage and r32 for r16.  This is a correctness path, not a fast
// one: latency-bound, one SM per sequence.
#include "mp_common.cuh"

namespace {

constexpr int GEN_THREADS = 256;
constexpr int GEN_QS = 64;      // checkpoint distance of the reverse
constexpr int GEN_EN = 64;      // state elements per thread (upper bound)

struct GenDims { int B, L, H, P, N, G; int PP, NG, EN; };

// threads: p = tid % PP (headdim index, idle when p >= P), ng = tid / PP; the thread owns state rows n = ng + k NG
__host__ __device__ inline bool gen_plan(GenDims& d) {
  int pp = 1;
  while (pp < d.P) pp <<= 1;
  if (pp > GEN_THREADS) return false;
  d.PP = pp; d.NG = GEN_THREADS / pp; d.EN = (d.N + d.NG - 1) / d.NG;
  return d.EN <= GEN_EN;
}

template <typename A>
__device__ __forceinline__ A gen_block_sum(A v, A* red) {   // red: GEN_THREADS / 32 + 1 values
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    A s = A(0);
    for (int w = 0; w < GEN_THREADS / 32; ++w) s += red[w];
    red[GEN_THREADS / 32] = s;
  }
  __syncthreads();
  const A r = red[GEN_THREADS / 32];
  __syncthreads();
  return r;
}

template <typename A> __device__ __forceinline__ A gen_exp(A v);
template <> __device__ __forceinline__ float gen_exp<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ double gen_exp<double>(double v) { return exp(v); }

// Shared-memory layout: sB[N] sC[N] sx[P] sg[P] sN1[N] sN2[N] red[NG * PP] small[16]
template <typename T, typename A, bool REVERSE>
__global__ void __launch_bounds__(GEN_THREADS) ssd_generic_kernel(const T* __restrict__ x, const A* __restrict__ dt,
                                                                  const A* __restrict__ Ah, const T* __restrict__ Bm,
                                                                  const T* __restrict__ Cm, T* __restrict__ y,
                                                                  const T* __restrict__ gy, T* __restrict__ gx,
                                                                  A* __restrict__ gdt, A* __restrict__ gA, A* __restrict__ gB,
                                                                  A* __restrict__ gC, A* __restrict__ ckpt, A* __restrict__ cs,
                                                                  GenDims d) {
  extern __shared__ __align__(16) unsigned char gen_smem[];
  A* sB = reinterpret_cast<A*>(gen_smem);
  A* sC = sB + d.N;
  A* sx = sC + d.N;
  A* sg = sx + d.P;
  A* sN1 = sg + d.P;
  A* sN2 = sN1 + d.N;
  A* red = sN2 + d.N;
  A* small = red + d.NG * d.PP;
  const int tid = threadIdx.x;
  const int p = tid % d.PP, ng = tid / d.PP;
  const bool live_p = p < d.P;
  const int b = blockIdx.x / d.H, h = blockIdx.x % d.H, grp = h / (d.H / d.G);
  const A a_h = Ah[h];
  const size_t np = static_cast<size_t>(d.N) * d.P;
  const int nck = (d.L + GEN_QS - 1) / GEN_QS;
  A* my_ckpt = REVERSE ? ckpt + static_cast<size_t>(blockIdx.x) * nck * np : nullptr;
  A* my_cs = REVERSE ? cs + static_cast<size_t>(blockIdx.x) * GEN_QS * np : nullptr;
  A S[GEN_EN];
#pragma unroll
  for (int k = 0; k < GEN_EN; ++k) S[k] = A(0);

  auto load_step = [&](int t, bool with_gy) {
    const size_t rowBC = (static_cast<size_t>(b) * d.L + t) * d.G + grp;
    const size_t rowX = (static_cast<size_t>(b) * d.L + t) * d.H + h;
    for (int i = tid; i < d.N; i += GEN_THREADS) { sB[i] = mp_up(Bm[rowBC * d.N + i]); sC[i] = mp_up(Cm[rowBC * d.N + i]); }
    for (int i = tid; i < d.P; i += GEN_THREADS) {
      sx[i] = mp_up(x[rowX * d.P + i]);
      if (with_gy) sg[i] = mp_up(gy[rowX * d.P + i]);
    }
  };

  // ---- forward sweep: y (forward launch) or state checkpoints (reverse launch) -------------------------------
  for (int t = 0; t < d.L; ++t) {
    __syncthreads();
    load_step(t, false);
    if (REVERSE && t % GEN_QS == 0) {
#pragma unroll
      for (int k = 0; k < GEN_EN; ++k) {
        const int n = ng + k * d.NG;
        if (k < d.EN && n < d.N && live_p) my_ckpt[(static_cast<size_t>(t / GEN_QS) * d.N + n) * d.P + p] = S[k];
      }
    }
    const A dtv = dt[(static_cast<size_t>(b) * d.L + t) * d.H + h];
    const A a = gen_exp<A>(dtv * a_h);
    __syncthreads();
    A acc = A(0);
#pragma unroll
    for (int k = 0; k < GEN_EN; ++k) {
      const int n = ng + k * d.NG;
      if (k < d.EN && n < d.N && live_p) {
        S[k] = a * S[k] + dtv * sB[n] * sx[p];
        acc += sC[n] * S[k];
      }
    }
    if (!REVERSE) {
      red[ng * d.PP + p] = acc;
      __syncthreads();
      if (tid < d.P) {
        A s = A(0);
        for (int q = 0; q < d.NG; ++q) s += red[q * d.PP + tid];
        y[((static_cast<size_t>(b) * d.L + t) * d.H + h) * d.P + tid] = mp_down<T>(s);
      }
    }
  }
  if constexpr (REVERSE) {

  // ---- reverse sweep --------------------------------------------------------------------------------------------
  A lam[GEN_EN];
#pragma unroll
  for (int k = 0; k < GEN_EN; ++k) lam[k] = A(0);
  A a_next = A(0);
  A ga_acc = A(0);   // thread 0 only
  for (int c = nck - 1; c >= 0; --c) {
    const int t0 = c * GEN_QS, t1 = min(d.L, t0 + GEN_QS);
    // states of the block, recomputed from its checkpoint
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GEN_EN; ++k) {
      const int n = ng + k * d.NG;
      S[k] = (k < d.EN && n < d.N && live_p) ? my_ckpt[(static_cast<size_t>(c) * d.N + n) * d.P + p] : A(0);
    }
    for (int t = t0; t < t1; ++t) {
      __syncthreads();
      load_step(t, false);
      const A dtv = dt[(static_cast<size_t>(b) * d.L + t) * d.H + h];
      const A a = gen_exp<A>(dtv * a_h);
      __syncthreads();
#pragma unroll
      for (int k = 0; k < GEN_EN; ++k) {
        const int n = ng + k * d.NG;
        if (k < d.EN && n < d.N && live_p) {
          S[k] = a * S[k] + dtv * sB[n] * sx[p];
          my_cs[(static_cast<size_t>(t - t0) * d.N + n) * d.P + p] = S[k];
        }
      }
    }
    // adjoint recurrence, newest step first (each thread re-reads only what it wrote itself)
    for (int t = t1 - 1; t >= t0; --t) {
      __syncthreads();
      load_step(t, true);
      for (int i = tid; i < d.N; i += GEN_THREADS) { sN1[i] = A(0); sN2[i] = A(0); }
      const A dtv = dt[(static_cast<size_t>(b) * d.L + t) * d.H + h];
      const A a = gen_exp<A>(dtv * a_h);
      __syncthreads();
      A gx_part = A(0), s2 = A(0);
#pragma unroll
      for (int k = 0; k < GEN_EN; ++k) {
        if (k < d.EN) {   // uniform over the CTA (the shuffles below need whole warps)
          const int n = ng + k * d.NG;
          const bool live = n < d.N && live_p;
          A vC = A(0), vB = A(0);
          if (live) {
            const A ht = my_cs[(static_cast<size_t>(t - t0) * d.N + n) * d.P + p];
            const A hp = t > t0 ? my_cs[(static_cast<size_t>(t - t0 - 1) * d.N + n) * d.P + p]
                                : my_ckpt[(static_cast<size_t>(c) * d.N + n) * d.P + p];
            lam[k] = sC[n] * sg[p] + a_next * lam[k];
            vC = ht * sg[p];
            vB = lam[k] * sx[p];
            gx_part += lam[k] * sB[n];
            s2 += lam[k] * hp;
          }
          // sum over the headdim index: the PP threads of one ng are contiguous
          const int width = d.PP < 32 ? d.PP : 32;
          for (int o = width >> 1; o > 0; o >>= 1) {
            vC += __shfl_xor_sync(0xffffffffu, vC, o);
            vB += __shfl_xor_sync(0xffffffffu, vB, o);
          }
          if (n < d.N && (p % width) == 0) { atomicAdd(sN1 + n, vC); atomicAdd(sN2 + n, vB); }
        }
      }
      red[ng * d.PP + p] = gx_part;
      __syncthreads();
      A s1 = A(0);
      if (tid < d.P) {
        A s = A(0);
        for (int q = 0; q < d.NG; ++q) s += red[q * d.PP + tid];
        gx[((static_cast<size_t>(b) * d.L + t) * d.H + h) * d.P + tid] = mp_down<T>(dtv * s);
        s1 = s * sx[tid];
      }
      const size_t rowBC = (static_cast<size_t>(b) * d.L + t) * d.G + grp;
      for (int i = tid; i < d.N; i += GEN_THREADS) {   // summed over the heads of the group (outputs were zeroed)
        atomicAdd(gC + rowBC * d.N + i, sN1[i]);
        atomicAdd(gB + rowBC * d.N + i, dtv * sN2[i]);
      }
      s1 = gen_block_sum<A>(s1, small);
      s2 = gen_block_sum<A>(s2, small);
      if (tid == 0) {
        gdt[(static_cast<size_t>(b) * d.L + t) * d.H + h] = s1 + a_h * a * s2;
        ga_acc += dtv * a * s2;
      }
      a_next = a;
    }
  }
  if (tid == 0) atomicAdd(gA + h, ga_acc);
  }   // REVERSE
}

template <typename A>
__global__ void gen_round_kernel(const A* __restrict__ src, void* __restrict__ dst, size_t n, int to_half) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  if (to_half) static_cast<__half*>(dst)[i] = __float2half_rn(static_cast<float>(src[i]));
}

size_t gen_smem_bytes(const GenDims& d, size_t acc) { return (4 * static_cast<size_t>(d.N) + 2 * d.P + static_cast<size_t>(d.NG) * d.PP + 16) * acc; }

}  // namespace

// Scratch of the generic path for storage type `dtype_key` (0 = r16, 1 = r32, 2 = r64): reverse only
// (state checkpoints, one block of recomputed states per sequence and, for r16, accumulator-typed gB / gC).
extern "C" len_t mpSsdScanGenericScratchBytes(uint32_t dtype_key, len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate,
                                              len_t ngroups, uint32_t reverse) {
  if (!reverse) return 256;
  const size_t acc = dtype_key == 2 ? 8 : 4;
  const size_t np = static_cast<size_t>(dstate) * headdim;
  const size_t nck = (seqlen + GEN_QS - 1) / GEN_QS;
  size_t bytes = static_cast<size_t>(batch) * heads * (nck + GEN_QS) * np * acc;
  if (dtype_key == 0) bytes += 2 * static_cast<size_t>(batch) * seqlen * ngroups * dstate * acc;
  return static_cast<len_t>(bytes + 1024);
}

template <typename T, typename A>
static void ssd_generic_forward(const void* x, const void* dt, const void* Av, const void* Bm, const void* Cm, void* y, len_t batch,
                                len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  GenDims d{static_cast<int>(batch), static_cast<int>(seqlen), static_cast<int>(heads), static_cast<int>(headdim),
            static_cast<int>(dstate), static_cast<int>(ngroups), 0, 0, 0};
  if (ngroups == 0 || heads % ngroups != 0) MP_FATAL("ssd_scan: heads %d not divisible by groups %d", d.H, d.G);
  if (!gen_plan(d)) MP_FATAL("ssd_scan: headdim %d x d_state %d is beyond the generic path (headdim <= 256, d_state * headdim <= 16384)", d.P, d.N);
  const size_t smem = gen_smem_bytes(d, sizeof(A));
  ssd_generic_kernel<T, A, false><<<d.B * d.H, GEN_THREADS, smem, mp_stream(ctx)>>>(
      static_cast<const T*>(x), static_cast<const A*>(dt), static_cast<const A*>(Av), static_cast<const T*>(Bm), static_cast<const T*>(Cm),
      static_cast<T*>(y), nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, d);
  MP_LAUNCH_CHECK();
}

template <typename T, typename A>
static void ssd_generic_reverse(const void* x, const void* dt, const void* Av, const void* Bm, const void* Cm, const void* gy, void* gx,
                                void* gdt, void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads,
                                len_t headdim, len_t dstate, len_t ngroups, StreamContext ctx) {
  if (batch == 0 || seqlen == 0 || heads == 0) return;
  GenDims d{static_cast<int>(batch), static_cast<int>(seqlen), static_cast<int>(heads), static_cast<int>(headdim),
            static_cast<int>(dstate), static_cast<int>(ngroups), 0, 0, 0};
  if (ngroups == 0 || heads % ngroups != 0) MP_FATAL("ssd_scan_reverse: heads %d not divisible by groups %d", d.H, d.G);
  if (!gen_plan(d)) MP_FATAL("ssd_scan_reverse: headdim %d x d_state %d is beyond the generic path", d.P, d.N);
  if (scratch == nullptr) MP_FATAL("ssd_scan_reverse: scratch must not be NULL (mpSsdScanGenericScratchBytes)");
  cudaStream_t st = mp_stream(ctx);
  const size_t np = static_cast<size_t>(d.N) * d.P;
  const size_t nck = (d.L + GEN_QS - 1) / GEN_QS;
  A* ckpt = static_cast<A*>(scratch);
  A* cs = ckpt + static_cast<size_t>(d.B) * d.H * nck * np;
  const size_t bc = static_cast<size_t>(d.B) * d.L * d.G * d.N;
  A* gB_acc = static_cast<A*>(gB);
  A* gC_acc = static_cast<A*>(gC);
  constexpr bool narrow = std::is_same<T, __half>::value;   // r16: group gradients accumulate in r32 scratch, rounded at the end
  if (narrow) { gB_acc = cs + static_cast<size_t>(d.B) * d.H * GEN_QS * np; gC_acc = gB_acc + bc; }
  MP_CUDA_CHECK(cudaMemsetAsync(gB_acc, 0, bc * sizeof(A), st));
  MP_CUDA_CHECK(cudaMemsetAsync(gC_acc, 0, bc * sizeof(A), st));
  MP_CUDA_CHECK(cudaMemsetAsync(gA, 0, static_cast<size_t>(d.H) * sizeof(A), st));
  const size_t smem = gen_smem_bytes(d, sizeof(A));
  ssd_generic_kernel<T, A, true><<<d.B * d.H, GEN_THREADS, smem, st>>>(
      static_cast<const T*>(x), static_cast<const A*>(dt), static_cast<const A*>(Av), static_cast<const T*>(Bm), static_cast<const T*>(Cm),
      nullptr, static_cast<const T*>(gy), static_cast<T*>(gx), static_cast<A*>(gdt), static_cast<A*>(gA), gB_acc, gC_acc, ckpt, cs, d);
  MP_LAUNCH_CHECK();
  if (narrow) {
    gen_round_kernel<A><<<static_cast<unsigned>((bc + 255) / 256), 256, 0, st>>>(gB_acc, gB, bc, 1);
    gen_round_kernel<A><<<static_cast<unsigned>((bc + 255) / 256), 256, 0, st>>>(gC_acc, gC, bc, 1);
    MP_LAUNCH_CHECK();
  }
}

// Entry points used by ssd.cu (r16 shapes outside the tensor-core path) and the r32 / r64 launchers.
void mp_ssd_generic_forward_r16(const void* x, const void* dt, const void* A, const void* B, const void* C, void* y, len_t batch, len_t seqlen,
                                len_t heads, len_t headdim, len_t dstate, len_t ngroups, StreamContext ctx) {
  ssd_generic_forward<__half, float>(x, dt, A, B, C, y, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
}
void mp_ssd_generic_reverse_r16(const void* x, const void* dt, const void* A, const void* B, const void* C, const void* gy, void* gx, void* gdt,
                                void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen, len_t heads, len_t headdim,
                                len_t dstate, len_t ngroups, StreamContext ctx) {
  ssd_generic_reverse<__half, float>(x, dt, A, B, C, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
}

extern "C" void launch_ssd_scan_r32(const void* x, const void* dt, const void* A, const void* B, const void* C, void* y, void* scratch,
                                    len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk,
                                    StreamContext ctx) {
  (void)scratch; (void)chunk;
  ssd_generic_forward<float, float>(x, dt, A, B, C, y, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
}
extern "C" void launch_ssd_scan_r64(const void* x, const void* dt, const void* A, const void* B, const void* C, void* y, void* scratch,
                                    len_t batch, len_t seqlen, len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk,
                                    StreamContext ctx) {
  (void)scratch; (void)chunk;
  ssd_generic_forward<double, double>(x, dt, A, B, C, y, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
}
extern "C" void launch_ssd_scan_reverse_r32(const void* x, const void* dt, const void* A, const void* B, const void* C, const void* gy,
                                            void* gx, void* gdt, void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen,
                                            len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx) {
  (void)chunk;
  ssd_generic_reverse<float, float>(x, dt, A, B, C, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
}
extern "C" void launch_ssd_scan_reverse_r64(const void* x, const void* dt, const void* A, const void* B, const void* C, const void* gy,
                                            void* gx, void* gdt, void* gA, void* gB, void* gC, void* scratch, len_t batch, len_t seqlen,
                                            len_t heads, len_t headdim, len_t dstate, len_t ngroups, len_t chunk, StreamContext ctx) {
  (void)chunk;
  ssd_generic_reverse<double, double>(x, dt, A, B, C, gy, gx, gdt, gA, gB, gC, scratch, batch, seqlen, heads, headdim, dstate, ngroups, ctx);
}
