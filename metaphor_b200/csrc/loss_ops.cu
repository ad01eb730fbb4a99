// Rank-1 losses and the momentum optimizer step.  The reference calls kernels of these names from
// src/loss/loss.zig:58-136 (`kernel_mse_loss_i_i`, `kernel_bce_loss_i_i`) and src/optm/optimizer.zig:263-273
// (`kernel_momentum`) but has no implementation of any of them; the argument order below is the one of those
// call sites (values, gradient out, target, scratch, reduced loss, n) resp. (w, g, momentum, rate, alpha, clip, n).
//
//   mse : loss = mean_i (x_i - t_i)^2                              grad_i = 2 (x_i - t_i) / n
//   bce : x holds probabilities p_i (the host applies the sigmoid in place first, loss.zig:117-119)
//         loss = -mean_i [t_i log p_i + (1 - t_i) log(1 - p_i)]      grad_i = (p_i - t_i) / n   (w.r.t. the logits)
//   momentum : m = alpha m + clip(g, lo, hi);  w -= rate m
//
// Loss reduction: one partial per CTA of 4096 elements into `scratch` (n / 4096 + 2 accumulator-typed slots, the
// reference's sizing), folded in a fixed order by a second one-CTA launch into `redux` (accumulator type, may be
// NULL when only the gradient is wanted; `grad` may be NULL when only the loss is wanted).
#include "mp_common.cuh"

namespace {

constexpr int LOSS_THREADS = 256;
constexpr int LOSS_PER_CTA = 4096;

template <typename T, bool BCE>
__global__ void __launch_bounds__(LOSS_THREADS) loss_partial_kernel(const T* __restrict__ x, T* __restrict__ grad,
                                                                    const T* __restrict__ trg,
                                                                    typename Acc<T>::type* __restrict__ scratch, size_t n) {
  using A = typename Acc<T>::type;
  __shared__ A red[LOSS_THREADS / 32];
  const A inv_n = A(1) / static_cast<A>(n);
  A acc = A(0);
  const size_t base = static_cast<size_t>(blockIdx.x) * LOSS_PER_CTA;
  for (int k = threadIdx.x; k < LOSS_PER_CTA; k += LOSS_THREADS) {
    const size_t i = base + k;
    if (i < n) {
      const A v = mp_up(x[i]), t = mp_up(trg[i]);
      A g;
      if (BCE) {
        const A tiny = A(1e-12);
        const A p = v < tiny ? tiny : (v > A(1) - tiny ? A(1) - tiny : v);
        acc -= t * log(p) + (A(1) - t) * log(A(1) - p);
        g = (v - t) * inv_n;
      } else {
        const A d = v - t;
        acc += d * d;
        g = A(2) * d * inv_n;
      }
      if (grad != nullptr) grad[i] = mp_down<T>(g);
    }
  }
  acc = warp_reduce<SumOp>(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    A s = A(0);
    for (int w = 0; w < LOSS_THREADS / 32; ++w) s += red[w];
    scratch[blockIdx.x] = s;
  }
}

template <typename A>
__global__ void __launch_bounds__(LOSS_THREADS) loss_fold_kernel(const A* __restrict__ scratch, A* __restrict__ redux, size_t parts,
                                                                 A inv_n) {
  __shared__ A red[LOSS_THREADS];
  A s = A(0);
  for (size_t i = threadIdx.x; i < parts; i += LOSS_THREADS) s += scratch[i];   // fixed order per thread
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = LOSS_THREADS / 2; o > 0; o >>= 1) {
    if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) redux[0] = red[0] * inv_n;
}

template <typename T, bool BCE>
void loss_launch(const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (n == 0) return;
  if (scratch == nullptr) MP_FATAL("loss: scratch must not be NULL (n / 4096 + 2 accumulator-typed slots)");
  const size_t parts = (n + LOSS_PER_CTA - 1) / LOSS_PER_CTA;
  cudaStream_t st = mp_stream(ctx);
  loss_partial_kernel<T, BCE><<<static_cast<unsigned>(parts), LOSS_THREADS, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(grad),
                                                                                    static_cast<const T*>(trg), static_cast<A*>(scratch), n);
  MP_LAUNCH_CHECK();
  if (redux != nullptr) {
    loss_fold_kernel<A><<<1, LOSS_THREADS, 0, st>>>(static_cast<const A*>(scratch), static_cast<A*>(redux), parts, A(1) / static_cast<A>(n));
    MP_LAUNCH_CHECK();
  }
}

template <typename T>
void mse_loss_i_i_impl(const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext ctx) {
  loss_launch<T, false>(x, grad, trg, scratch, redux, n, ctx);
}
template <typename T>
void bce_loss_i_i_impl(const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext ctx) {
  loss_launch<T, true>(x, grad, trg, scratch, redux, n, ctx);
}

template <typename T>
__global__ void __launch_bounds__(256) momentum_kernel(T* __restrict__ w, const T* __restrict__ g, T* __restrict__ m,
                                                       typename Acc<T>::type rate, typename Acc<T>::type alpha,
                                                       typename Acc<T>::type lo, typename Acc<T>::type hi, size_t n) {
  using A = typename Acc<T>::type;
  constexpr int PN = Pack<T>::N;
  const size_t nvec = n / PN;
  const bool vec = mp_aligned16(w) && mp_aligned16(g) && mp_aligned16(m);
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  auto one = [&](A wv, A gv, A& mv) {
    const A c = gv < lo ? lo : (gv > hi ? hi : gv);
    mv = alpha * mv + c;
    return wv - rate * mv;
  };
  if (vec) {
    for (size_t i = tid; i < nvec; i += stride) {
      A wf[PN], gf[PN], mf[PN];
      unpack<T>(ld_pack_stream(w, i), wf);
      unpack<T>(ld_pack_stream(g, i), gf);
      unpack<T>(ld_pack_stream(m, i), mf);
#pragma unroll
      for (int e = 0; e < PN; ++e) wf[e] = one(wf[e], gf[e], mf[e]);
      st_pack_stream(w, i, pack<T>(wf));
      st_pack_stream(m, i, pack<T>(mf));
    }
    for (size_t i = nvec * PN + tid; i < n; i += stride) {
      A mv = mp_up(m[i]);
      w[i] = mp_down<T>(one(mp_up(w[i]), mp_up(g[i]), mv));
      m[i] = mp_down<T>(mv);
    }
  } else {
    for (size_t i = tid; i < n; i += stride) {
      A mv = mp_up(m[i]);
      w[i] = mp_down<T>(one(mp_up(w[i]), mp_up(g[i]), mv));
      m[i] = mp_down<T>(mv);
    }
  }
}

template <typename T>
void momentum_impl(void* w, const void* g, void* m, double rate, double alpha, double lo, double hi, len_t n, StreamContext ctx) {
  using A = typename Acc<T>::type;
  if (n == 0) return;
  const size_t work = (n + Pack<T>::N - 1) / Pack<T>::N;
  size_t grid = (work + 255) / 256;
  if (grid > (1u << 30)) grid = 1u << 30;
  momentum_kernel<T><<<static_cast<unsigned>(grid), 256, 0, mp_stream(ctx)>>>(static_cast<T*>(w), static_cast<const T*>(g), static_cast<T*>(m),
                                                                          static_cast<A>(rate), static_cast<A>(alpha), static_cast<A>(lo),
                                                                          static_cast<A>(hi), n);
  MP_LAUNCH_CHECK();
}

}  // namespace

MP_STAMP3(mse_loss_i_i, (const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext ctx),
          (x, grad, trg, scratch, redux, n, ctx))
MP_STAMP3(bce_loss_i_i, (const void* x, void* grad, const void* trg, void* scratch, void* redux, len_t n, StreamContext ctx),
          (x, grad, trg, scratch, redux, n, ctx))
MP_STAMP3(momentum, (void* w, const void* g, void* m, double rate, double alpha, double clip_lo, double clip_hi, len_t n, StreamContext ctx),
          (w, g, m, rate, alpha, clip_lo, clip_hi, n, ctx))
