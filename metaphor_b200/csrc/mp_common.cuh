// Shared definitions of the sm_100a device layer: per-stream state, error
// macros, 128-bit packs, streaming loads/stores, warp/CTA reductions.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <type_traits>

#include "../../include/mp_types.h"
#include "../../include/mp_kernels.h"
#include "../../include/mp_device_utils.h"

// ---------------------------------------------------------------------------
// Error convention of the reference (kernel_header.h:64-98): print and exit.
// ---------------------------------------------------------------------------
#define MP_CUDA_CHECK(expr)                                                     \
  do {                                                                          \
    cudaError_t mp_err__ = (expr);                                              \
    if (mp_err__ != cudaSuccess) {                                              \
      printf("%s in %s at line %d\n", cudaGetErrorString(mp_err__), __FILE__,   \
             __LINE__);                                                         \
      fflush(stdout);                                                           \
      exit(EXIT_FAILURE);                                                       \
    }                                                                           \
  } while (0)

// Driver-API results (entry points are fetched through the runtime, the
// library does not link libcuda).
#define MP_CU_CHECK(expr)                                                       \
  do {                                                                          \
    CUresult mp_res__ = (expr);                                                 \
    if (mp_res__ != CUDA_SUCCESS) {                                             \
      printf("CUDA driver error %d in %s at line %d\n",                         \
             static_cast<int>(mp_res__), __FILE__, __LINE__);                   \
      fflush(stdout);                                                           \
      exit(EXIT_FAILURE);                                                       \
    }                                                                           \
  } while (0)

// Launch errors (bad configuration, missing image) surface here without a sync.
#define MP_LAUNCH_CHECK() MP_CUDA_CHECK(cudaPeekAtLastError())

#define MP_FATAL(...)                                                           \
  do {                                                                          \
    printf(__VA_ARGS__);                                                        \
    printf(" (%s:%d)\n", __FILE__, __LINE__);                                   \
    fflush(stdout);                                                             \
    exit(EXIT_FAILURE);                                                         \
  } while (0)

// ---------------------------------------------------------------------------
// Per-stream state stored in StreamContext.blas_handle.
// ---------------------------------------------------------------------------
static constexpr uint64_t MP_STATE_MAGIC = 0x4d50423230305354ull;  // "MPB200ST"

struct MpStreamState {
  uint64_t magic;
  cudaStream_t stream;
  int device;
  int sm_count;
  bool owns_stream;
  void* workspace;          // device, workspace_bytes long, 256-byte aligned
  size_t workspace_bytes;
  uint32_t* status_dev;     // one device word, zero when healthy
  uint32_t* status_host;    // pinned host landing slot for mpGetStatus
  // Helper streams and events for launchers that run independent kernel chains side by side (forked from and
  // joined back into `stream`, also under stream capture); created on first use, destroyed with the state.
  cudaStream_t aux_stream[7];          // 0-2: side lanes, 3-6: one sub-lane per lane
  cudaEvent_t aux_fork, aux_join[7], aux_sub_fork[4];
  bool aux_ready;
};

// Creates the helper streams / events of a state on first use.
static inline void mp_aux_init(MpStreamState* st) {
  if (st->aux_ready) return;
  for (int i = 0; i < 7; ++i) {
    MP_CUDA_CHECK(cudaStreamCreateWithFlags(&st->aux_stream[i], cudaStreamNonBlocking));
    MP_CUDA_CHECK(cudaEventCreateWithFlags(&st->aux_join[i], cudaEventDisableTiming));
  }
  for (int i = 0; i < 4; ++i) MP_CUDA_CHECK(cudaEventCreateWithFlags(&st->aux_sub_fork[i], cudaEventDisableTiming));
  MP_CUDA_CHECK(cudaEventCreateWithFlags(&st->aux_fork, cudaEventDisableTiming));
  st->aux_ready = true;
}

static inline cudaStream_t mp_stream(StreamContext ctx) {
  return static_cast<cudaStream_t>(ctx.cuda_stream.ptr);
}

// The state object, or nullptr when the caller passed a bare stream.
static inline MpStreamState* mp_state_or_null(StreamContext ctx) {
  MpStreamState* s = static_cast<MpStreamState*>(ctx.blas_handle.ptr);
  if (s != nullptr && s->magic != MP_STATE_MAGIC) {
    MP_FATAL("StreamContext.blas_handle does not come from mpInitStream/mpWrapStream");
  }
  return s;
}

// For launchers that need workspace / status: a state object is mandatory,
// like the cuBLAS handle the reference dereferences in the same slot.
static inline MpStreamState* mp_state(StreamContext ctx) {
  MpStreamState* s = mp_state_or_null(ctx);
  if (s == nullptr) MP_FATAL("this launcher needs a StreamContext from mpInitStream/mpWrapStream");
  return s;
}

int mp_sm_count_current_device();  // device_utils.cu, cached per device

static inline int mp_sm_count(StreamContext ctx) {
  MpStreamState* s = mp_state_or_null(ctx);
  return s ? s->sm_count : mp_sm_count_current_device();
}

// ---------------------------------------------------------------------------
// Arithmetic type used inside kernels: fp32 for r16/r32, fp64 for r64.
// ---------------------------------------------------------------------------
template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type mp_up(T x) { return x; }
template <> __device__ __forceinline__ float mp_up<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T mp_down(typename Acc<T>::type x) { return static_cast<T>(x); }
template <> __device__ __forceinline__ __half mp_down<__half>(float x) { return __float2half_rn(x); }

// Host scalar (double) to T with a single rounding, as the reference's
// static_cast<Scalar>(double) does in every launcher.
template <typename T> static inline T mp_host_cast(double x) { return static_cast<T>(x); }
template <> inline __half mp_host_cast<__half>(double x) { return __double2half(x); }

// ---------------------------------------------------------------------------
// 16-byte packs with streaming (evict-first) global accesses.
// ---------------------------------------------------------------------------
template <typename T>
struct alignas(16) Pack {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Pack<T> ld_pack_stream(const T* base, size_t vec_index) {
  union { uint4 u; Pack<T> p; } x;
  x.u = __ldcs(reinterpret_cast<const uint4*>(base) + vec_index);
  return x.p;
}
template <typename T>
__device__ __forceinline__ Pack<T> ld_pack(const T* base, size_t vec_index) {
  union { uint4 u; Pack<T> p; } x;
  x.u = *(reinterpret_cast<const uint4*>(base) + vec_index);
  return x.p;
}
template <typename T>
__device__ __forceinline__ void st_pack_stream(T* base, size_t vec_index, const Pack<T>& p) {
  union { uint4 u; Pack<T> p; } x;
  x.p = p;
  __stcs(reinterpret_cast<uint4*>(base) + vec_index, x.u);
}
template <typename T>
__device__ __forceinline__ void st_pack(T* base, size_t vec_index, const Pack<T>& p) {
  union { uint4 u; Pack<T> p; } x;
  x.p = p;
  *(reinterpret_cast<uint4*>(base) + vec_index) = x.u;
}

// Pack <-> arithmetic-type arrays.  The r16 forms convert two values per
// instruction (half2 <-> float2).
template <typename T>
__device__ __forceinline__ void unpack(const Pack<T>& p, typename Acc<T>::type* out) {
#pragma unroll
  for (int e = 0; e < Pack<T>::N; ++e) out[e] = mp_up(p.v[e]);
}
template <>
__device__ __forceinline__ void unpack<__half>(const Pack<__half>& p, float* out) {
  const __half2* h = reinterpret_cast<const __half2*>(p.v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ Pack<T> pack(const typename Acc<T>::type* in) {
  Pack<T> r;
#pragma unroll
  for (int e = 0; e < Pack<T>::N; ++e) r.v[e] = mp_down<T>(in[e]);
  return r;
}
template <>
__device__ __forceinline__ Pack<__half> pack<__half>(const float* in) {
  Pack<__half> r;
  __half2* h = reinterpret_cast<__half2*>(r.v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
  return r;
}

__host__ __device__ static inline bool mp_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// Reductions.
// ---------------------------------------------------------------------------
struct SumOp { template <typename A> __device__ __forceinline__ static A apply(A a, A b) { return a + b; } };
struct MaxOp { template <typename A> __device__ __forceinline__ static A apply(A a, A b) { return a > b ? a : b; } };

template <typename Op, typename A>
__device__ __forceinline__ A warp_reduce(A v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// Butterfly over the low `WIDTH` lanes only (WIDTH a power of two <= 32).
template <typename Op, int WIDTH, typename A>
__device__ __forceinline__ A warp_reduce_width(A v) {
#pragma unroll
  for (int off = WIDTH / 2; off > 0; off >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// All threads of the CTA get the result.  `smem` holds >= 32 values of A and
// may be reused right after the call returns (two barriers inside).
template <typename Op, int THREADS, typename A>
__device__ __forceinline__ A cta_reduce(A v, A* smem, A identity) {
  constexpr int WARPS = THREADS / 32;
  v = warp_reduce<Op>(v);
  if constexpr (WARPS == 1) return v;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  (void)identity;
  A r = smem[lane & (WARPS - 1)];  // WARPS is a power of two: every lane holds one of the partials
  r = warp_reduce_width<Op, WARPS>(r);
  __syncthreads();
  return r;
}

// Stamp the three extern "C" entry points of one launcher from a template
// `impl<T>(args...)`.
#define MP_STAMP3(name, PARAMS, ARGS)                                              \
  extern "C" void launch_##name##_r16 PARAMS { name##_impl<__half> ARGS; }         \
  extern "C" void launch_##name##_r32 PARAMS { name##_impl<float> ARGS; }          \
  extern "C" void launch_##name##_r64 PARAMS { name##_impl<double> ARGS; }
