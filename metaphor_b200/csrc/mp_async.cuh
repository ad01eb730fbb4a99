// Asynchronous-copy primitives for sm_100a: shared-memory mbarriers with
// BOUNDED waits, 1-D bulk copies (cp.async.bulk), tiled TMA loads
// (cp.async.bulk.tensor, every copy addressed to a single CTA) and the proxy fences
// that go with them.
//
// Every wait gives up after MP_WAIT_LIMIT_NS, records MP_STATUS_WAIT_TIMEOUT in
// the stream's status word and reports failure to the caller, which must stop
// issuing work and leave the kernel; the host reads the word with mpGetStatus.
#pragma once

#include "mp_common.cuh"

#ifndef MP_WAIT_LIMIT_NS
#define MP_WAIT_LIMIT_NS 2000000000ull  // 2 s: the limit when the stream's state carries none
#endif

__device__ __forceinline__ uint32_t mp_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t mp_globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The stream's status block: word 0 = status, bytes 8..15 = wait limit in nanoseconds (0 = the default above),
// set by mpSetWaitLimit or the MP_SPIN_LIMIT_US environment variable.  Read only on the slow path of a wait.
__device__ __forceinline__ uint64_t mp_wait_limit_ns(const uint32_t* status) {
  if (status == nullptr) return MP_WAIT_LIMIT_NS;
  const uint64_t v = *reinterpret_cast<const volatile uint64_t*>(status + 2);
  return v != 0 ? v : MP_WAIT_LIMIT_NS;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mp_smem_u32(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (TMA unit).
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mp_smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mp_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(mp_smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Same test, but the warp may be suspended by the hardware for up to `hint_ns`
// while the phase is incomplete (a waiting warp then stops competing for issue
// slots with the warps that do the work).
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(mp_smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

// Bounded wait for the phase with the given parity.  Returns false (after
// setting the status word) if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = mp_globaltimer_ns();
  const uint64_t limit = mp_wait_limit_ns(status);
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait_suspend(bar, parity, 20000u)) return true;
    if (mp_globaltimer_ns() - t0 > limit) {
      if (status != nullptr) atomicExch(status, MP_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   mp_smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(mp_smem_u32(bar))
               : "memory");
}

// Same with an L2 evict-first policy: streamed-once inputs do not displace
// data other kernels keep resident.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_load_1d_hint(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar,
                                                  uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          mp_smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(mp_smem_u32(bar)), "l"(policy)
      : "memory");
}

// 1-D bulk copy shared -> global (bulk async-group completion).
__device__ __forceinline__ void bulk_store_1d(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(mp_smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N committed bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Orders generic-proxy shared-memory writes before async-proxy (TMA) reads.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Named barrier over a subset of the CTA's warps (count = participating threads).
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
