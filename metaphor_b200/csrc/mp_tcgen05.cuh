// 5th-generation tensor core (tcgen05) and tiled-TMA primitives for sm_100a,
// as inline PTX: TMEM allocation, UMMA shared-memory / instruction descriptors,
// tcgen05.mma / commit / ld, and cp.async.bulk.tensor loads (each addressed to a single CTA).
#pragma once

#include "mp_async.cuh"

// ------------------------------ TMA (tiled) --------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tile load: coordinates are (x = innermost element index, y = row index).
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          mp_smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(mp_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// 2-D tile store shared -> global (bulk async group).  Elements outside the
// tensor are not written, so edge tiles need no masking.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(mp_smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

// 3-D forms (x, y as above, z = batch index): the tile in shared memory has the 2-D layout.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          mp_smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(mp_smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(mp_smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

// ------------------------------ TMEM ---------------------------------------
// Executed by ONE full warp.  ncols: power of two in [32, 512].  The base
// address is written to *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mp_smem_u32(smem_slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------ descriptors --------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1:
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version = 1
//   bits [61,64) layout type (2 = SWIZZLE_128B)
// K-major operand tile (rows of 128 bytes along K, 8-row groups of 1024 bytes):
//   LBO unused (1), SBO = 1024 bytes.
// MN-major operand tile (k-rows of 128 bytes along MN, 8 k-rows = 1024 bytes,
//   next 128-byte column block `block_bytes` further): LBO = block_bytes, SBO = 1024.
//
// 32-bit MN-major operands (tf32) must use layout type 1 instead
// (SWIZZLE_128B_BASE32B: 32-byte chunks swizzled within groups of four 128-byte
// k-rows, written by TMA with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B); their
// SBO is the pitch of such a 4-row group, 512 bytes.
constexpr uint32_t UMMA_LAYOUT_SW128 = 2, UMMA_LAYOUT_SW128_BASE32B = 1;
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type = UMMA_LAYOUT_SW128) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout_type) << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::tf32, fp32 accumulation:
//   [4,6) D format (1 = F32)   [7,10) A format   [10,13) B format (0 = F16, 1 = BF16, 2 = TF32)
//   [15] A major  [16] B major (0 = K, 1 = MN)   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_instr_desc(uint32_t ab_format, uint32_t a_mn_major, uint32_t b_mn_major,
                                                       uint32_t m, uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}
constexpr uint32_t UMMA_FMT_F16 = 0, UMMA_FMT_BF16 = 1, UMMA_FMT_TF32 = 2;

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
template <bool TF32>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (TF32) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// The mbarrier receives one arrival when every tcgen05.mma issued so far by
// this thread has completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mp_smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread i
// of the warp reads lane i of the warp's TMEM quarter).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// Same for 16 consecutive columns -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded mbarrier wait that also gives up as soon as another role of the CTA
// has raised `*abort` (so one timeout ends every loop of the CTA quickly).
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, uint32_t* status, volatile int* abort) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = mp_globaltimer_ns();
  const uint64_t limit = mp_wait_limit_ns(status);
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait_suspend(bar, parity, 20000u)) return true;
    if (*abort != 0) return false;
    if (mp_globaltimer_ns() - t0 > limit) {
      *abort = 1;
      if (status != nullptr) atomicExch(status, MP_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
}

// ------------------------------ CTA pairs (cta_group::2) ---------------------
// Two CTAs of a cluster (ranks 0 and 1) work on one 256-row tile: each holds its 128 rows of A and one
// half of B's columns in its own shared memory and its 128 accumulator rows in its own TMEM; the MMA is
// issued by one thread of rank 0 and reads both CTAs' shared memory at the same offsets.  Every copy and
// every barrier arrival below is addressed to exactly one CTA.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {   // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One arrival on the barrier at the same shared-memory offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta) {
  asm volatile(
      "{\n.reg .b32 remote;\n"
      "mapa.shared::cluster.u32 remote, %0, %1;\n"
      "mbarrier.arrive.shared::cluster.b64 _, [remote];\n}\n" ::"r"(mp_smem_u32(bar)),
      "r"(cta)
      : "memory");
}
// Tile load whose byte count is credited to the barrier at `bar`'s offset in rank 0's shared memory
// (bit 24 of a shared::cluster address is the rank within the pair).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          mp_smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(mp_smem_u32(bar) & 0xFEFFFFFFu), "r"(x), "r"(y)
      : "memory");
}
// Executed by the same warp index of BOTH CTAs, with the same smem_slot offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mp_smem_u32(smem_slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A (128 rows per CTA) * B (N/2 columns per CTA); ONE thread of rank 0.
__device__ __forceinline__ void umma_pair_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at `bar`'s offset in EVERY CTA of `cta_mask` (bit i = cluster rank i) when every pair
// MMA issued so far by this thread has completed: both CTAs of a pair learn of a free stage / a finished
// accumulator from the hardware instead of through a relayed software arrival.
__device__ __forceinline__ void umma_commit_pair_to(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(mp_smem_u32(bar)),
               "h"(cta_mask)
               : "memory");
}
// One arrival on rank 0's barrier when every pair MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mp_smem_u32(bar))
               : "memory");
}
