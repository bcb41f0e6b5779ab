// Shared device/host helpers for the sm_100a kernels: status codes, bounded
// mbarrier waits, TMA / tcgen05 PTX wrappers and tensor-map construction.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/samb200.h"

namespace samb {

// ----------------------------------------------------------------------------------------------
// Device status word.  A kernel that gives up on a wait stores
//   (SAMB_DEV_TIMEOUT << 24) | (site << 16) | (blockIdx.x & 0xffff)
// with atomicCAS(status, 0, code), so the first failure is kept.
// ----------------------------------------------------------------------------------------------
constexpr uint32_t kDevTimeout = 0x7Eu;
constexpr uint32_t kDevNot24 = 0x7Du;     // status-word tag: a weight group of four held more than two non-zeros

// Poll budget of one wait: ~4 M polls, the late ones 64 ns apart => a fraction of a second.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// One arrival per warp instead of 32: every lane has already issued its own fences; __syncwarp orders
// the lanes' writes before lane 0's (release) arrive.  128 same-address arrivals would serialise.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

// Non-blocking poll (try_wait may park the thread for a while; this never does).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false after the poll budget (or as soon as another thread of the CTA
// has flagged an abort), having recorded the site in the status word and raised the CTA-wide
// abort flag.  Callers leave their role loop on false; every wait in a kernel is bounded, so the
// whole CTA drains and reaches its teardown.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, uint32_t site, uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 2048u) {
      if (*abort_flag) return false;
      __nanosleep(64);
    }
  }
  *abort_flag = 1;
  if (status != nullptr) atomicCAS(status, 0, int((kDevTimeout << 24) | ((site & 0xffu) << 16) | (blockIdx.x & 0xffffu)));
  return false;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// TMA (no multicast anywhere: every CTA fetches its own tiles from this GPU's memory)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; kind::f16 (bf16/fp16 inputs, fp32 accumulate)
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Predicated forms: every lane of the warp executes the statement (warp-uniform control flow, so the
// descriptors can live in uniform registers); only lanes with `issue != 0` really issue.
__device__ __forceinline__ void umma_f16_ss_if(uint32_t issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ts_if(uint32_t issue, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void tc_commit_if(uint32_t issue, uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(smem_u32(bar)), "r"(issue)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::i8 (s8 inputs, s32 accumulate)
__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// kind::i8 with a 2:4-sparse A operand: A in shared memory holds the kept half of every group of four
// K elements; the 4-bit position codes (one bit per logical K element, 64 bits per row per MMA of
// logical K = 64) sit in tensor memory at e_tmem, row r of A in lane r.
__device__ __forceinline__ void umma_i8_sp_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared memory -> tensor memory, 128 lanes x 128 bits (4 columns); ordered with the MMAs that the
// same thread issues after it.
__device__ __forceinline__ void tmem_cp_128x128b(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// ---- CTA pairs (thread-block cluster of two, tcgen05 cta_group::2): one MMA spans both CTAs' tensor
// memory (M = 256: 128 rows each) and reads half of the B operand from each CTA's shared memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {          // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a shared-memory object of this CTA) in the CTA of the given rank
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Arrival without release semantics: for a thread that has nothing to publish (its tensor-memory loads are already
// complete) and must not pay for a cluster-scope fence.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {   // same warp of both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load into this CTA's shared memory whose bytes are counted on the barrier at cluster address bar_cluster
// (the leader CTA's barrier); no multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_sp_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t e_tmem,
                                                   uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::2.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared memory -> tensor memory in both CTAs of the pair (each from its own shared memory, same offsets).
__device__ __forceinline__ void tmem_cp_128x128b_pair(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// Arrives (once all MMAs issued so far by this thread have completed) on the barrier at the given
// shared::cluster address (this CTA's or the peer's: see map_to_cta).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets TMEM lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start>>4 | LBO>>4 <<16 | SBO>>4 <<32 |
// version(1)<<46 | swizzle<<61.
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint64_t swizzle) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32) | (uint64_t(1) << 46) | (swizzle << 61);
}

// Instruction descriptor: D format bits[4,6), A format [7,10), B format [10,13), A major bit 15,
// B major bit 16 (0 = K-major), N>>3 at [17,23), M>>4 at [24,29).
constexpr uint32_t kFmtF16 = 0, kFmtBF16 = 1;      // kind::f16 operand formats
constexpr uint32_t kFmtU8 = 0, kFmtS8 = 1;         // kind::i8 operand formats
constexpr uint32_t kAccF32 = 1, kAccS32 = 2;       // accumulator formats
__host__ __device__ constexpr uint32_t make_idesc(uint32_t acc_fmt, uint32_t a_fmt, uint32_t b_fmt, int M, int N,
                                                  bool a_mn_major = false, bool b_mn_major = false) {
  return (acc_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// Exact-form GELU x * Phi(x) = max(x, 0) - |x| * erfc(|x| / sqrt 2) / 2.  log2(erfc(a / sqrt 2) / 2) is smooth on
// [0, 6.08] (beyond it the term is below 1e-9 |x|) and a degree-7 polynomial in a = |x| (Chebyshev fit) follows it
// closely enough that the result is within 5.1e-7 of the exact GELU everywhere, far below the bf16 output rounding:
// seven FMAs and one ex2, no division (the erf rational approximations cost a second special-function op, which is
// what binds the int8 GEMM epilogue).
__device__ __forceinline__ float gelu_erf(float x) {
  const float a = fminf(fabsf(x), 6.0811f);
  float q = fmaf(-1.926999857e-06f, a, 6.350679178e-05f);
  q = fmaf(q, a, -9.461226873e-04f);
  q = fmaf(q, a, 8.571726270e-03f);
  q = fmaf(q, a, -5.409686640e-02f);
  q = fmaf(q, a, -4.583186507e-01f);
  q = fmaf(q, a, -1.151316047e+00f);
  q = fmaf(q, a, -9.999877214e-01f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(q));
  return fmaf(-fabsf(x), e, fmaxf(x, 0.0f));
}

// Packed fp32 pairs (sm_100: one instruction performs two IEEE fp32 operations on a 64-bit register pair; each
// half is rounded exactly as the scalar instruction would round it).  They halve the issue slots of fp32 math in
// kernels that are bound by instruction issue rather than by the FMA pipe.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 ffma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 fadd2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 fsub2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 fmul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// the two bf16 halves of a word as an fp32 pair
__device__ __forceinline__ f32x2 bf16x2_to_f32x2(uint32_t w) {
  return pack2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// gelu_erf on a pair: the polynomial runs on packed fp32 instructions (seven for two elements); the clamp,
// the two ex2 and the max(x, 0) stay scalar.  Each half gets exactly the bits gelu_erf gives it.
__device__ __forceinline__ f32x2 gelu_erf2(f32x2 x2) {
  float x0, x1;
  unpack2(x2, x0, x1);
  const f32x2 a2 = pack2(fminf(fabsf(x0), 6.0811f), fminf(fabsf(x1), 6.0811f));
  f32x2 q = ffma2(pack2(-1.926999857e-06f, -1.926999857e-06f), a2, pack2(6.350679178e-05f, 6.350679178e-05f));
  q = ffma2(q, a2, pack2(-9.461226873e-04f, -9.461226873e-04f));
  q = ffma2(q, a2, pack2(8.571726270e-03f, 8.571726270e-03f));
  q = ffma2(q, a2, pack2(-5.409686640e-02f, -5.409686640e-02f));
  q = ffma2(q, a2, pack2(-4.583186507e-01f, -4.583186507e-01f));
  q = ffma2(q, a2, pack2(-1.151316047e+00f, -1.151316047e+00f));
  q = ffma2(q, a2, pack2(-9.999877214e-01f, -9.999877214e-01f));
  float q0, q1, e0, e1;
  unpack2(q, q0, q1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(q0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(q1));
  return ffma2(pack2(-fabsf(x0), -fabsf(x1)), pack2(e0, e1), pack2(fmaxf(x0, 0.0f), fmaxf(x1, 0.0f)));
}

// Eight accumulator columns of one output row through the GEMM epilogue arithmetic, two at a time:
// int8: (float(acc) * a_scale) * w_scale[n]; then + bias[n]; then the exact GELU.  `ws` / `bs` point at eight
// consecutive per-column values (16-byte aligned, shared memory).  Same roundings as the scalar sequence.
template <bool kInt8, bool kScale, bool kBias, bool kGelu>
__device__ __forceinline__ void epilogue8(const uint32_t* r, float a_scale, const float* ws, const float* bs,
                                          float (&v)[8]) {
  const f32x2 as2 = pack2(a_scale, a_scale);
  ulonglong2 w01 = make_ulonglong2(0ull, 0ull), w23 = w01, b01 = w01, b23 = w01;
  if (kScale) {
    w01 = *reinterpret_cast<const ulonglong2*>(ws);
    w23 = *reinterpret_cast<const ulonglong2*>(ws + 4);
  }
  if (kBias) {
    b01 = *reinterpret_cast<const ulonglong2*>(bs);
    b23 = *reinterpret_cast<const ulonglong2*>(bs + 4);
  }
  const f32x2 wv[4] = {w01.x, w01.y, w23.x, w23.y}, bv[4] = {b01.x, b01.y, b23.x, b23.y};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f32x2 x;
    if (kInt8) x = fmul2(pack2(float(int(r[2 * j])), float(int(r[2 * j + 1]))), as2);
    else x = pack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
    if (kScale) x = fmul2(x, wv[j]);
    if (kBias) x = fadd2(x, bv[j]);
    if (kGelu) x = gelu_erf2(x);
    unpack2(x, v[2 * j], v[2 * j + 1]);
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
      "elect.sync R|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------------------------
// Tiled tensor map over a row-major view.  dims/strides innermost first; strides[0] is implied
// (element size).  Returns 0 or a negative SAMB_E_* code.
int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

int check_device_arch();   // 0 if the current device is sm_100, SAMB_E_ARCH otherwise
// CTA-pair GEMM (gemm_pair.cu); SAMB_E_SHAPE = not covered, use the single-CTA kernel
int launch_gemm_pair(bool int8, const void* A, int64_t lda, const void* W, int64_t ldw, const float* a_scale,
                     const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                     void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int head_dim, int32_t* status,
                     void* stream, float* row_absmax = nullptr);
// The int8 Linear GEMM (gemm_tc.cu) that also leaves, through atomic maxima, the largest |bf16(out[m, n])| of every
// output row m in row_absmax[m] (float, non-negative, zeroed by the caller beforehand).
int launch_gemm_i8_rowmax(const int8_t* Aq, int64_t lda, const float* a_scale, const int8_t* Wq, int64_t ldw,
                          const float* w_scale, const float* bias, const void* residual, int64_t ldr, int64_t res_rows,
                          void* out, int64_t ldo, int64_t M, int N, int K, int epilogue, int32_t* status, void* stream,
                          float* row_absmax);
// The 2:4-sparse int8 Linear GEMM (gemm_sp24.cu); row_absmax as in launch_gemm_i8_rowmax (may be null).
int launch_gemm_i8_sp24(const int8_t* Xq, int64_t ldx, const float* x_scale, const int8_t* Wc, int64_t ldc,
                        const uint8_t* meta, const float* w_scale, const float* bias, const void* residual,
                        int64_t ldr, int64_t res_rows, void* out, int64_t ldo, int64_t T, int N, int K, int epilogue,
                        int32_t* status, void* stream, float* row_absmax);
int sm_count();

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SAMB_OK : SAMB_E_LAUNCH;
}

}  // namespace samb
