// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM
// kernels use: mbarriers, TMA tensor loads, tcgen05 MMA / TMEM.  Every wait is
// bounded: it returns false after a cycle budget instead of spinning forever.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same with a suspend-time hint: the hardware may park the thread for up to `ns`
// nanoseconds (or until the phase completes), so that a waiting warp does not take issue
// slots from the warps that do the arithmetic.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}

// Pause between polls: a waiting warp that polls back to back takes issue slots from the
// warps that do the arithmetic (measured: the 4096^3 GEMM is 4 % faster with the pause).
#ifndef MB_WAIT_BACKOFF_NS
#define MB_WAIT_BACKOFF_NS 20
#endif

// Wait for the phase with the given parity to complete.  Gives up after
// `budget` clock cycles or as soon as *abort_flag becomes non-zero; returns
// false in both cases.  (mbarrier.try_wait itself parks the thread for a short,
// implementation-defined time per poll; a longer suspend-time hint made wake-ups late.)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile int *abort_flag,
                                          long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    __nanosleep(MB_WAIT_BACKOFF_NS);
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - start > budget) return false;
  }
}

// A wait for roles that are far ahead of the pipeline (producer, preparation):
// sleeps between polls so that the polling does not take issue slots from the
// warps that do the arithmetic.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity,
                                                  volatile int *abort_flag, long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    __nanosleep(64);
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - start > budget) return false;
  }
}

// The same for a whole warp that waits together: every lane polls, and the
// warp takes one common decision, so that it stays converged for the
// warp-aligned instructions that follow (tcgen05.ld, __syncwarp, ...).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile int *abort_flag, long long budget) {
  const bool ok = mbar_wait(bar, parity, abort_flag, budget);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ bool mbar_wait_warp_relaxed(uint32_t bar, uint32_t parity,
                                                       volatile int *abort_flag,
                                                       long long budget) {
  const bool ok = mbar_wait_relaxed(bar, parity, abort_flag, budget);
  return __all_sync(0xffffffffu, ok);
}

// Ask for the 128-byte line that holds `p` to be brought into L2.
__device__ __forceinline__ void prefetch_l2(const void *p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Barrier among `threads` threads (a multiple of 32) of the CTA; id 0 is __syncthreads'.
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- TMA ----------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map))
               : "memory");
}

// Untiled bulk copy global -> shared of this CTA, completion counted in bytes on an mbarrier of
// this CTA.  Both addresses 16-byte aligned, the size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void *src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

// 3-D tiled load global -> shared of this CTA, completion counted in bytes on
// an mbarrier of this CTA.  c0 is the innermost coordinate and must keep the
// copy 16-byte aligned (for uint8: a multiple of 16).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap *map,
                                            uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0),
        "r"(c1), "r"(c2)
      : "memory");
}

// Ask for the box of a 3-D tiled tensor to be brought into L2 (no shared memory, no completion
// to wait for): lets a producer run further ahead of HBM than its shared-memory ring allows.
// 4-D tiled load (for an NHWC tensor: c0 = channel byte, c1 = column, c2 = row, c3 = image).
// c0 must keep the copy 16-byte aligned; the other coordinates may lie outside the tensor
// (negative or too large): those elements arrive as the map's fill value, zero.
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap *map, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap *map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

// 3-D tiled store shared -> global (bulk async-group completion).  Writes outside the
// tensor's extents are clipped by the hardware.  c0 must keep the store 16-byte aligned,
// and no coordinate may be negative.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src_smem, int c0,
                                             int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until all but the newest N bulk groups of this thread have finished READING their
// shared-memory source (the buffer may be overwritten) ...
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// ... or have completed entirely (their global writes are done).
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- CTA pairs (a cluster of two) -----------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Every thread of every CTA of the cluster; orders shared-memory accesses (barrier
// initialisation before, remote arrivals after) across the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The shared::cluster address of `addr` (a shared::cta address of this CTA's layout) in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

// Arrive on an mbarrier of another CTA of the cluster (address from mapa_shared).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // (default semantics: a .release.cluster here made every arrival cost most of a microsecond)
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Wait on an mbarrier of this CTA that a thread of the other CTA arrives on.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                  long long budget) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    __nanosleep(MB_WAIT_BACKOFF_NS);
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - start > budget) return false;
  }
}

// A tile into THIS CTA's shared memory whose arrival is counted on an mbarrier of the pair's
// even CTA (`bar_cluster`: a shared::cluster address from mapa_shared).  No multicast: every CTA
// fetches its own bytes.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst_smem, const CUtensorMap *map, uint32_t bar_cluster,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---- tcgen05 / TMEM -----------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   dst_smem),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
               "r"(ncols)
               : "memory");
}

// The same three for a CTA pair: one warp of EACH of the two CTAs executes them; both get
// the same columns.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], uint8/int8 inputs, int32 accumulation.
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc,
                                          uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same over a CTA pair, issued by one thread of the even CTA: M = 256 (each CTA's 128 rows
// of A from its own shared memory into its own tensor memory), each CTA holding half of B's
// N columns at the same shared-memory offset.
__device__ __forceinline__ void mma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Completion of the pair's MMAs issued so far arrives on the mbarrier at this shared-memory
// offset in every CTA of `cta_mask`.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], tf32 inputs, fp32 accumulation.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc,
                                            uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem], tf32 inputs, fp32 accumulation: A lies in tensor memory,
// lane = row of A, one 32-bit column per k.
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem,
                                            uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16 consecutive 32-bit columns of this warp's 32 TMEM lanes <- one register per column.
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// Make an mbarrier of this CTA track completion of all MMAs issued so far by
// this thread.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          bar)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives
// columns [col, col+32) of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
      "[%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
        "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
        "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Wait for outstanding tcgen05.ld and tie the destination registers to the
// wait, so that the compiler cannot schedule arithmetic on them above it (the
// load writes its registers asynchronously; they are valid only after this).
__device__ __forceinline__ void tmem_ld_wait_x16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                 "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                 "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors ---------------------------------------------------------------

// Shared-memory matrix descriptor (64-bit) for tcgen05.mma:
//  [0,14)  start address >> 4      [16,30) leading-dimension byte offset >> 4
//  [32,46) stride-dimension byte offset >> 4       [46,48) version = 1
//  [49,52) base offset (0: tiles are 1024-byte aligned)
//  [61,64) swizzle mode: 0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(swizzle & 7u) << 61;
  return d;
}

// Instruction descriptor (32-bit) for dense tcgen05.mma:
//  [4,6) accumulator format (1 = f32, 2 = s32)   [7,10) A format   [10,13) B format
//  [15] A is MN-major   [16] B is MN-major   [17,23) N >> 3   [24,29) M >> 4
// kind::i8 formats: 0 = unsigned 8-bit, 1 = signed 8-bit.
// kind::tf32 / f16 formats: 0 = f16, 1 = bf16, 2 = tf32.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_fmt, uint32_t a_fmt,
                                                  uint32_t b_fmt, bool a_mn_major,
                                                  bool b_mn_major, uint32_t m, uint32_t n) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace sm100
