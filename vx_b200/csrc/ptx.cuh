/* ptx.cuh -- the sm_100a instructions the tensor-core kernels are made of:
 * mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
 * (TMEM allocation, MMA, commit, load) and the descriptors they take.
 *
 * Every wait is bounded: it gives up after kWaitCycles SM cycles and returns
 * false, so that a kernel can record where it stopped and leave, instead of
 * spinning on a GPU that other people share.
 */
#ifndef VXB_PTX_CUH
#define VXB_PTX_CUH

#include <cuda.h>
#include <stdint.h>

namespace vxb {
namespace ptx {

constexpr long long kWaitCycles = 1ll << 31; /* about a second */

__device__ inline uint32_t smem_addr(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

/* ---- mbarrier ------------------------------------------------------------- */
__device__ inline void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(count));
}
__device__ inline void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ inline void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ inline void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                   smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ inline void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar))
               : "memory");
}
__device__ inline bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done)
               : "r"(smem_addr(bar)), "r"(parity)
               : "memory");
  return done != 0;
}
/* Wait for the phase with this parity to end. `stop` is a shared flag that any
   role sets when it gives up; seeing it set ends this wait too. */
__device__ inline bool mbar_wait(uint64_t *bar, uint32_t parity,
                                 volatile int *stop) {
  if (mbar_try_wait(bar, parity))
    return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity))
        return true;
    if (*stop || clock64() - t0 > kWaitCycles)
      return false;
  }
}

/* The same wait with no stop flag: for a role that has given up already and
   only waits for its own copies to land before it leaves. */
__device__ inline bool mbar_wait_alone(uint64_t *bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - t0 > kWaitCycles)
      return false;
  return true;
}

/* ---- TMA -------------------------------------------------------------------
 * Tiled loads into this CTA's shared memory, completion counted in bytes on an
 * mbarrier. x is the innermost coordinate; x * element size must be a multiple
 * of 16 bytes. */
__device__ inline void tma_load_2d(void *dst, const CUtensorMap *map, int x,
                                   int y, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::"
               "complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_addr(dst)),
               "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
               : "memory");
}
__device__ inline void tma_load_4d(void *dst, const CUtensorMap *map, int c0,
                                   int c1, int c2, int c3, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::"
               "complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                   smem_addr(dst)),
               "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
               "r"(smem_addr(bar))
               : "memory");
}
/* An untiled bulk copy of `bytes` (a multiple of 16; both addresses 16-byte
   aligned) from global memory into this CTA's shared memory. */
__device__ inline void bulk_load(void *dst, const void *src, uint32_t bytes,
                                 uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::"
               "bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
/* Ask L2 for `bytes` (a multiple of 16, from a 16-byte aligned address):
   nothing is written anywhere the program can see. */
__device__ inline void bulk_prefetch_l2(const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes)
               : "memory");
}
__device__ inline void tma_prefetch_desc(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
/* Tiled store from shared memory, tracked by the bulk async-group. */
__device__ inline void tma_store_2d(const CUtensorMap *map, const void *src,
                                    int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group "
               "[%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_addr(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ inline void tma_store_4d(const CUtensorMap *map, const void *src,
                                    int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group "
               "[%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_addr(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ inline void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int kPending> __device__ inline void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
template <int kPending> __device__ inline void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

/* ---- tcgen05: tensor memory ----------------------------------------------- */
/* One whole warp allocates `cols` (a power of two, 32..512) TMEM columns; the
   base address lands in *slot (shared memory). */
__device__ inline void tmem_alloc(uint32_t *slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::
                   "r"(smem_addr(slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                   : "memory");
}
__device__ inline void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base),
               "r"(cols)
               : "memory");
}
__device__ inline void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ inline void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

/* ---- tcgen05: descriptors --------------------------------------------------
 * Shared-memory matrix descriptor (64 bits): start address >> 4 in bits 0-13,
 * leading byte offset >> 4 in 16-29, stride byte offset >> 4 in 32-45, the
 * constant 1 in bits 46-47 (sm_100 format), swizzle mode in 61-63
 * (2 = 128-byte swizzle). */
__device__ inline uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                           uint32_t sbo_bytes) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) |
         ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) |
         (2ull << 61);
}
/* Instruction descriptor for kind::f16 with an f32 accumulator: D format f32
   (bits 4-5 = 1), A and B format in 7-9 and 10-12 (0 f16, 1 bf16), A/B
   major-ness in bits 15/16 (1 = the M or N index is the contiguous one), N>>3
   in 17-22, M>>4 in 24-28. */
__host__ __device__ inline uint32_t idesc_f16(bool bf16, bool a_mn_major,
                                              bool b_mn_major, int m, int n) {
  const uint32_t fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

/* D[tmem] (+)= A[smem] * B[smem]; issued by one thread. */
__device__ inline void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc,
                                   uint64_t b_desc, uint32_t idesc,
                                   uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::
                   "r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
/* D[tmem] (+)= A[tmem] * B[smem]. */
__device__ inline void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem,
                                   uint64_t b_desc, uint32_t idesc,
                                   uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::
                   "r"(d_tmem),
               "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
/* The mbarrier gets one arrival when every MMA this thread issued so far has
   finished. */
__device__ inline void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::"
               "cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}

/* ---- tcgen05: TMEM <-> registers -------------------------------------------
 * 32x32b: lane i of the warp reads TMEM lane (base lane + i); .xN gives N
 * consecutive 32-bit columns. A warp may only touch the 32 lanes of its own
 * quarter: lanes 32*(warp_id % 4) .. +31. */
__device__ inline void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
        "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ inline void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
__device__ inline void tmem_ld_wait_for(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
/* The same wait, tied to the registers of one load: nothing that reads r can
   be scheduled above it, which matters when another load is already in flight
   into a second set of registers. */
__device__ inline void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
        "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]),
        "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
        "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]),
        "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]),
        "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]),
        "+r"(r[31])
      :
      : "memory");
}
__device__ inline void tmem_st_32x32b_x16(uint32_t taddr,
                                          const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
      "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ inline void tmem_st_32x32b_x32(uint32_t taddr,
                                          const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, "
      "%31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
      "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
      "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ inline void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

/* ---- CTA pairs (cta_group::2) ------------------------------------------------
 * Two CTAs of a cluster of two, on the two SMs of one TPC, act as one 256-row
 * tensor-core unit: CTA 0 of the pair (the leader) issues the MMAs, which read
 * the A rows and the B columns that each CTA holds in its OWN shared memory (at
 * the same offsets) and write each CTA's half of the accumulator into that
 * CTA's tensor memory. No load here carries a cluster multicast: each CTA
 * fetches its own halves. */
__device__ inline uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
/* The shared::cluster address of the same variable in CTA `rank` of the
   cluster. */
__device__ inline uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(saddr), "r"(rank));
  return out;
}
/* All threads of all CTAs of the cluster meet. */
__device__ inline void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
/* One arrival on an mbarrier that may be in another CTA of the cluster
   (a shared::cluster address from map_to_cta). */
__device__ inline void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                   cluster_addr)
               : "memory");
}
/* try_wait that also sees what other CTAs of the cluster did before they
   arrived. */
__device__ inline bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done)
               : "r"(smem_addr(bar)), "r"(parity)
               : "memory");
  return done != 0;
}
__device__ inline bool mbar_wait_cluster(uint64_t *bar, uint32_t parity,
                                         volatile int *stop) {
  if (mbar_try_wait_cluster(bar, parity))
    return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait_cluster(bar, parity))
        return true;
    if (*stop || clock64() - t0 > kWaitCycles)
      return false;
  }
}
/* A tiled load into THIS CTA's shared memory whose byte count is reported to
   an mbarrier given as a shared::cluster address: the leader's. */
__device__ inline void tma_load_2d_pair(void *dst, const CUtensorMap *map, int x,
                                        int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global."
               "mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_addr(dst)),
               "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}
/* TMEM of both CTAs of the pair: one warp of EACH CTA executes these. */
__device__ inline void tmem_alloc_pair(uint32_t *slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::
                   "r"(smem_addr(slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::
                   : "memory");
}
__device__ inline void tmem_dealloc_pair(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base),
               "r"(cols)
               : "memory");
}
/* D[tmem of both CTAs] (+)= A * B with M = 256: issued by one thread of the
   leader CTA. */
__device__ inline void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc,
                                        uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::
                   "r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}
/* One arrival on the mbarrier at this offset in BOTH CTAs of the pair when
   every MMA this thread issued so far has finished. */
__device__ inline void umma_commit_pair(uint64_t *bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster."
               "multicast::cluster.b64 [%0], %1;" ::"r"(smem_addr(bar)),
               "h"(both)
               : "memory");
}

__device__ inline bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "elect.sync _|p, 0xffffffff;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(pred));
  return pred != 0;
}

} // namespace ptx
} // namespace vxb

#endif /* VXB_PTX_CUH */
