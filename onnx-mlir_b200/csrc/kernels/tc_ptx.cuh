// Inline-PTX wrappers for the Blackwell tensor-core path shared by the int8
// GEMM and the attention kernel: mbarriers with bounded waits, TMA tile loads,
// tensor-memory allocation / load / store, tcgen05.mma issue and commit, and
// the shared-memory matrix descriptors of 128-byte-swizzled tiles.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace omcuda {

namespace {

// Default upper bound of one device-side wait, in nanoseconds of %globaltimer
// (omcudaDevSetWaitLimitNs changes it; the kernels receive it as an argument).
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// ---- PTX wrappers -------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}

// Non-blocking look at a barrier phase (mbarrier.test_wait never suspends the
// thread): used to start the poll of the next pipeline stage before the
// current stage's MMAs are issued, so that its latency is hidden behind them.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting.  The clock starts
// with this wait (it is first read after 256 failed polls, so a wait that
// succeeds at once never touches it): the limit is time without progress, not
// kernel lifetime, and a long persistent launch is not cut short.
__device__ __forceinline__ bool mbar_wait(
    uint32_t bar, uint32_t parity, volatile int *abort_flag, uint64_t limit_ns) {
  uint32_t spins = 0;
  uint64_t t_start = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag)
        return false;
      const uint64_t now = global_timer();
      if (t_start == 0) {
        t_start = now;
      } else if (now - t_start > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// Starts the fetch of a tensor map (a kernel parameter) so that the first
// TMA operation on it does not wait for the descriptor.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map,
    int32_t x, int32_t y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// L2 eviction policies for TMA copies: evict_first for data that streams
// through once (outputs, operands read by one tile row), evict_last for the
// operand every tile re-reads (the weights).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map,
    int32_t x, int32_t y, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d_hint(
    const CUtensorMap *map, uint32_t src, int32_t x, int32_t y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint"
      " [%0, {%2, %3}], [%1], %4;" ::"l"(map),
      "r"(src), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// TMA store of a shared-memory box to global memory (bulk async group).
__device__ __forceinline__ void tma_store_2d(
    const CUtensorMap *map, uint32_t src, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
      "r"(src), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Until the stores committed so far have read their shared-memory source.
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Until the stores committed so far are complete.
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Makes shared-memory writes of this thread visible to the async (TMA) proxy.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_dst),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                   : "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Four MMAs over the four 32-byte K slices of one 128-byte operand row,
// issued back to back from one asm block: a lone thread's instructions between
// two tcgen05.mma (descriptor arithmetic, predicate set-up) delay the next
// issue by tens of cycles each, and the tensor pipe idles meanwhile.  The
// descriptors of slice k are those of slice 0 plus 2 k (32 bytes >> 4).
__device__ __forceinline__ void umma_i8_x4(uint32_t d_tmem, uint64_t adesc,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile("{\n\t"
               ".reg .pred p, t;\n\t"
               ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "setp.eq.b32 t, 0, 0;\n\t"
               "add.u64 a1, %1, 2;\n\t"
               "add.u64 a2, %1, 4;\n\t"
               "add.u64 a3, %1, 6;\n\t"
               "add.u64 b1, %2, 2;\n\t"
               "add.u64 b2, %2, 4;\n\t"
               "add.u64 b3, %2, 6;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %3, t;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], a2, b2, %3, t;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], a3, b3, %3, t;\n\t"
               "}" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
               : "memory");
}

// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread
// has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          bar)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
        "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
        "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128
// bytes with the 128-byte swizzle (what the TMA loads above write): eight rows
// form one 1024-byte swizzle atom, so the stride between 8-row groups is 1024
// bytes; the leading-dimension offset is not used by swizzled K-major layouts.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused)
  d |= (uint64_t)(1024u >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                    // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                    // layout: 128-byte swizzle
  return d;
}


// ---- thread-block-cluster helpers (2-CTA kernel) -------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Address of the same shared-memory location in another CTA of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on an mbarrier that may live in the peer CTA (cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                   cluster_addr)
               : "memory");
}

// TMA load of one CTA of a pair; completion bytes go to the mbarrier at
// cluster address `bar` (the leader CTA's).  Plain load: every CTA fetches
// its own tile, nothing is multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst,
    const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst,
    const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_dst),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::
                   : "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr),
               "r"(ncols)
               : "memory");
}

// One MMA over both CTAs of the pair: M = 256 (128 rows from each CTA's A
// tile), N = BN (each CTA's shared memory holds half of the B tile), K = 32.
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t adesc,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}

// The same four-slice issue for the CTA pair.
__device__ __forceinline__ void umma_i8_pair_x4(uint32_t d_tmem, uint64_t adesc,
    uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first) {
  asm volatile("{\n\t"
               ".reg .pred p, t;\n\t"
               ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "setp.eq.b32 t, 0, 0;\n\t"
               "add.u64 a1, %1, 2;\n\t"
               "add.u64 a2, %1, 4;\n\t"
               "add.u64 a3, %1, 6;\n\t"
               "add.u64 b1, %2, 2;\n\t"
               "add.u64 b2, %2, 4;\n\t"
               "add.u64 b3, %2, 6;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], a1, b1, %3, t;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], a2, b2, %3, t;\n\t"
               "tcgen05.mma.cta_group::2.kind::i8 [%0], a3, b3, %3, t;\n\t"
               "}" ::"r"(d_tmem),
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
               : "memory");
}

// Arrives, once the MMAs issued so far have completed, on the mbarrier at this
// shared-memory offset in every CTA whose bit is set in cta_mask.  (This is a
// barrier signal, not a data load.)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

} // namespace

// Host-side helpers shared by the tensor-core kernels (gemm_tc.cu).
int make_tma_map_2d(CUtensorMap *map, const void *base, int64_t rows,
    int64_t cols, int64_t pitch, int box_cols, int box_rows, int esize,
    int swizzle_bytes);
// Per-device status word the tensor-core kernels raise on a bounded-wait
// timeout (device of the calling thread), and the wait limit they are given.
int *tc_status_word();
uint64_t tc_wait_limit_ns();

} // namespace omcuda
