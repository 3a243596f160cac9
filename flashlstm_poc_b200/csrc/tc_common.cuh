// sm_100a primitives for the tensor-core path, written as inline PTX:
//   mbarrier (init / expect-tx / bounded wait), TMA tiled loads and stores
//   (cp.async.bulk.tensor, one CTA per copy), tcgen05 (TMEM alloc, UMMA issue, commit, TMEM loads),
//   shared-memory matrix descriptors and the UMMA instruction descriptor.
// Every wait is bounded: after its limit (kWaitLimitNs unless the launch passes another one) the waiter raises
// an abort word and returns false, so a kernel always terminates and the host reports FLSTM_ERR_TIMEOUT
// instead of hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace flstm_b200 {
namespace tc {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s: the default limit of every device-side wait
// After an abort a producer still waits this long for ring stages whose copies can no longer complete (one half of a
// stage was fetched ahead of a barrier that then failed); copies that were started land well within it.
constexpr unsigned long long kAbortDrainNs = 20000ull;
constexpr int kMaxRingStages = 32;  // ring stages are tracked in 32-bit masks

// ------------------------------------------------------------------ small utilities
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  `abort_word` lives in shared memory and is shared by every waiter of the CTA.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_word,
                                          unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_test_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (*abort_word) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_word = 1;
                return false;
            }
        }
    }
    return true;
}
// Bounded wait that does not look at the abort word: used on the way out of a kernel to let copies that are
// still in flight towards this CTA's shared memory land before the CTA exits.
__device__ __forceinline__ bool mbar_drain(uint64_t *bar, uint32_t parity, unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_test_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0 && global_timer_ns() - t0 > limit_ns) return false;
    }
    return true;
}

// ------------------------------------------------------------------ proxies and fences
// global memory only: what a TMA load of data that other SMs wrote with ordinary stores needs
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------ TMA (tiled, 2-D)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// global -> shared; x is the innermost coordinate (elements) and must be a multiple of 16 bytes
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *m, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *m, int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *m, int x, int y, int z, int w, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// the same copies with the mbarrier given as a shared-memory address
__device__ __forceinline__ void tma_load_2d_addr(void *smem_dst, const CUtensorMap *m, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_addr(void *smem_dst, const CUtensorMap *m, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_addr(void *smem_dst, const CUtensorMap *m, int x, int y, int z, int w, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// shared -> global
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *m, const void *smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *m, const void *smem_src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
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

// ------------------------------------------------------------------ TMEM
// Allocation is warp-wide; the base address is written to `slot` in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 32 lanes x 32-bit, 32 consecutive columns: thread i of the warp gets lane (base_lane + i)
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ UMMA
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 64 16-bit elements x R rows with SWIZZLE_128B produces).
// Groups of 8 rows are 1024 bytes apart (SBO); the tile base must be 1024-byte aligned.  Advancing
// along K inside the 128-byte row is done by adding the byte offset (>>4) to the start address.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);      // bits [0,14): start address >> 4
    d |= (uint64_t)1 << 16;                            // bits [16,30): leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                  // bits [32,46): stride byte offset >> 4
    d |= (uint64_t)1 << 46;                            // bits [46,48): descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                            // bits [61,64): SWIZZLE_128B
    return d;
}
// MN-major operand tile: rows are K indices, each row holds 64 consecutive M (or N) elements (128 B,
// 128-byte swizzle).  8 K-rows form a 1024-byte group (SBO); a second block of 64 M/N elements lies
// `lbo_bytes` further (LBO).  Advancing K by 16 elements = +2048 bytes on the start address.
__device__ __forceinline__ uint64_t umma_desc_mnmajor_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulator, A/B both f16 (0) or bf16 (1).
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n, int ab_format, int a_mn_major, int b_mn_major) {
    return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)a_mn_major << 15) |
           ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Same, with the accumulate flag known at compile time (no predicate set-up in the issue loop).
template <bool ACC>
__device__ __forceinline__ void umma_f16_imm(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    if (ACC) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.eq.u32 p, 1, 1;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
            : "memory");
    } else {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.eq.u32 p, 1, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
            : "memory");
    }
}
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every UMMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ------------------------------------------------------------------ CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 0 and 1) drive one UMMA of M = 256: each holds 128 rows of A and N/2 rows of B
// in its own shared memory at the same offsets, each gets its 128 accumulator rows in its own tensor memory.
// Only the leader (rank 0) issues the UMMAs and waits on the "operands landed" barrier, which both CTAs' TMA
// loads complete; its commits then signal barriers in BOTH CTAs that the operands / the accumulator may be
// reused / read.  No load is multicast: every CTA fetches its own halves.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// global -> this CTA's shared memory; the bytes are counted on the mbarrier at `bar_cluster_addr`, which may
// belong to the peer CTA of the pair (the leader's "operands landed" barrier)
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *m, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const CUtensorMap *m, int x, int y, int z, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(void *smem_dst, const CUtensorMap *m, int x, int y, int z, int w,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the pair; issued by ONE thread of the leader CTA
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_f16_pair_imm(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    umma_f16_pair(d_tmem, a_desc, b_desc, idesc, ACC ? 1u : 0u);
}
// One arrival on the mbarrier at this offset in BOTH CTAs of the pair when every UMMA issued so far by this
// thread has completed (a commit is a signal, not a load: the operands are never multicast).  Two separate
// commits, one per CTA, work too but cost the pair kernels 10-40 % of their throughput.
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar_local_addr) {
    asm volatile(
        "{\n"
        ".reg .b16 m;\n"
        "mov.b16 m, 3;\n"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n"
        "}\n" ::"r"(bar_local_addr)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// The same without release semantics: for arrivals that order nothing but tensor-memory reuse (the reads have
// completed in the arriving thread), so the arrival need not wait for the thread's earlier global stores.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait on a barrier that CTAs of the cluster arrive on
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_w,
                                                  unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (*abort_w) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_w = 1;
                return false;
            }
        }
    }
    return true;
}

// ------------------------------------------------------------------ host: tensor maps
// 2-D/3-D row-major 16-bit tensors, box inner extent 64 elements (128 B) with the 128-byte swizzle.
int make_tensor_map_2d(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t row_pitch_elems,
                       uint32_t box_rows, uint32_t box_cols, bool swizzle128);
int make_tensor_map_3d(CUtensorMap *out, const void *base, uint64_t d2, uint64_t rows, uint64_t cols,
                       uint64_t row_pitch_elems, uint64_t d2_pitch_elems, uint32_t box_rows, uint32_t box_cols,
                       bool swizzle128);
// Dense (d2, rows, cols) tensor of 2- or 4-byte elements, box 1 x box_rows x box_cols whose rows are 32, 64
// or 128 bytes; swizzle span = the row size, so row r of the tile sits at r * row_bytes in shared memory
// with its 16-byte chunk index XOR-ed by address bits 7.. (the staging tiles of the step epilogue).
int make_tensor_map_3d_tile(CUtensorMap *out, const void *base, int elem_bytes, uint64_t d2, uint64_t rows, uint64_t cols,
                            uint32_t box_rows, uint32_t box_cols);
// A (steps, rows, width) 16-bit tensor seen as (steps, width/64, rows, 64): one box of
// 1 x chunks x box_rows x 64 lands in shared memory as `chunks` consecutive [box_rows x 128 B]
// swizzled K-major UMMA operand tiles, so one copy brings several 64-wide K chunks of a tile.
int make_tensor_map_chunked(CUtensorMap *out, const void *base, uint64_t steps, uint64_t rows, uint64_t width,
                            uint32_t box_rows, uint32_t chunks);

}  // namespace tc
}  // namespace flstm_b200
