// spg_tc.cuh -- raw PTX wrappers for the sm_100a asynchronous machinery (mbarrier, TMA bulk-tensor
// copies, tcgen05 MMA / tensor memory) shared by the tensor-core kernels.  Every wait is bounded.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace spgtc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Bounded wait on the phase with the given parity.  Once the abort flag is up every wait returns false at
// once; when the bound is hit the flag is raised and `code` recorded in *status.
// every try_wait may suspend the warp for up to this long; the iteration limits below count such attempts
#ifndef SPG_WAIT_HINT_NS
#define SPG_WAIT_HINT_NS 20000u
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status, int code,
                                          uint32_t limit = 1u << 16)
{
    {
        // the common case: the phase is already complete (one plain attempt, no abort check, no time hint)
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        // the time hint lets the hardware suspend the warp until the phase completes (or the time is up) instead of
        // spinning in the issue slots that the working warps of the same scheduler need
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(SPG_WAIT_HINT_NS) : "memory");
        if (ok) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}

// The same bounded wait for a role whose whole warp runs convergently (the TMA and MMA warps): the loop lives inside
// one asm block, so the compiler sees straight-line code and keeps warp-uniform values (descriptors, addresses,
// counters) in uniform registers -- tcgen05.mma and the bulk-tensor copies take their operands from there, and a value
// that has become "divergent" costs a register-to-uniform move per operand and instruction.  Nothing is returned:
// when the abort flag is up (or the bound is hit, which raises it and records `code`) the wait simply ends and the
// caller carries on; every later wait then ends at once, so the role runs out of its loops quickly.
__device__ __forceinline__ void mbar_wait_uniform(uint32_t bar, uint32_t parity, uint32_t abort_flag_smem, int32_t *status, int code,
                                                  uint32_t limit = 1u << 16)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .u32 n, a;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n\t"
        "@p bra SPG_WAIT_DONE;\n\t"
        "mov.u32 n, 0;\n\t"
        "ld.volatile.shared.u32 a, [%2];\n\t"
        "setp.ne.u32 q, a, 0;\n\t"
        "@q bra SPG_WAIT_DONE;\n\t"
        "SPG_WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1, %6;\n\t"
        "@p bra SPG_WAIT_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "and.b32 a, n, 15;\n\t"
        "setp.ne.u32 q, a, 0;\n\t"
        "@q bra SPG_WAIT_LOOP;\n\t"
        "ld.volatile.shared.u32 a, [%2];\n\t"
        "setp.ne.u32 q, a, 0;\n\t"
        "@q bra SPG_WAIT_DONE;\n\t"
        "setp.lt.u32 q, n, %5;\n\t"
        "@q bra SPG_WAIT_LOOP;\n\t"
        "st.volatile.shared.u32 [%2], 1;\n\t"
        "atom.global.cas.b32 a, [%3], 0, %4;\n\t"
        "SPG_WAIT_DONE:\n\t"
        "}"
        ::"r"(bar), "r"(parity), "r"(abort_flag_smem), "l"(status), "r"(code), "r"(limit), "r"(SPG_WAIT_HINT_NS) : "memory");
}

// The same for a barrier that the other CTA of a pair arrives on.  No thread reads what the other CTA's threads wrote:
// the waiter only issues tensor-core or bulk-copy work that reads each CTA's own shared memory through the async
// proxy, behind the writers' proxy fence and this barrier, so the default (CTA-scope) acquire is used, which measured
// 30 cycles cheaper per call than the cluster-scope form.  The first attempt is a plain try_wait (21 cycles when the
// phase is complete); the abort flag is only looked at every 16 failed attempts.
__device__ __forceinline__ void mbar_wait_uniform_cluster(uint32_t bar, uint32_t parity, uint32_t abort_flag_smem, int32_t *status, int code,
                                                          uint32_t limit = 1u << 16)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        ".reg .u32 n, a;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n\t"
        "@p bra SPG_WAITC_DONE;\n\t"
        "mov.u32 n, 0;\n\t"
        "SPG_WAITC_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1, %6;\n\t"
        "@p bra SPG_WAITC_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "and.b32 a, n, 15;\n\t"
        "setp.ne.u32 q, a, 0;\n\t"
        "@q bra SPG_WAITC_LOOP;\n\t"
        "ld.volatile.shared.u32 a, [%2];\n\t"
        "setp.ne.u32 q, a, 0;\n\t"
        "@q bra SPG_WAITC_DONE;\n\t"
        "setp.lt.u32 q, n, %5;\n\t"
        "@q bra SPG_WAITC_LOOP;\n\t"
        "st.volatile.shared.u32 [%2], 1;\n\t"
        "atom.global.cas.b32 a, [%3], 0, %4;\n\t"
        "SPG_WAITC_DONE:\n\t"
        "}"
        ::"r"(bar), "r"(parity), "r"(abort_flag_smem), "l"(status), "r"(code), "r"(limit), "r"(SPG_WAIT_HINT_NS) : "memory");
}

// one lane of a convergent warp (the same lane every time)
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// untiled bulk copy global -> this CTA's shared memory, completing on an mbarrier (16-byte aligned addresses and size)
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap *map) { asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory"); }

// generic-proxy shared-memory writes -> visible to the async proxy (TMA / tensor core reads)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f16 (fp16/bf16 operands, fp32 accumulate), one CTA.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// mbarrier arrives once all tcgen05 operations issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart, tile base
// 1024-byte aligned.  Advancing K by 16 elements inside the tile adds 32 bytes (+2 in the address field).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1u << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1u << 46;
    d |= (uint64_t)2u << 61;
    return d;
}
// instruction descriptor: fp32 accumulator, A/B formats (0 = f16, 1 = bf16), both K-major, M = 128, N = n
__host__ __device__ inline uint32_t idesc_f16(uint32_t a_fmt, uint32_t b_fmt, uint32_t n)
{
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// ---- CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) -----------------------------------------------------
// One MMA instruction, issued by the pair's first CTA, multiplies a 256-row tile: each CTA's shared memory holds its own
// 128 rows of A and its half of B's rows (N/2), and each CTA's tensor memory receives its own 128 rows of the accumulator.
// Per CTA that halves the B bytes that have to be streamed and kept in shared memory.

__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same location in the shared memory of CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// arrive on a barrier that may live in the other CTA of the cluster (address from mapa).  Default semantics (release at
// CTA scope): the arriving warp's shared-memory writes are in its own CTA's shared memory, fenced for the async proxy,
// before the arrive leaves; the waiter reads them only through tensor-core instructions.  The cluster-scope release
// measured 1300 cycles per arrive in this kernel, the default form 60.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// all threads of both CTAs
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// the barrier at the same shared-memory offset in BOTH CTAs of the pair arrives once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// Tile load into THIS CTA's shared memory whose completion is counted on a barrier of the pair's first CTA (no multicast:
// each CTA fetches its own tile).  `leader_bar` is a shared::cluster address (mapa(bar, 0)).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t leader_bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
// instruction descriptor of the pair MMA: M = 256 over the two CTAs
__host__ __device__ inline uint32_t idesc_f16_pair(uint32_t a_fmt, uint32_t b_fmt, uint32_t n)
{
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

}  // namespace spgtc
