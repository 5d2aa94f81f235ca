// PTX wrappers shared by the kernels that use the 5th-generation tensor cores:
// mbarriers with bounded waits, TMA tile loads, tcgen05 products, commits, tensor
// memory loads and stores, and the shared-memory operand descriptors.
#pragma once
#include "common.cuh"
#include <cuda.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_NS 2000000000ull        // a wait gives up after two seconds
// which kernel family a give-up is reported for: the including file defines it (1: products,
// 2: prefill attention); the status word holds (family << 8) | place of the wait
#ifndef TC_FAMILY
#define TC_FAMILY 0
#endif

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait; false if it gave up (or another role already did).  The bound is in time: a
// try_wait may itself block for a while, so counting polls would bound nothing.
__device__ __forceinline__ unsigned long long tc_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, int where,
                                          unsigned long long limit_ns = TC_WAIT_NS) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = tc_now_ns();
    for (unsigned it = 1;; ++it) {
        if (mbar_try(bar, parity)) return true;
        // the flag and the clock are looked at every few polls only: each look at the flag is a read of
        // shared memory, and a block's waiting threads would otherwise fill the pipe that the tensor
        // cores read their operands through
        if ((it & 7) == 0 && *abort_flag) return false;
        if ((it & 63) == 0 && tc_now_ns() - t0 > limit_ns) break;
    }
    *abort_flag = where;
    zlm_report_status((TC_FAMILY << 8) | where);
    return false;
}
// the same for a whole warp: one lane polls, all lanes get the answer (and, through the warp's
// barrier, see what the arriving threads wrote before)
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, unsigned parity, volatile int* abort_flag, int where) {
    int ok = 0;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, where) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}
// after a wait gave up: lets copies that are still in flight land (at most 10 ms each)
__device__ __forceinline__ void mbar_drain(uint64_t* bar, unsigned parity) {
    const unsigned long long t0 = tc_now_ns();
    while (!mbar_try(bar, parity) && tc_now_ns() - t0 < 10000000ull) {}
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 columns of this thread's lane, without the wait: several loads can be in flight, then tc_wait_ld()
__device__ __forceinline__ void tc_ld16_nowait(unsigned taddr, float* v) {
    unsigned* r = (unsigned*)v;
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(unsigned taddr, float* v) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// shared-memory operand descriptor: K-major tile whose rows are 128 bytes, 128-byte
// swizzle; 8-row groups are 1024 bytes apart.  Fields in units of 16 bytes.
__device__ __forceinline__ uint64_t make_desc(unsigned smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);     // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                          // 128-byte swizzle
    return d;
}


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_st16(unsigned taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// generic-proxy writes to shared memory become visible to the tensor cores' (async proxy) reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// operand descriptor with explicit leading / stride byte offsets (in bytes), 128-byte swizzle
__device__ __forceinline__ uint64_t make_desc_ex(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// ---------------------------------------------------------------- a pair of blocks on one tile
// Two blocks of a cluster (ranks 0 and 1) work on one tile: each loads its half of both operands,
// rank 0 issues products that read both halves and write both blocks' tensor memory.
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// every thread of both blocks
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the address, in the cluster's window, of block `rank`'s copy of a shared-memory object
__device__ __forceinline__ unsigned cluster_addr(const void* p, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
// tile load into this block's shared memory whose bytes count at rank 0's mbarrier
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, unsigned bar_rank0) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_rank0) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the products issued so far have retired, at the mbarrier at this place in both blocks
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_at(unsigned cluster_address) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_address) : "memory");
}
// bounded wait on a barrier at which the other block of the pair arrives too
__device__ __forceinline__ bool mbar_try_pair(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_pair(uint64_t* bar, unsigned parity, volatile int* abort_flag, int where) {
    if (mbar_try_pair(bar, parity)) return true;
    const unsigned long long t0 = tc_now_ns();
    for (unsigned it = 1;; ++it) {
        if (mbar_try_pair(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 63) == 0 && tc_now_ns() - t0 > TC_WAIT_NS) break;
    }
    *abort_flag = where;
    zlm_report_status((TC_FAMILY << 8) | where);
    return false;
}

typedef CUresult (*ZlmEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
ZlmEncodeTiledFn zlm_tensor_map_encoder();
// 2-D bf16 tensor map: `rows` rows of `cols` elements, row stride `ld` elements; box = box_rows x box_cols
// (box_cols * 2 bytes = 128: the swizzle span), zero fill outside
int zlm_make_map_2d(CUtensorMap* m, const void* ptr, long long rows, int cols, long long ld, int box_rows, int box_cols);
