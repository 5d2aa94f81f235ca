// bf16 matrix product Y[T,N] = X[T,K] . W[N,K]^T for prefill-sized T on the
// 5th-generation tensor cores: operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), products issued by one thread with
// tcgen05.mma (128 x 256 x 16 per instruction), fp32 accumulators in tensor
// memory, read back with tcgen05.ld for the epilogue.
//
// Three forms, by the number of tokens T:
//  * many tokens (from 385): persistent, a cluster of two blocks per 256-token x BN-output
//    tile (tcgen05 with cta_group::2, gemm_tc_pair_kernel); the single-block persistent kernel
//    with 128 x BN tiles stays selectable (gemm_tc_persistent_kernel);
//  * few tokens (17 to 384): the operands swap places, 128 rows of W against a tile of 32, 64
//    or 128 tokens, so that W, which is what the step has to read, still streams through
//    full-height products; one block per tile and share of K where that is one round of the
//    GPU (gemm_tc_kernel), else persistent blocks (gemm_tc_few_kernel); K is cut into shares
//    where the tiles alone would not fill the SMs, and a second kernel adds the shares in a
//    fixed order.
// In all of them warp 0 is the TMA producer, warp 1 allocates tensor memory and issues the
// products, warps 2..5 are the epilogue.  A ring of (first-operand tile 128x64,
// second-operand tile x64) is handed back and forth with mbarriers: `full` is completed by
// the TMA's byte count, `empty` by tcgen05.commit when the products that read a stage have
// retired.
//
// Every wait is bounded: a wait that does not come true leaves its mark in the library's
// status word (zlm_status, in pinned host memory) and makes every role leave its loop; the
// block then waits, again bounded, for copies still in flight, frees its tensor
// memory and returns.
//
// out_i = sum_j W[i,j] x_j with bf16 operands and fp32 accumulation
// (src/kernels/linear/matvec/kernels/bfloat.zig:43-67; the reference's batched
// product: src/kernels/linear/matmul/root.zig:62-81).
#define TC_FAMILY 1
#include "tc_common.cuh"

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// a thread's 16 consecutive outputs (columns n .. n+15) of token `row` in the wanted mode
template <int MODE>
__device__ __forceinline__ void store_row16(const float* v, void* Y, int row, int n, int T, int N, int ldy) {
    if (row >= T || n >= N) return;
    const bool whole = n + 16 <= N;
#ifdef ZLM_BOUNDS_CHECK
    {
        const int cols = whole ? 16 : N - n;
        const bool ok = MODE == 3 ? ZLM_CHK((__nv_bfloat16*)Y + (size_t)row * ldy + n / 2, 16)
                      : MODE == 0 ? ZLM_CHK((__nv_bfloat16*)Y + (size_t)row * ldy + n, cols * 2)
                                  : ZLM_CHK((float*)Y + (size_t)row * ldy + n, cols * 4);
        if (!ok) return;
    }
#endif
    __nv_bfloat162 t;
#define ZLM_PK(a, b) (t = __floats2bfloat162_rn(a, b), *(unsigned*)&t)
    if (MODE == 3) {
        __nv_bfloat16* y = (__nv_bfloat16*)Y + (size_t)row * ldy + n / 2;
        if (whole && ((uintptr_t)y & 15) == 0) {
            uint4 p;
            p.x = ZLM_PK(silu_mul(v[0], v[8]), silu_mul(v[1], v[9]));
            p.y = ZLM_PK(silu_mul(v[2], v[10]), silu_mul(v[3], v[11]));
            p.z = ZLM_PK(silu_mul(v[4], v[12]), silu_mul(v[5], v[13]));
            p.w = ZLM_PK(silu_mul(v[6], v[14]), silu_mul(v[7], v[15]));
            *(uint4*)y = p;
        } else if (whole) {
            for (int i = 0; i < 8; ++i) y[i] = __float2bfloat16_rn(silu_mul(v[i], v[8 + i]));
        }
    } else if (MODE == 0) {
        __nv_bfloat16* y = (__nv_bfloat16*)Y + (size_t)row * ldy + n;
        if (whole && ((uintptr_t)y & 15) == 0) {
            uint4 p0, p1;
            p0.x = ZLM_PK(v[0], v[1]); p0.y = ZLM_PK(v[2], v[3]); p0.z = ZLM_PK(v[4], v[5]); p0.w = ZLM_PK(v[6], v[7]);
            p1.x = ZLM_PK(v[8], v[9]); p1.y = ZLM_PK(v[10], v[11]); p1.z = ZLM_PK(v[12], v[13]); p1.w = ZLM_PK(v[14], v[15]);
            *(uint4*)y = p0;
            *(uint4*)(y + 8) = p1;
        } else {
            for (int i = 0; i < 16 && n + i < N; ++i) y[i] = __float2bfloat16_rn(v[i]);
        }
    } else {
        float* y = (float*)Y + (size_t)row * ldy + n;
        if (whole && ((uintptr_t)y & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (MODE == 1) {
                    const float4 old = *(const float4*)(y + i);
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *(float4*)(y + i) = o;
            }
        } else {
            for (int i = 0; i < 16 && n + i < N; ++i) y[i] = MODE == 1 ? y[i] + v[i] : v[i];
        }
    }
#undef ZLM_PK
}

// this thread's output `row`, tokens t0 .. t0+15, in the wanted mode; every lane of the warp calls it
template <int MODE>
__device__ __forceinline__ void store_swapped16(const float* v, void* Y, int row, int t0, int T, int N, int ldy, int lane) {
    if (MODE == 3) {
        // lanes 0-7 and 16-23 hold gate channels, lanes 8-15 and 24-31 the matching up
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float u = __shfl_down_sync(0xffffffffu, v[i], 8);
            if ((lane & 8) == 0 && row < N && t0 + i < T) {
                const int ch = (row >> 4) * 8 + (row & 7);
                if (!ZLM_CHK((__nv_bfloat16*)Y + (size_t)(t0 + i) * ldy + ch, 2)) continue;
                ((__nv_bfloat16*)Y)[(size_t)(t0 + i) * ldy + ch] = __float2bfloat16_rn(silu_mul(v[i], u));
            }
        }
        return;
    }
    if (row >= N) return;
#ifdef ZLM_BOUNDS_CHECK
    for (int i = 0; i < 16 && t0 + i < T; ++i)
        if (!ZLM_CHK((char*)Y + ((size_t)(t0 + i) * ldy + row) * (MODE == 0 ? 2 : 4), MODE == 0 ? 2 : 4)) return;
#endif
    if (MODE == 1) {
        float old[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) old[i] = t0 + i < T ? __ldcg((const float*)Y + (size_t)(t0 + i) * ldy + row) : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (t0 + i < T) ((float*)Y)[(size_t)(t0 + i) * ldy + row] = old[i] + v[i];
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (t0 + i >= T) break;
            const size_t off = (size_t)(t0 + i) * ldy + row;
            if (MODE == 0) ((__nv_bfloat16*)Y)[off] = __float2bfloat16_rn(v[i]);
            else ((float*)Y)[off] = v[i];
        }
    }
}

// MODE 0: Y bf16 = acc; MODE 1: Y fp32 += acc; MODE 2: Y fp32 = acc;
// MODE 3: the outputs come in groups of 16 = 8 gate + 8 up channels; Y bf16 [T, N/2] = silu(gate) * up;
// MODE 4: the block sums its share of K (blockIdx.z of gridDim.z) and stores the fp32 partial
// product to Y [gridDim.z][T][N]; zlm_gemm_tc adds the shares up in a second kernel.
// The few-token form as stand-alone blocks: the first operand is W (128 outputs), the second X
// (a tile of BN tokens); one block per tile and share of K.
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               void* __restrict__ Y, int T, int N, int K, int ldy) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(sB + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    unsigned* tmem_slot = (unsigned*)(acc_full + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0row = blockIdx.x * TC_BM, b0row = blockIdx.y * BN;
    const int KB_all = (K + TC_BK - 1) / TC_BK;
    // this block's share of the k blocks (all of them unless the grid splits K)
    const int kb_per = (KB_all + gridDim.z - 1) / gridDim.z;
    const int kb_lo = blockIdx.z * kb_per;
    const int KB = max(0, min(KB_all, kb_lo + kb_per) - kb_lo);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"((unsigned)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_launch_dependents();
    // Set-up above overlaps the kernel before.  So do the first loads of W, which no kernel of the
    // step writes: the ring's stages are all free at the start, and the producer fills them with W
    // before it waits for the kernel before, with the activations after.  Everybody else waits here;
    // operands from other kernels and Y are touched after the wait only.
    const int early = min(KB, STAGES);
    if (warp == 0 && lane == 0) {
        for (int kb = 0; kb < early; ++kb) {
            mbar_expect_tx(&full[kb], A_BYTES + B_BYTES);
            tma_load_2d(sA + kb * A_BYTES, &map_a, (kb_lo + kb) * TC_BK, a0row, &full[kb]);
        }
    }
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int issued = early;
            for (int kb = 0; kb < early; ++kb)
                tma_load_2d(sB + kb * B_BYTES, &map_b, (kb_lo + kb) * TC_BK, b0row, &full[kb]);
            for (int kb = early; kb < KB; ++kb) {
                const int s = kb % STAGES;
                const unsigned round = kb / STAGES;
                if (!mbar_wait(&empty[s], (round & 1) ^ 1, abort_flag, 1)) break;
                mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                tma_load_2d(sA + s * A_BYTES, &map_a, (kb_lo + kb) * TC_BK, a0row, &full[s]);
                tma_load_2d(sB + s * B_BYTES, &map_b, (kb_lo + kb) * TC_BK, b0row, &full[s]);
                issued = kb + 1;
            }
            if (*abort_flag) {
                // copies may still be landing in this block's shared memory: wait for them (bounded)
                for (int kb = max(0, issued - STAGES); kb < issued; ++kb)
                    mbar_drain(&full[kb % STAGES], (kb / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N = BN, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                   ((unsigned)(TC_BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < KB && ok; ++kb) {
                const int s = kb % STAGES;
                const unsigned round = kb / STAGES;
                ok = mbar_wait(&full[s], round & 1, abort_flag, 2);
                if (!ok) break;
                tc_fence_after();
                // one descriptor per stage, advanced by constants (the start address field counts
                // 16-byte units and does not carry): the issuing thread has no instruction to spare
                const uint64_t ad = make_desc(smem_u32(sA + s * A_BYTES)), bd = make_desc(smem_u32(sB + s * B_BYTES));
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    tc_mma(tmem_base, ad + ((k * 32) >> 4), bd + ((k * 32) >> 4), idesc, (kb | k) != 0);
                tc_commit(&empty[s]);          // the stage is free once these products have read it
            }
            tc_commit(acc_full);               // arrives when every product issued so far has retired
        }
    } else {
        // epilogue: warp w may touch tensor-memory lanes 32 (w % 4) .. + 31; a lane is a row of the tile
        const int lg = warp & 3;
        const bool ok = mbar_wait_warp(acc_full, 0, abort_flag, 3);
        tc_fence_after();
        const int arow = a0row + lg * 32 + lane;
        if (ok && !*abort_flag) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                tc_ld16(tmem_base + ((unsigned)(lg * 32) << 16) + (unsigned)c, v);     // warp-wide
                if (KB == 0) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;     // a share of K with nothing in it
                }
                // this thread: output arow, tokens b0row + c .. + 15; a warp's lanes are 32
                // neighbouring outputs, so every token's store is one coalesced line
                const int t0 = b0row + c;
                if constexpr (MODE == 4) {
                    if (arow < N) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (t0 + i < T && ZLM_CHK((float*)Y + ((size_t)blockIdx.z * T + t0 + i) * N + arow, 4))
                                ((float*)Y)[((size_t)blockIdx.z * T + t0 + i) * N + arow] = v[i];
                    }
                } else {
                    store_swapped16<MODE>(v, Y, arow, t0, T, N, ldy, lane);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((unsigned)BN) : "memory");
    }
}

// ---------------------------------------------------------------------------
// The many-token form as a persistent kernel: one block per SM walks the 128 x 256
// tiles of Y (token tiles fastest, so that blocks that run together share a tile of
// W).  Tensor memory holds two accumulators; while the epilogue warps drain one,
// the product warp already fills the other, and the TMA ring never stops between
// tiles.  acc_full[b] / acc_empty[b] hand accumulator b back and forth.
// ---------------------------------------------------------------------------
// The order in which the persistent kernels walk the tiles of Y: token tiles fastest, so that the
// blocks that run together share a tile of W; but in groups of `gm` token tiles, all output tiles
// of a group before the next group, so that a group's activations (gm x BM x K) stay in L2 while
// its output tiles are walked.  Without the groups a step of 65,000 tokens re-reads its 534 MB of
// activations from DRAM for every output tile.
__device__ __forceinline__ void tile_of(int tile, int m_tiles, int n_tiles, int gm, int& m, int& n) {
    const int per_group = gm * n_tiles;
    const int group = tile / per_group, r = tile - group * per_group;
    const int m0 = group * gm, gm_here = min(gm, m_tiles - m0);
    n = r / gm_here;
    m = m0 + r - n * gm_here;
}
// token tiles per group: the group's activations take about 64 MB of the 126 MB L2
static int tile_group(int bm, int K) {
    const long long bytes = (long long)bm * K * 2;
    const long long g = (64ll << 20) / (bytes > 0 ? bytes : 1);
    return (int)(g < 4 ? 4 : g);
}

#define TCP_ACC 256          // tensor-memory columns between the two accumulators (an allocation is a power of two)
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          void* __restrict__ Y, int T, int N, int K, int ldy, int gm) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(sB + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    unsigned* tmem_slot = (unsigned*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (T + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"((unsigned)(2 * TCP_ACC)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;            // k blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                int tm, tn;
                tile_of(tile, m_tiles, n_tiles, gm, tm, tn);
                const int a0row = tm * TC_BM, b0row = tn * BN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                    tma_load_2d(sA + s * A_BYTES, &map_a, kb * TC_BK, a0row, &full[s]);
                    tma_load_2d(sB + s * B_BYTES, &map_b, kb * TC_BK, b0row, &full[s]);
                }
            }
            if (*abort_flag) {
                // copies may still be landing in this block's shared memory: wait for them (bounded)
                for (unsigned j = it > (unsigned)STAGES ? it - STAGES : 0; j < it; ++j)
                    mbar_drain(&full[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                   ((unsigned)(TC_BM >> 4) << 24);
            unsigned it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
                const unsigned buf = local & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag, 4);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t ad = make_desc(smem_u32(sA + s * A_BYTES)), bd = make_desc(smem_u32(sB + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma(tmem_base + buf * TCP_ACC, ad + ((k * 32) >> 4), bd + ((k * 32) >> 4), idesc, (kb | k) != 0);
                    tc_commit(&empty[s]);
                }
                tc_commit(&acc_full[buf]);
            }
            if (!ok) { tc_commit(&acc_full[0]); tc_commit(&acc_full[1]); }     // let the epilogue out
        }
    } else {
        const int lg = warp & 3;
        unsigned local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const unsigned buf = local & 1;
            int tm, tn;
            tile_of(tile, m_tiles, n_tiles, gm, tm, tn);
            const int a0row = tm * TC_BM, b0row = tn * BN;
            const bool ok = mbar_wait_warp(&acc_full[buf], (local >> 1) & 1, abort_flag, 3);
            tc_fence_after();
            if (!ok || *abort_flag) break;
            const int arow = a0row + lg * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                tc_ld16(tmem_base + ((unsigned)(lg * 32) << 16) + buf * TCP_ACC + (unsigned)c, v);
                store_row16<MODE>(v, Y, arow, b0row + c, T, N, ldy);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);      // one arrival per epilogue warp
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((unsigned)(2 * TCP_ACC)) : "memory");
    }
}

// ---------------------------------------------------------------------------
// MODE 5: the q/k/v projection with what follows it folded into the epilogue: per-head
// RMSNorm of q and k, the rotation of q and k by the token's position, and the write of k
// and v into the paged cache; only q goes to Y.  The separate pass over the projection's
// output (read 25 MB, write 25 MB per layer at 2,048 tokens) disappears, and the norm sees
// the fp32 sums instead of their bf16 roundings.  An epilogue thread owns one token row of
// the tile and walks its columns, so a head (head_dim columns, a divisor of the tile's
// width) is all in one thread: the sum of squares is a first walk over the head's tensor
// memory columns, the second walk norms, rotates the halves against each other (columns c
// and c + head_dim/2 of the same thread) and stores.  cos and sin come from a table
// [2][head_dim/2][T] that is computed once per step for all layers (zlm_rope_table).
// Order and arithmetic as the stand-alone kernel (rope_kv.cuh): norm, then rotation, then
// the cache write; v as it is (src/architectures/impl/qwen3/block.zig:26-30,
// src/kernels/transformer/norm.zig:128-166, src/kernels/transformer/rope.zig:161-206).
// ---------------------------------------------------------------------------
struct QkvEpilogue {
    const void* q_w;            // [hd] norm weights (null: no norm)
    const void* k_w;
    int w_dtype;
    float eps;
    const float* cos_sin;       // [2][hd/2][T] (null: no rotation)
    const int* token_pos;       // [T]
    const int* token_slot;      // [T]
    const int* block_table;
    int table_stride;
    __nv_bfloat16* pool;        // [pages][2][nkv][ZLM_PAGE][hd]
    int nq, nkv, hd;
};

__device__ __forceinline__ void qkv_store16(__nv_bfloat16* dst, const float* v) {
    if (!ZLM_CHK(dst, 32)) return;
    __nv_bfloat162 t;
    uint4 a, b;
#define ZLM_PK2(x, y) (t = __floats2bfloat162_rn(x, y), *(unsigned*)&t)
    a.x = ZLM_PK2(v[0], v[1]); a.y = ZLM_PK2(v[2], v[3]); a.z = ZLM_PK2(v[4], v[5]); a.w = ZLM_PK2(v[6], v[7]);
    b.x = ZLM_PK2(v[8], v[9]); b.y = ZLM_PK2(v[10], v[11]); b.z = ZLM_PK2(v[12], v[13]); b.w = ZLM_PK2(v[14], v[15]);
#undef ZLM_PK2
    *(uint4*)dst = a;
    *(uint4*)(dst + 8) = b;
}

// one token row (this thread's lane of tensor memory at `taddr`, tile columns [n0, n0 + BN))
template <int BN>
__device__ __forceinline__ void qkv_epilogue_row(const QkvEpilogue& ep, unsigned taddr, __nv_bfloat16* Y, int row, int n0,
                                                 int T, int N, int ldy) {
    const int hd = ep.hd, half = hd >> 1;
    int pos = 0, page = 0;
    // a row beyond the step's tokens (or, in the bounds-check build, one whose integers lie outside
    // the tensors passed) still walks tensor memory with its warp, and stores nothing
    bool live = row < T && ZLM_CHK(ep.token_pos + row, 4);
    if (live) {
        pos = ep.token_pos[row];
        if (ep.nkv > 0) {
            live = ZLM_CHK(ep.token_slot + row, 4);
            if (live) {
                const int* entry = ep.block_table + (size_t)ep.token_slot[row] * ep.table_stride + pos / ZLM_PAGE;
                live = ZLM_CHK(entry, 4);
                if (live) page = *entry;
            }
        }
    }
    const VecW qw{ep.q_w, ep.w_dtype}, kw{ep.k_w, ep.w_dtype};
    // the table is [2][hd/2][T]: the warp's 32 rows read 32 neighbouring floats of one angle
    const float* cs_row = ep.cos_sin ? ep.cos_sin + min(row, T - 1) : nullptr;
    const float* sn_row = ep.cos_sin ? ep.cos_sin + (size_t)half * T + min(row, T - 1) : nullptr;
    for (int c0 = 0; c0 < BN; c0 += hd) {                 // the tile's heads; warp-uniform
        const int n = n0 + c0;
        if (n >= N) break;
        const int j = n / hd;                             // head among q heads, then k heads, then v heads
        const int kind = j < ep.nq ? 0 : (j < ep.nq + ep.nkv ? 1 : 2);
        __nv_bfloat16* dst;
        if (kind == 0) {
            dst = Y + (size_t)row * ldy + n;
        } else {
            const int kvh = kind == 1 ? j - ep.nq : j - ep.nq - ep.nkv;
            dst = ep.pool + ((((size_t)page * 2 + (kind - 1)) * ep.nkv + kvh) * ZLM_PAGE + (pos % ZLM_PAGE)) * hd;
        }
        if (kind == 2) {
#pragma unroll 1
            for (int c = 0; c < hd; c += 16) {
                float v[16];
                tc_ld16(taddr + (unsigned)(c0 + c), v);
                if (live) qkv_store16(dst + c, v);
            }
            continue;
        }
        const VecW& w = kind == 0 ? qw : kw;
        float inv = 1.f;
        if (w.p) {
            float ss = 0.f;
#pragma unroll 1
            for (int c = 0; c < hd; c += 16) {
                float v[16];
                tc_ld16(taddr + (unsigned)(c0 + c), v);
#pragma unroll
                for (int i = 0; i < 16; ++i) ss = fmaf(v[i], v[i], ss);
            }
            inv = 1.0f / sqrtf(ss / (float)hd + ep.eps);
        }
#pragma unroll 1
        for (int c = 0; c < half; c += 16) {
            float lo[16], hi[16];
            tc_ld16_nowait(taddr + (unsigned)(c0 + c), lo);
            tc_ld16_nowait(taddr + (unsigned)(c0 + half + c), hi);
            tc_wait_ld();
            if (w.p) {
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const float4 wl = w.load4(c + i), wh = w.load4(half + c + i);
                    lo[i] = (lo[i] * inv) * wl.x; lo[i + 1] = (lo[i + 1] * inv) * wl.y;
                    lo[i + 2] = (lo[i + 2] * inv) * wl.z; lo[i + 3] = (lo[i + 3] * inv) * wl.w;
                    hi[i] = (hi[i] * inv) * wh.x; hi[i + 1] = (hi[i + 1] * inv) * wh.y;
                    hi[i + 2] = (hi[i + 2] * inv) * wh.z; hi[i + 3] = (hi[i + 3] * inv) * wh.w;
                }
            }
            if (cs_row && live) {
                float cc[16], sn[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    cc[e] = __ldg(cs_row + (size_t)(c + e) * T);
                    sn[e] = __ldg(sn_row + (size_t)(c + e) * T);
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float x0 = lo[e], x1 = hi[e];
                    lo[e] = x0 * cc[e] - x1 * sn[e];
                    hi[e] = x0 * sn[e] + x1 * cc[e];
                }
            }
            if (live) {
                qkv_store16(dst + c, lo);
                qkv_store16(dst + half + c, hi);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// The persistent kernel on pairs of blocks (tcgen05 with cta_group::2): a cluster of two
// blocks, on neighbouring SMs, walks tiles of 256 tokens x BN outputs.  Each block loads its
// 128 tokens and its half of the BN rows of W; rank 0 issues 256 x BN x 16 products that read
// both blocks' shared memory and accumulate into both blocks' tensor memory (each holds the
// 128 rows of its own tokens).  Per product a block reads 128 x 16 of W instead of 256 x 16:
// the single-block kernel's shared-memory pipe (operand reads plus TMA writes at the pipe's
// 128 bytes a cycle) is what this relieves.  Barriers: full[s] lives in rank 0 and counts
// the bytes of both blocks' loads; empty[s], acc_full[b] exist in both blocks and are
// signalled by multicast commits; acc_empty[b] lives in rank 0 and is arrived at by the
// epilogue warps of both blocks.
// ---------------------------------------------------------------------------
#define TCQ_BM 256
// The epilogue hands its results to the copy engine: a warp puts 32 rows x 64 bytes of output
// into shared memory (TCQ_RING such boxes of its own, in the 64-byte swizzle, which keeps the
// row-per-thread 16-byte writes free of bank conflicts) and one bulk store of the box writes
// them; where the product adds into the fp32 stream, one reduce-add of the box
// (cp.reduce.async.bulk.tensor, .add on f32) does the read-modify-write in L2.  The
// row-per-thread loads and stores that this replaces touched 32 rows per instruction, 32
// memory transactions each: 20 us for the fp32 stream's tile of 256 x 240, as long as the
// tile's products at K = 4,096 and all of it exposed after a block's last tile.  The copy
// engine clips a box at the matrix's edges.  TCQ_BOX_ACC: accumulator columns that make a box.
#define TCQ_RING 4
#define TCQ_BOX_BYTES (32 * 64)
#define TCQ_BOX_ACC(MODE) ((MODE) == 3 ? 64 : (MODE) == 0 ? 32 : 16)
#define TCQ_OUT_BYTES (4 * TCQ_RING * TCQ_BOX_BYTES)
template <int BN, int STAGES, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_y, void* __restrict__ Y, int T, int N, int K, int ldy, int gm,
                    int y_tma, const QkvEpilogue ep) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = (BN / 2) * TC_BK * 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * A_BYTES;
    unsigned char* sOut = sB + STAGES * B_BYTES;          // 1024-aligned: every stage is a multiple of 1 KB
    uint64_t* full = (uint64_t*)(sOut + TCQ_OUT_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    unsigned* tmem_slot = (unsigned*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int KB = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (T + TCQ_BM - 1) / TCQ_BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"((unsigned)(2 * TCP_ACC)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the other block's barriers are initialised before anything arrives there
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_launch_dependents();
    // The first tile's first loads of W (which no kernel of the step writes) go out before the wait
    // for the kernel before: the ring's stages are all free at the start.  The tokens of those
    // stages follow after the wait, and nothing else of another kernel's is touched before it.
    int early = 0;
    if (warp == 0 && lane == 0 && pair < tiles) {
        int tm, tn;
        tile_of(pair, m_tiles, n_tiles, gm, tm, tn);
        const int b0row = tn * BN + rank * (BN / 2);
        early = min(KB, STAGES);
        for (int kb = 0; kb < early; ++kb) {
            if (rank == 0) mbar_expect_tx(&full[kb], 2 * (A_BYTES + B_BYTES));
            tma_load_2d_pair(sB + kb * B_BYTES, &map_b, kb * TC_BK, b0row, cluster_addr(&full[kb], 0));
        }
    }
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs) {
                int tm, tn;
                tile_of(tile, m_tiles, n_tiles, gm, tm, tn);
                const int a0row = tm * TCQ_BM + rank * TC_BM;
                const int b0row = tn * BN + rank * (BN / 2);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    const unsigned bar0 = cluster_addr(&full[s], 0);
                    if ((int)it < early) {      // the stage's W is on its way already
                        tma_load_2d_pair(sA + s * A_BYTES, &map_a, kb * TC_BK, a0row, bar0);
                        continue;
                    }
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, 1)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
                    tma_load_2d_pair(sA + s * A_BYTES, &map_a, kb * TC_BK, a0row, bar0);
                    tma_load_2d_pair(sB + s * B_BYTES, &map_b, kb * TC_BK, b0row, bar0);
                }
            }
            if (*abort_flag && rank == 0) {
                for (unsigned j = it > (unsigned)STAGES ? it - STAGES : 0; j < it; ++j)
                    mbar_drain(&full[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // fp32 accumulate, bf16 x bf16, both K-major, N = BN, M = 256 over the two blocks
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                   ((unsigned)(TCQ_BM >> 4) << 24);
            unsigned it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
                const unsigned buf = local & 1;
                ok = mbar_wait_pair(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag, 4);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t ad = make_desc(smem_u32(sA + s * A_BYTES)), bd = make_desc(smem_u32(sB + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma_pair(tmem_base + buf * TCP_ACC, ad + ((k * 32) >> 4), bd + ((k * 32) >> 4), idesc, (kb | k) != 0);
                    tc_commit_pair(&empty[s]);
                }
                tc_commit_pair(&acc_full[buf]);
            }
            if (!ok) { tc_commit_pair(&acc_full[0]); tc_commit_pair(&acc_full[1]); }     // let the epilogues out
        }
    } else {
        const int lg = warp & 3;
        unsigned local = 0, boxes = 0;
        const unsigned empty0[2] = {cluster_addr(&acc_empty[0], 0), cluster_addr(&acc_empty[1], 0)};
        for (int tile = pair; tile < tiles; tile += pairs, ++local) {
            const unsigned buf = local & 1;
            int tm, tn;
            tile_of(tile, m_tiles, n_tiles, gm, tm, tn);
            const int a0row = tm * TCQ_BM + rank * TC_BM, b0row = tn * BN;
            const bool ok = mbar_wait_warp(&acc_full[buf], (local >> 1) & 1, abort_flag, 3);
            tc_fence_after();
            if (!ok || *abort_flag) break;
            const int arow = a0row + lg * 32 + lane;
            if constexpr (MODE == 5) {
                qkv_epilogue_row<BN>(ep, tmem_base + ((unsigned)(lg * 32) << 16) + buf * TCP_ACC, (__nv_bfloat16*)Y, arow,
                                     b0row, T, N, ldy);
            } else if (y_tma && BN % TCQ_BOX_ACC(MODE) == 0) {
                // a box is 32 rows x 64 bytes of output: 16 fp32 sums, 32 bf16 values, or the 32 bf16
                // results of 64 gate/up sums; a thread writes its row's four 16-byte pieces
                constexpr int ACC = TCQ_BOX_ACC(MODE);
                const unsigned taddr = tmem_base + ((unsigned)(lg * 32) << 16) + buf * TCP_ACC;
                unsigned char* const ring = sOut + lg * (TCQ_RING * TCQ_BOX_BYTES);
                const int n_out = MODE == 3 ? N / 2 : N;
#pragma unroll 1
                for (int c = 0; c < BN; c += ACC, ++boxes) {
                    const int x = MODE == 3 ? (b0row + c) / 2 : b0row + c;
                    if (x >= n_out || a0row + lg * 32 >= T) break;     // nothing of this box lies inside (warp-uniform)
                    // the box about to be overwritten was handed over TCQ_RING boxes ago: wait until
                    // the copy engine has read it (the later ones may still be on their way)
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(TCQ_RING - 1) : "memory");
                    __syncwarp();
                    unsigned char* const row = ring + (boxes % TCQ_RING) * TCQ_BOX_BYTES + lane * 64;
                    const int sw = (lane >> 1) & 3;
                    __nv_bfloat162 t;
#define ZLM_PK(a, b) (t = __floats2bfloat162_rn(a, b), *(unsigned*)&t)
#pragma unroll
                    for (int part = 0; part < ACC / 16; ++part) {
                        float v[16];
                        tc_ld16(taddr + (unsigned)(c + part * 16), v);
                        if (MODE == 3) {
                            uint4 pk;
                            pk.x = ZLM_PK(silu_mul(v[0], v[8]), silu_mul(v[1], v[9]));
                            pk.y = ZLM_PK(silu_mul(v[2], v[10]), silu_mul(v[3], v[11]));
                            pk.z = ZLM_PK(silu_mul(v[4], v[12]), silu_mul(v[5], v[13]));
                            pk.w = ZLM_PK(silu_mul(v[6], v[14]), silu_mul(v[7], v[15]));
                            *(uint4*)(row + ((part ^ sw) << 4)) = pk;
                        } else if (MODE == 0) {
                            uint4 p0, p1;
                            p0.x = ZLM_PK(v[0], v[1]); p0.y = ZLM_PK(v[2], v[3]); p0.z = ZLM_PK(v[4], v[5]); p0.w = ZLM_PK(v[6], v[7]);
                            p1.x = ZLM_PK(v[8], v[9]); p1.y = ZLM_PK(v[10], v[11]); p1.z = ZLM_PK(v[12], v[13]); p1.w = ZLM_PK(v[14], v[15]);
                            *(uint4*)(row + (((2 * part) ^ sw) << 4)) = p0;
                            *(uint4*)(row + (((2 * part + 1) ^ sw) << 4)) = p1;
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *(float4*)(row + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                    }
#undef ZLM_PK
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        const unsigned src = smem_u32(ring + (boxes % TCQ_RING) * TCQ_BOX_BYTES);
                        if (MODE == 1)
                            asm volatile(
                                "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];\n"
                                ::"l"(&map_y), "r"(x), "r"(a0row + lg * 32), "r"(src) : "memory");
                        else
                            asm volatile(
                                "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];\n"
                                ::"l"(&map_y), "r"(x), "r"(a0row + lg * 32), "r"(src) : "memory");
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    tc_ld16(tmem_base + ((unsigned)(lg * 32) << 16) + buf * TCP_ACC + (unsigned)c, v);
                    store_row16<MODE>(v, Y, arow, b0row + c, T, N, ldy);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_at(empty0[buf]);
        }
        // the boxes handed to the copy engine have been written before the block leaves
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither block leaves while the other may still read its memory or signal it
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((unsigned)(2 * TCP_ACC)) : "memory");
    }
}

// ---------------------------------------------------------------------------
// The few-token form (17 to 384 tokens) as a persistent kernel.  W is the 128-row operand,
// the tokens are the product's N (a tile of BN = 32, 64 or 128).  A work item is a tile of
// 128 outputs x BN tokens and one of `ks` shares of K; one block per SM walks the items, its
// TMA ring and its two accumulators running on across items, so that an item's start and its
// epilogue hide behind its neighbours' streams (the stand-alone blocks of gemm_tc_kernel pay
// both for every item, which at a few hundred KB of W per item is most of their time).
// The first `whole` tiles are items of their own (all of K, written in the wanted mode); each
// of the other tiles is `ks` items, which leave their fp32 shares in scratch memory for
// gemm_tc_reduce_kernel.  (Adding the shares up inside this kernel, by the epilogue warps of the
// item that finishes a tile last, was built and gave the same bits; under the load of the weight
// stream its reads of the shares took several times as long as the whole second kernel does.)
// ---------------------------------------------------------------------------
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_few_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   void* __restrict__ Y, int T, int N, int K, int ldy, int whole, int ks,
                   float* __restrict__ part) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(sB + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    unsigned* tmem_slot = (unsigned*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB_all = (K + TC_BK - 1) / TC_BK;
    const int kb_per = (KB_all + ks - 1) / ks;
    const int n_tiles = (N + TC_BM - 1) / TC_BM, t_tiles = (T + BN - 1) / BN;
    const int rest = max(1, n_tiles * t_tiles - whole);       // tiles that are cut along K
    const int items = whole + (n_tiles * t_tiles - whole) * ks;
    constexpr unsigned ACC = BN < 32 ? 32 : BN;      // tensor-memory columns of one accumulator

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(2 * ACC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_launch_dependents();

    // item -> (tile of outputs, tile of tokens, share of K); the share's k blocks
#define ZLM_ITEM(item)                                                        \
    const bool split = (item) >= whole;                                       \
    const int z = split ? ((item) - whole) / rest : 0;                        \
    const int tile = split ? whole + ((item) - whole) % rest : (item);        \
    const int a0row = (tile / t_tiles) * TC_BM, b0row = (tile % t_tiles) * BN; \
    const int kb_lo = z * kb_per;                                             \
    const int KB = split ? max(0, min(KB_all, kb_lo + kb_per) - kb_lo) : KB_all;

    // The first item's first loads of W (which no kernel of the step writes) go out before the wait
    // for the kernel before: the ring's stages are all free at the start.  The activations of those
    // stages follow after the wait, and nothing else of another kernel's is touched before it.
    int early = 0;
    if (warp == 0 && lane == 0 && (int)blockIdx.x < items) {
        ZLM_ITEM((int)blockIdx.x)
        (void)b0row;
        early = min(KB, STAGES);
        for (int kb = 0; kb < early; ++kb) {
            mbar_expect_tx(&full[kb], A_BYTES + B_BYTES);
            tma_load_2d(sA + kb * A_BYTES, &map_w, (kb_lo + kb) * TC_BK, a0row, &full[kb]);
        }
    }
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
                ZLM_ITEM(item)
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    if ((int)it < early) {      // the stage's W is on its way already
                        tma_load_2d(sB + s * B_BYTES, &map_x, (kb_lo + kb) * TC_BK, b0row, &full[s]);
                        continue;
                    }
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                    tma_load_2d(sA + s * A_BYTES, &map_w, (kb_lo + kb) * TC_BK, a0row, &full[s]);
                    tma_load_2d(sB + s * B_BYTES, &map_x, (kb_lo + kb) * TC_BK, b0row, &full[s]);
                }
            }
            if (*abort_flag) {
                for (unsigned j = it > (unsigned)STAGES ? it - STAGES : 0; j < it; ++j)
                    mbar_drain(&full[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                   ((unsigned)(TC_BM >> 4) << 24);
            unsigned it = 0, local = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++local) {
                ZLM_ITEM(item)
                (void)a0row; (void)b0row; (void)split;
                const unsigned buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag, 4);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t ad = make_desc(smem_u32(sA + s * A_BYTES)), bd = make_desc(smem_u32(sB + s * B_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma(tmem_base + buf * ACC, ad + ((k * 32) >> 4), bd + ((k * 32) >> 4), idesc, (kb | k) != 0);
                    tc_commit(&empty[s]);
                }
                tc_commit(&acc_full[buf]);
            }
            if (!ok) { tc_commit(&acc_full[0]); tc_commit(&acc_full[1]); }     // let the epilogue out
        }
    } else {
        const int lg = warp & 3;
        const size_t TN = (size_t)T * N;
        unsigned local = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
            ZLM_ITEM(item)
            const unsigned buf = local & 1;
            const bool ok = mbar_wait_warp(&acc_full[buf], (local >> 1) & 1, abort_flag, 3);
            tc_fence_after();
            if (!ok || *abort_flag) break;
            const int row = a0row + lg * 32 + lane;
            const unsigned taddr = tmem_base + ((unsigned)(lg * 32) << 16) + buf * ACC;
            if (!split) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    tc_ld16(taddr + (unsigned)c, v);
                    store_swapped16<MODE>(v, Y, row, b0row + c, T, N, ldy, lane);
                }
            } else {
                // this item's share of the tile
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    tc_ld16(taddr + (unsigned)c, v);
                    if (row < N) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (b0row + c + i < T && ZLM_CHK(part + (size_t)z * TN + (size_t)(b0row + c + i) * N + row, 4))
                                part[(size_t)z * TN + (size_t)(b0row + c + i) * N + row] = KB ? v[i] : 0.f;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
#undef ZLM_ITEM
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * ACC) : "memory");
    }
}

// adds the K shares of the outputs from n_from on up in the order 0 .. splits-1 and finishes the
// product there in the wanted mode (n_from is a multiple of 128)
template <int MODE>
__global__ void gemm_tc_reduce_kernel(void* __restrict__ Y, const float* __restrict__ part, int T, int N, int ldy,
                                      int splits, int n_from) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)T * N;
    const int width = N - n_from;
    const size_t count = (size_t)T * (MODE == 3 ? width / 2 : width);
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        if (MODE == 3) {
            // channel c of token t; its gate is output (c/8)*16 + c%8, its up 8 further
            const size_t t = e / (width / 2);
            const int c = n_from / 2 + (int)(e - t * (width / 2));
            const size_t g = t * N + (size_t)(c >> 3) * 16 + (c & 7);
            float sg = 0.f, su = 0.f;
            if (!ZLM_CHK(part + g, 4) || !ZLM_CHK(part + (splits - 1) * total + g + 8, 4) ||
                !ZLM_CHK((__nv_bfloat16*)Y + t * ldy + c, 2))
                continue;
            for (int s = 0; s < splits; ++s) { sg += part[s * total + g]; su += part[s * total + g + 8]; }
            ((__nv_bfloat16*)Y)[t * ldy + c] = __float2bfloat16_rn(silu_mul(sg, su));
        } else {
            const size_t t = e / width;
            const int n = n_from + (int)(e - t * width);
            float sum = 0.f;
            const size_t off = t * ldy + n;
            if (!ZLM_CHK(part + t * N + n, 4) || !ZLM_CHK(part + (splits - 1) * total + t * N + n, 4) ||
                !ZLM_CHK((char*)Y + off * (MODE == 0 ? 2 : 4), MODE == 0 ? 2 : 4))
                continue;
            for (int s = 0; s < splits; ++s) sum += part[s * total + t * N + n];
            if (MODE == 0) ((__nv_bfloat16*)Y)[off] = __float2bfloat16_rn(sum);
            else if (MODE == 1) ((float*)Y)[off] += sum;
            else ((float*)Y)[off] = sum;
        }
    }
}

static int launch_reduce(void* Y, const float* scratch, int T, int N, int ldy, int mode, int splits, int n_from,
                         cudaStream_t st) {
    const size_t elems = (size_t)T * (N - n_from) / (mode == 3 ? 2 : 1);
    int blocks = (int)((elems + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (mode == 0) zlm_launch(gemm_tc_reduce_kernel<0>, dim3(blocks), dim3(256), 0, st, Y, scratch, T, N, ldy, splits, n_from);
    else if (mode == 1) zlm_launch(gemm_tc_reduce_kernel<1>, dim3(blocks), dim3(256), 0, st, Y, scratch, T, N, ldy, splits, n_from);
    else if (mode == 2) zlm_launch(gemm_tc_reduce_kernel<2>, dim3(blocks), dim3(256), 0, st, Y, scratch, T, N, ldy, splits, n_from);
    else zlm_launch(gemm_tc_reduce_kernel<3>, dim3(blocks), dim3(256), 0, st, Y, scratch, T, N, ldy, splits, n_from);
    return zlm_check_launch("gemm_tc_reduce");
}

// ---------------------------------------------------------------- host side
ZlmEncodeTiledFn zlm_tensor_map_encoder() {
    static ZlmEncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (ZlmEncodeTiledFn)p;
    }
    return fn;
}

int zlm_make_map_2d(CUtensorMap* m, const void* ptr, long long rows, int cols, long long ld, int box_rows, int box_cols) {
    ZlmEncodeTiledFn enc = zlm_tensor_map_encoder();
    if (!enc) {
        zlm_set_error("tensor map: the driver does not provide cuTensorMapEncodeTiled");
        return ZLM_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        zlm_set_error("tensor map: cuTensorMapEncodeTiled failed with %d (rows=%lld cols=%d ld=%lld)", (int)r, rows, cols, ld);
        return ZLM_ERR_CUDA;
    }
    return ZLM_OK;
}

// A rows x cols matrix of 4-byte (fp32) or 2-byte (bf16) elements, row stride ld elements, as the
// target of stores and reduce-adds of boxes box_rows x box_cols; a box row is 64 bytes, kept in
// the 64-byte swizzle.
int zlm_make_map_out(CUtensorMap* m, const void* ptr, long long rows, int cols, long long ld, int elem_bytes,
                     int box_rows, int box_cols) {
    ZlmEncodeTiledFn enc = zlm_tensor_map_encoder();
    if (!enc) {
        zlm_set_error("tensor map: the driver does not provide cuTensorMapEncodeTiled");
        return ZLM_ERR_CUDA;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr,
                     dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        zlm_set_error("tensor map: cuTensorMapEncodeTiled failed with %d for an output (rows=%lld cols=%d ld=%lld)", (int)r,
                      rows, cols, ld);
        return ZLM_ERR_CUDA;
    }
    return ZLM_OK;
}

// rows x K bf16 matrix, row stride ld elements; box = box_rows x 64 elements
static int make_map(CUtensorMap* m, const void* ptr, int rows, int K, int ld, int box_rows) {
    return zlm_make_map_2d(m, ptr, rows, K, ld, box_rows, TC_BK);
}

template <int BN, int STAGES>
static int launch_tc(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy, int mode,
                     int ksplit, float* scratch, cudaStream_t st, bool add_shares = true) {
    CUtensorMap mx, mw;
    int rc = make_map(&mx, X, T, K, ldx, BN);
    if (rc) return rc;
    rc = make_map(&mw, W, N, K, K, TC_BM);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + 1024 + 256;
    dim3 grid((N + TC_BM - 1) / TC_BM, (T + BN - 1) / BN, ksplit);
    ZLM_REQUIRE(grid.y <= 65535, "gemm_tc: the product is too large (T=%d N=%d)", T, N);
    const int kmode = ksplit > 1 ? 4 : mode;
    void* dst = ksplit > 1 ? (void*)scratch : Y;
#define ZLM_TC_LAUNCH(M)                                                                                   \
    {                                                                                                      \
        auto kern = gemm_tc_kernel<BN, STAGES, M>;                                                         \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                                                                      \
        if (!attr_set) {                                                                                   \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) {                                                                        \
                zlm_set_error("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
                return ZLM_ERR_CUDA;                                                                       \
            }                                                                                              \
            attr_set = true;                                                                               \
        }                                                                                                  \
        zlm_launch(kern, grid, dim3(TC_THREADS), smem, st, mw, mx, dst, T, N, K, ldy);                     \
    }
    if (kmode == 0) ZLM_TC_LAUNCH(0)
    else if (kmode == 1) ZLM_TC_LAUNCH(1)
    else if (kmode == 2) ZLM_TC_LAUNCH(2)
    else if (kmode == 3) ZLM_TC_LAUNCH(3)
    else ZLM_TC_LAUNCH(4)
#undef ZLM_TC_LAUNCH
    rc = zlm_check_launch("gemm_tc");
    if (rc || ksplit <= 1 || !add_shares) return rc;
    return launch_reduce(Y, scratch, T, N, ldy, mode, ksplit, 0, st);
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

template <int BN, int STAGES>
static int launch_tc_persistent(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy, int mode,
                                cudaStream_t st) {
    CUtensorMap mx, mw;
    int rc = make_map(&mx, X, T, K, ldx, TC_BM);
    if (rc) return rc;
    rc = make_map(&mw, W, N, K, K, BN);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + 1024 + 256;
    const long long tiles = (long long)((T + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
    const int blocks = (int)(tiles < sm_count() ? tiles : sm_count());
#define ZLM_TCP_LAUNCH(M)                                                                                  \
    {                                                                                                      \
        auto kern = gemm_tc_persistent_kernel<BN, STAGES, M>;                                              \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                                                                      \
        if (!attr_set) {                                                                                   \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) {                                                                        \
                zlm_set_error("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
                return ZLM_ERR_CUDA;                                                                       \
            }                                                                                              \
            attr_set = true;                                                                               \
        }                                                                                                  \
        zlm_launch(kern, dim3(blocks), dim3(TC_THREADS), smem, st, mx, mw, Y, T, N, K, ldy, tile_group(TC_BM, K)); \
    }
    if (mode == 0) ZLM_TCP_LAUNCH(0)
    else if (mode == 1) ZLM_TCP_LAUNCH(1)
    else if (mode == 2) ZLM_TCP_LAUNCH(2)
    else ZLM_TCP_LAUNCH(3)
#undef ZLM_TCP_LAUNCH
    return zlm_check_launch("gemm_tc_persistent");
}

template <int BN, int STAGES>
static int launch_tc_pair(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy, int mode,
                          cudaStream_t st, const QkvEpilogue* qkv = nullptr) {
    const QkvEpilogue ep = qkv ? *qkv : QkvEpilogue{};
    CUtensorMap mx, mw;
    int rc = make_map(&mx, X, T, K, ldx, TC_BM);
    if (rc) return rc;
    rc = make_map(&mw, W, N, K, K, BN / 2);
    if (rc) return rc;
    // the results go through the copy engine where the output's rows can be described to it
    // (16-byte aligned rows); else the threads store row by row
    const int ybytes = (mode == 0 || mode == 3) ? 2 : 4;
    const int y_tma = mode >= 0 && mode <= 3 && ((size_t)ldy * ybytes) % 16 == 0 && (uintptr_t)Y % 16 == 0 &&
                      (mode != 3 || N % 2 == 0);
    CUtensorMap my = mx;
    if (y_tma) {
        rc = zlm_make_map_out(&my, Y, T, mode == 3 ? N / 2 : N, ldy, ybytes, 32, 64 / ybytes);
        if (rc) return rc;
    }
    const size_t smem = (size_t)STAGES * (TC_BM + BN / 2) * TC_BK * 2 + TCQ_OUT_BYTES + 1024 + 256;
    const long long tiles = (long long)((T + TCQ_BM - 1) / TCQ_BM) * ((N + BN - 1) / BN);
    const int pairs = (int)(tiles < sm_count() / 2 ? tiles : sm_count() / 2);
#define ZLM_TCQ_LAUNCH(M)                                                                                  \
    {                                                                                                      \
        auto kern = gemm_tc_pair_kernel<BN, STAGES, M>;                                                    \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                                                                      \
        if (!attr_set) {                                                                                   \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) {                                                                        \
                zlm_set_error("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
                return ZLM_ERR_CUDA;                                                                       \
            }                                                                                              \
            attr_set = true;                                                                               \
        }                                                                                                  \
        zlm_launch(kern, dim3(2 * pairs), dim3(TC_THREADS), smem, st, mx, mw, my, Y, T, N, K, ldy, tile_group(TCQ_BM, K), y_tma, ep); \
    }
    if (mode == 0) ZLM_TCQ_LAUNCH(0)
    else if (mode == 1) ZLM_TCQ_LAUNCH(1)
    else if (mode == 2) ZLM_TCQ_LAUNCH(2)
    else if (mode == 5) {
        if constexpr (BN == 256 || BN == 128) ZLM_TCQ_LAUNCH(5)
    }
    else ZLM_TCQ_LAUNCH(3)
#undef ZLM_TCQ_LAUNCH
    return zlm_check_launch("gemm_tc_pair");
}

// Which many-token form runs, and how wide its tiles are: 0 lets the dispatcher choose (pairs of
// blocks; the width by the rule in zlm_gemm_tc).  form 1: single blocks, 2: pairs; width 256, 240
// or 224 (pairs: 128 too).  For tests and measurements.
static int g_tc_form = 0, g_tc_width = 0;
extern "C" int zlm_gemm_tc_set_form(int form, int width) {
    ZLM_REQUIRE(form >= 0 && form <= 2, "gemm_tc: form %d", form);
    ZLM_REQUIRE(width == 0 || width == 256 || width == 240 || width == 224 || (width == 128 && form == 2),
                "gemm_tc: tile width %d", width);
    g_tc_form = form;
    g_tc_width = width;
    return ZLM_OK;
}

// How the few-token form cuts a product: tokens in tiles of bn; the first `whole` tiles of
// 128 outputs x bn tokens (as many full rounds of one tile per SM as there are) are computed
// in one piece; each of the others is cut along K into `ks` shares, as many as fill the last
// round (at most 8, each at least 8 k blocks), and a second kernel adds the shares up.
struct FewPlan { int bn, whole, ks, t_tiles; };
static FewPlan few_plan(int T, int N, int K) {
    FewPlan p;
    p.bn = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
    p.t_tiles = (T + p.bn - 1) / p.bn;
    const int tiles = ((N + TC_BM - 1) / TC_BM) * p.t_tiles, sms = sm_count();
    const int kb = (K + TC_BK - 1) / TC_BK;
    p.whole = tiles / sms * sms;
    p.whole -= p.whole % p.t_tiles;          // the split tiles are whole rows of token tiles: outputs from some n on
    const int rest = tiles - p.whole;
    p.ks = 1;
    if (rest > 0) p.ks = max(1, min(min(8, sms / rest), kb / 8));
    if (p.ks == 1) p.whole = tiles;
    return p;
}

template <int BN, int STAGES>
static int launch_tc_few(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy, int mode,
                         const FewPlan& plan, float* scratch, cudaStream_t st) {
    CUtensorMap mx, mw;
    int rc = make_map(&mx, X, T, K, ldx, BN);
    if (rc) return rc;
    rc = make_map(&mw, W, N, K, K, TC_BM);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + 1024 + 256;
    const int tiles = ((N + TC_BM - 1) / TC_BM) * plan.t_tiles;
    const long long items = plan.whole + (long long)(tiles - plan.whole) * plan.ks;
    const int blocks = (int)(items < sm_count() ? items : sm_count());
#define ZLM_TCF_LAUNCH(M)                                                                                  \
    {                                                                                                      \
        auto kern = gemm_tc_few_kernel<BN, STAGES, M>;                                                     \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                                                                      \
        if (!attr_set) {                                                                                   \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) {                                                                        \
                zlm_set_error("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
                return ZLM_ERR_CUDA;                                                                       \
            }                                                                                              \
            attr_set = true;                                                                               \
        }                                                                                                  \
        zlm_launch(kern, dim3(blocks), dim3(TC_THREADS), smem, st, mw, mx, Y, T, N, K, ldy, plan.whole, plan.ks, scratch); \
    }
    if (mode == 0) ZLM_TCF_LAUNCH(0)
    else if (mode == 1) ZLM_TCF_LAUNCH(1)
    else if (mode == 2) ZLM_TCF_LAUNCH(2)
    else ZLM_TCF_LAUNCH(3)
#undef ZLM_TCF_LAUNCH
    rc = zlm_check_launch("gemm_tc_few");
    if (rc || plan.ks <= 1) return rc;
    return launch_reduce(Y, scratch, T, N, ldy, mode, plan.ks, plan.whole / plan.t_tiles * TC_BM, st);
}

// 1 if the tensor-memory kernel takes this product (else use zlm_gemm_bf16_mma)
extern "C" int zlm_gemm_tc_supported(int T, int N, int K, int ldx) {
    return (T >= 1 && N >= 8 && K >= 8 && K % 8 == 0 && ldx % 8 == 0) ? 1 : 0;
}

// shares of K whose fp32 partial products need scratch memory (T * N floats each)
extern "C" int zlm_gemm_tc_ksplit(int T, int N, int K) {
    if (T > 384) return 1;
    return few_plan(T, N, K).ks;
}

// The width of the many-token forms' tiles (0 for the few-token forms, up to 384 tokens).  Tiles run
// in rounds of one per SM (or pair of SMs), and a round costs its width: N = 4096 at 2,048 tokens
// is 128 tiles of 256 columns on 74 pairs (2 rounds, the second 73 % full) or 144 of 240 (2 rounds,
// 97 % full).  A narrower tile re-reads the activations more often, so it has to win by more than
// 5 % in rounds x width (measured at 2,048 tokens: N = 4096 and 6144 gain 2-3 % with 240 columns,
// N = 24576 loses 3 % with 224 although it saves a round of 12).  128 columns (pairs only): half
// the reuse of the activations per product, so only where the wider tiles would leave a third of
// the pairs idle (N = 1024 at 2,048 tokens: 32 tiles on 74 pairs).
extern "C" int zlm_gemm_tc_tile_width(int T, int N, int K) {
    (void)K;
    if (T <= 384) return 0;
    if (g_tc_width) return g_tc_width;
    const bool pairs = g_tc_form != 1;
    const long long m_tiles = pairs ? (T + TCQ_BM - 1) / TCQ_BM : (T + TC_BM - 1) / TC_BM;
    const long long slots = pairs ? sm_count() / 2 : sm_count();
    auto cost = [&](int bn) { return ((m_tiles * ((N + bn - 1) / bn) + slots - 1) / slots) * bn; };
    int best = 256;
    for (int bn : {240, 224})
        if (cost(bn) * 100 < cost(256) * 95 && cost(bn) < cost(best)) best = bn;
    if (pairs && cost(128) * 100 < cost(best) * 70) best = 128;
    return best;
}

// mode 0: Y bf16 = X W^T; mode 1: Y fp32 += X W^T; mode 2: Y fp32 = X W^T;
// mode 3: Y bf16 [T, N/2] = silu(gate) * up, W's rows in groups of 8 gate + 8 up (N a multiple of 16).
// scratch: zlm_gemm_tc_ksplit(T, N, K) * T * N floats if that number of shares is more than 1, else unused.
extern "C" int zlm_gemm_tc(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy, int mode,
                           float* scratch, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(zlm_gemm_tc_supported(T, N, K, ldx), "gemm_tc: shape T=%d N=%d K=%d (row stride %d) is not taken", T, N, K, ldx);
    ZLM_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    ZLM_REQUIRE(mode >= 0 && mode <= 3, "gemm_tc: mode %d", mode);
    ZLM_REQUIRE(mode != 3 || N % 16 == 0, "gemm_tc: the fused gate/up product needs N=%d to be a multiple of 16", N);
    const int ks = zlm_gemm_tc_ksplit(T, N, K);
    ZLM_REQUIRE(ks == 1 || scratch, "gemm_tc: scratch for %d shares of K is missing", ks);
    // few tokens: W is the 128-row operand so that it streams at full height
    if (T <= 384) {
        const FewPlan plan = few_plan(T, N, K);
        const long long tiles = (long long)((N + TC_BM - 1) / TC_BM) * plan.t_tiles;
        if (plan.whole + (tiles - plan.whole) * plan.ks <= sm_count()) {
            // one round of blocks: nothing for a persistent block to overlap, and the stand-alone
            // blocks are a microsecond or two faster there (here all tiles are cut alike)
            if (T <= 32) return launch_tc<32, 8>(Y, X, W, T, N, K, ldx, ldy, mode, plan.ks, scratch, st);
            if (T <= 64) return launch_tc<64, 8>(Y, X, W, T, N, K, ldx, ldy, mode, plan.ks, scratch, st);
            return launch_tc<128, 6>(Y, X, W, T, N, K, ldx, ldy, mode, plan.ks, scratch, st);
        }
        if (T <= 32) return launch_tc_few<32, 8>(Y, X, W, T, N, K, ldx, ldy, mode, plan, scratch, st);
        if (T <= 64) return launch_tc_few<64, 8>(Y, X, W, T, N, K, ldx, ldy, mode, plan, scratch, st);
        return launch_tc_few<128, 6>(Y, X, W, T, N, K, ldx, ldy, mode, plan, scratch, st);
    }
    const int width = zlm_gemm_tc_tile_width(T, N, K);
    if (g_tc_form != 1) {
        if (width == 128) return launch_tc_pair<128, 8>(Y, X, W, T, N, K, ldx, ldy, mode, st);
        if (width == 240) return launch_tc_pair<240, 6>(Y, X, W, T, N, K, ldx, ldy, mode, st);
        if (width == 224) return launch_tc_pair<224, 6>(Y, X, W, T, N, K, ldx, ldy, mode, st);
        return launch_tc_pair<256, 6>(Y, X, W, T, N, K, ldx, ldy, mode, st);
    }
    if (width == 240) return launch_tc_persistent<240, 4>(Y, X, W, T, N, K, ldx, ldy, mode, st);
    if (width == 224) return launch_tc_persistent<224, 4>(Y, X, W, T, N, K, ldx, ldy, mode, st);
    return launch_tc_persistent<256, 4>(Y, X, W, T, N, K, ldx, ldy, mode, st);
}

// A few-token product that runs as one round of stand-alone blocks cuts K into shares and leaves
// them as fp32 [shares][T][N] in scratch; a second kernel adds them up.  Where the kernel that
// reads the product next can do that on its way (the norm that follows a product into the fp32
// stream, the norm / rotation / cache write that follows the q/k/v projection), the caller asks
// for the shares alone: zlm_gemm_tc_shares_plan tells how many there would be (0: this product is
// not of that form), zlm_gemm_tc_shares leaves them, zlm_gemm_tc_add_shares is the second kernel
// for a caller that has to finish the product after all.
extern "C" int zlm_gemm_tc_shares_plan(int T, int N, int K, int ldx) {
    if (T <= 16 || T > 384 || !zlm_gemm_tc_supported(T, N, K, ldx)) return 0;
    const FewPlan plan = few_plan(T, N, K);
    const long long tiles = (long long)((N + TC_BM - 1) / TC_BM) * plan.t_tiles;
    if (plan.ks <= 1 || plan.whole != 0 || tiles * plan.ks > sm_count()) return 0;
    return plan.ks;
}
extern "C" int zlm_gemm_tc_shares(const void* X, const void* W, int T, int N, int K, int ldx, float* scratch,
                                  cudaStream_t st) {
    const int ks = zlm_gemm_tc_shares_plan(T, N, K, ldx);
    ZLM_REQUIRE(ks > 1 && scratch, "gemm_tc_shares: the product T=%d N=%d K=%d is not cut into shares", T, N, K);
    ZLM_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    if (T <= 32) return launch_tc<32, 8>(nullptr, X, W, T, N, K, ldx, N, 0, ks, scratch, st, false);
    if (T <= 64) return launch_tc<64, 8>(nullptr, X, W, T, N, K, ldx, N, 0, ks, scratch, st, false);
    return launch_tc<128, 6>(nullptr, X, W, T, N, K, ldx, N, 0, ks, scratch, st, false);
}
extern "C" int zlm_gemm_tc_add_shares(void* Y, const float* scratch, int T, int N, int ldy, int mode, int ks, cudaStream_t st) {
    ZLM_REQUIRE(ks > 1 && scratch && mode >= 0 && mode <= 2, "gemm_tc_add_shares: %d shares, mode %d", ks, mode);
    return launch_reduce(Y, scratch, T, N, ldy, mode, ks, 0, st);
}

// 1 if the q/k/v projection of T tokens can carry norm, rotation and cache write in its epilogue:
// the many-token form on pairs of blocks, heads that divide a tile of 256 or 128 columns, the
// whole head rotated (or none of it).
extern "C" int zlm_gemm_tc_qkv_supported(int T, int N, int K, int ldx, int nq, int nkv, int hd, int n_rot) {
    if (!zlm_gemm_tc_supported(T, N, K, ldx) || T <= 384 || g_tc_form == 1) return 0;
    if (hd < 32 || hd % 32 != 0 || 256 % hd != 0 || N != (nq + 2 * nkv) * hd) return 0;
    if (n_rot != 0 && n_rot != hd) return 0;
    if (g_tc_width != 0 && g_tc_width != 256 && g_tc_width != 128) return 0;
    return 1;
}

// q [T, nq*hd] bf16 (row stride ldy) = norm+rotate(X Wq^T); k (normed, rotated) and v go to the
// tokens' places in the paged pool.  cos_sin: [2][hd/2][T] from zlm_rope_table, or null.
extern "C" int zlm_gemm_tc_qkv(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy,
                               const void* q_w, const void* k_w, int w_dtype, float eps, const float* cos_sin,
                               const int* token_pos, const int* token_slot, const int* block_table, int table_stride,
                               void* pool, int nq, int nkv, int hd, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(zlm_gemm_tc_qkv_supported(T, N, K, ldx, nq, nkv, hd, cos_sin ? hd : 0),
                "gemm_tc_qkv: T=%d N=%d K=%d with %d+2x%d heads of %d is not a shape the fused projection takes",
                T, N, K, nq, nkv, hd);
    ZLM_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)Y % 16 == 0) && ldy % 8 == 0 &&
                ((uintptr_t)pool % 16 == 0), "gemm_tc_qkv: operands must be 16-byte aligned");
    ZLM_REQUIRE((q_w == nullptr) == (k_w == nullptr) || nkv == 0, "gemm_tc_qkv: one norm weight without the other");
    ZLM_REQUIRE(nkv == 0 || (pool && block_table && token_slot), "gemm_tc_qkv: the cache is missing");
    QkvEpilogue ep{q_w, k_w, w_dtype, eps, cos_sin, token_pos, token_slot, block_table, table_stride,
                   (__nv_bfloat16*)pool, nq, nkv, hd};
    // tiles of whole heads: 256 columns, or 128 where 256 would leave pairs of SMs idle
    int width = g_tc_width ? g_tc_width : zlm_gemm_tc_tile_width(T, N, K);
    if (width != 128 || 128 % hd != 0) width = 256;
    if (width == 128) return launch_tc_pair<128, 8>(Y, X, W, T, N, K, ldx, ldy, 5, st, &ep);
    return launch_tc_pair<256, 6>(Y, X, W, T, N, K, ldx, ldy, 5, st, &ep);
}

// cos and sin of pos[t] * inv_freq[i] for the step's tokens: out[0][t][i] = cos, out[1][t][i] = sin.
// The angle and its sine and cosine are computed in fp32, as the stand-alone rotation kernel does.
__global__ void rope_table_kernel(float* __restrict__ out, const float* __restrict__ inv_freq,
                                  const int* __restrict__ token_pos, int T, int half) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();              // the table may still be read by the products of the step before
    if (idx >= T * half) return;
    const int i = idx / T, t = idx - i * T;         // [cos | sin][angle][token]: a warp of the product's epilogue reads along tokens
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(inv_freq + i, 4) || !ZLM_CHK(out + idx, 4) ||
        !ZLM_CHK(out + (size_t)T * half + idx, 4))
        return;
    float sn, cs;
    sincosf((float)token_pos[t] * inv_freq[i], &sn, &cs);
    out[idx] = cs;
    out[(size_t)T * half + idx] = sn;
}
extern "C" int zlm_rope_table(float* out, const float* inv_freq, int n_rot, const int* token_pos, int T, cudaStream_t st) {
    if (T == 0 || n_rot == 0) return ZLM_OK;
    ZLM_REQUIRE(n_rot > 0 && n_rot % 2 == 0 && T > 0, "rope_table: n_rot=%d T=%d", n_rot, T);
    const int half = n_rot / 2;
    const long long n = (long long)T * half;
    zlm_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, out, inv_freq, token_pos, T, half);
    return zlm_check_launch("rope_table");
}

// ---------------------------------------------------------------------------------------
// The give-up path on purpose.  One block with the roles of the product kernels, built from
// the same helpers: the producer loads one tile of `src` by TMA; the issuer allocates tensor
// memory and then waits, with the short limit given, on a barrier at which nobody ever
// arrives; an epilogue warp waits with the ordinary limit on another such barrier and must
// be released by the abort flag, not by its own clock.  Then everyone walks to the end as the
// product kernels do: the producer lets its copy land, tensor memory is freed, the kernel
// returns.  Nothing faults and nothing is left waiting.  out[0] = the status code it reported,
// out[1] = 1 if the epilogue warp was released by the flag, out[2] = nanoseconds the kernel took,
// out[3] = 1 if the tile had landed when the producer looked.
// ---------------------------------------------------------------------------------------
#define TC_TEST_WHERE 0x7e
__global__ void __launch_bounds__(96, 1)
gemm_tc_giveup_kernel(const __grid_constant__ CUtensorMap map, unsigned long long limit_ns, int* __restrict__ out) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + TC_BM * TC_BK * 2);
    uint64_t* never_a = full + 1;
    uint64_t* never_b = full + 2;
    unsigned* tmem_slot = (unsigned*)(full + 3);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long t0 = tc_now_ns();
    if (threadIdx.x == 0) {
        mbar_init(full, 1);
        mbar_init(never_a, 1);
        mbar_init(never_b, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(64u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(full, TC_BM * TC_BK * 2);
            tma_load_2d(smem, &map, 0, 0, full);
            // the producer's own wait: released by the flag once the issuer has given up
            const bool ok = mbar_wait(never_b, 0, abort_flag, 1);
            if (!ok) mbar_drain(full, 0);
            out[3] = mbar_try(full, 0) ? 1 : 0;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const bool ok = mbar_wait(never_a, 0, abort_flag, TC_TEST_WHERE, limit_ns);
            out[0] = ok ? 0 : ((TC_FAMILY << 8) | TC_TEST_WHERE);
        }
    } else {
        const bool ok = mbar_wait(never_b, 0, abort_flag, 3);
        if (lane == 0) out[1] = (!ok && *abort_flag == TC_TEST_WHERE) ? 1 : 0;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(64u) : "memory");
    }
    if (threadIdx.x == 0) out[2] = (int)min(tc_now_ns() - t0, 2000000000ull);
}

// For tests: runs the give-up path once with a wait limit of `limit_ns` (at most 100 ms).
// src: 128 x 64 bf16, 16-byte aligned; out: 4 ints (see the kernel).
extern "C" int zlm_test_bounded_wait(const void* src, int* out, unsigned long long limit_ns, cudaStream_t st) {
    ZLM_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ull, "test_bounded_wait: the limit must be at most 100 ms");
    CUtensorMap m;
    int rc = zlm_make_map_2d(&m, src, TC_BM, TC_BK, TC_BK, TC_BM, TC_BK);
    if (rc) return rc;
    zlm_launch(gemm_tc_giveup_kernel, dim3(1), dim3(96), TC_BM * TC_BK * 2 + 1024 + 256, st, m, limit_ns, out);
    return zlm_check_launch("test_bounded_wait");
}

ZLM_TRANSLATION_UNIT(gemm_tcgen05)
