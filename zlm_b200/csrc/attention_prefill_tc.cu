// Prefill attention on the 5th-generation tensor cores, head size 128, bf16 paged cache.
//
// A block owns 128 query tokens of one sequence and HPC (1 or 2) query heads of one kv
// group, and walks the keys these tokens may see in steps of 128 (two pages of the cache);
// the heads of a block share the K and V tiles in shared memory.
//   warp 0      TMA producer: the Q tiles once, then a ring of K steps and one of V steps
//   warp 1      issues every head's S = Q K^T (128 x 128, fp32 in tensor memory) and
//               O += P V (128 x 128 in tensor memory) with tcgen05.mma: the warp stays whole and
//               one elected lane issues the 8 products of a step from one block of instructions
//               (measured alone, such a block issues a product every 65 cycles, the tensor cores'
//               rate; a thread issuing them one by one needs 108 each, and two issuing warps
//               slow each other)
//   4 warps per head: softmax, thread = query row.  They take the row's 128 scores into
//               registers (and give S back: the next step's S is computed while this step's
//               softmax runs), mask by the row's own position and window, keep a running maximum
//               and sum in fp32, write P as bf16 into shared memory in the layout the second
//               product wants, and at the end scale O by 1/sum and store it.
// The running maximum is lazy: O is only rescaled (read from tensor memory, scaled,
// written back) when a row's maximum grows by more than 2^8; otherwise the old
// reference stays, which changes nothing in exact arithmetic (the same reference is
// used for P and for the sum) and keeps P below 2^8.
// A sequence with an odd number of pages loads its last page twice; the second copy's keys
// lie beyond every row's position and are masked.  Every wait is bounded (see gemm_tcgen05.cu).
//
// Formula: s_t = (q . k_t) / sqrt(hd) for t in [t_start, pos], softmax, o = sum p_t v_t
// (src/kernels/transformer/attention.zig:86-164; per-row bound in block prefill:
// src/runtime/executor.zig:565-584; window start: :93-98).
#define TC_FAMILY 2
#include "tc_common.cuh"
#include <math.h>

#define FA_BM 128          // query rows per block
#define FA_HD 128          // head size this kernel is built for
#define FA_BK 128          // keys per step: two pages
#define FA_RESCALE 8.0f    // log2 units
#define FA_THREADS(H) (64 + 128 * (H))      // producer, issuing warp, 4 softmax warps per head


// 2^x on the special-function unit; the arguments here are at most 2^8 after the lazy rescale
__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned fa_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}
// Eight products from one block of instructions, issued by one elected lane of a whole warp;
// descriptors count in units of 16 bytes.
// S = Q K^T over the head's 128 dims: both operands K-major in two halves of 64 dims, 16 KB
// apart (128 rows of 128 bytes); 16 dims are 32 bytes on.  The first product overwrites.
__device__ __forceinline__ void fa_issue_s8(unsigned tmem_d, uint64_t qd, uint64_t kd, unsigned idesc) {
    asm volatile(
        "{\n\t.reg .pred q, p0, p1;\n\t.reg .b64 da, db;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
        "add.u64 da, %1, 2;\n\tadd.u64 db, %2, 2;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 4;\n\tadd.u64 db, %2, 4;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 6;\n\tadd.u64 db, %2, 6;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1024;\n\tadd.u64 db, %2, 1024;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1026;\n\tadd.u64 db, %2, 1026;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1028;\n\tadd.u64 db, %2, 1028;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1030;\n\tadd.u64 db, %2, 1030;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(qd), "l"(kd), "r"(idesc) : "memory");
}
// O (+)= P V over the step's 128 keys, 16 keys a product.  P K-major in two halves of 64 keys
// (16 KB apart; 16 keys are 32 bytes on); V MN-major, a page after the other (16 KB apart), 16
// keys are 2 KB on.  The first product accumulates unless it is the block's first step.
__device__ __forceinline__ void fa_issue_pv8(unsigned tmem_d, uint64_t pd, uint64_t vd, unsigned idesc, unsigned acc_first) {
    asm volatile(
        "{\n\t.reg .pred q, p0, p1;\n\t.reg .b64 da, db;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
        "add.u64 da, %1, 2;\n\tadd.u64 db, %2, 128;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 4;\n\tadd.u64 db, %2, 256;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 6;\n\tadd.u64 db, %2, 384;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1024;\n\tadd.u64 db, %2, 1024;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1026;\n\tadd.u64 db, %2, 1152;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1028;\n\tadd.u64 db, %2, 1280;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "add.u64 da, %1, 1030;\n\tadd.u64 db, %2, 1408;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p1;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(pd), "l"(vd), "r"(idesc), "r"(acc_first) : "memory");
}
// an arrival at `bar` once the products issued so far have retired, from the same elected lane
__device__ __forceinline__ void fa_commit(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(smem_u32(bar)) : "memory");
}

template <int HPC>
__global__ void __launch_bounds__(FA_THREADS(HPC), 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_start, int R, int tiles_per_seq, int nq, int nkv,
                            float scale_log2, int window) {
    constexpr int KST = HPC == 2 ? 1 : 2;                           // stages of keys and of values: what fits beside
    constexpr int VST = HPC == 2 ? 2 : 3;                           // the Q and P tiles (7 tiles of 32 KB in all)
    constexpr unsigned Q_BYTES = FA_BM * FA_HD * 2;                 // two halves of [128][64]
    constexpr unsigned P_BYTES = FA_BM * FA_BK * 2;                 // two halves of [128 rows][64 keys]
    constexpr unsigned PAGE_BYTES = ZLM_PAGE * FA_HD * 2;           // K or V of one page: two halves of [64][64]
    constexpr unsigned KV_BYTES = 2 * PAGE_BYTES;                   // K or V of a step
    static_assert(Q_BYTES / 2 == 16384 && P_BYTES / 2 == 16384 && KV_BYTES / 2 == 16384 && PAGE_BYTES == 16384,
                  "the constants of the issue blocks");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                                       // [HPC] Q tiles
    unsigned char* sP = sQ + HPC * Q_BYTES;                         // [HPC] P tiles
    unsigned char* sK = sP + HPC * P_BYTES;                         // [KST]: dims 0..63 of the 128 keys, then dims 64..127
    unsigned char* sV = sK + KST * KV_BYTES;                        // [VST]: page 0 (two halves), page 1
    uint64_t* q_full = (uint64_t*)(sV + VST * KV_BYTES);
    uint64_t* k_full = q_full + 1;             // [KST]      TMA bytes landed
    uint64_t* k_empty = k_full + KST;          // [KST]      the heads' S = Q K^T of that step retired
    uint64_t* v_full = k_empty + KST;          // [VST]
    uint64_t* v_empty = v_full + VST;          // [VST]      the heads' O += P V of that step retired
    uint64_t* s_full = v_empty + VST;          // [HPC]      S = Q K^T retired
    uint64_t* s_empty = s_full + HPC;          // [HPC]      the softmax warps have S in registers
    uint64_t* p_full = s_empty + HPC;          // [HPC]      P written (and O rescaled if needed)
    uint64_t* pv_done = p_full + HPC;          // [HPC]      O += P V of a step retired: P may be overwritten, O is at rest
    unsigned* tmem_slot = (unsigned*)(pv_done + HPC);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    {
        // the tiles leave less than a kilobyte for rounding the base up to the 1024 bytes that the
        // swizzled tiles want; if that ever is not enough, the block says so and leaves
        unsigned dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;\n" : "=r"(dyn));
        if ((unsigned char*)(tmem_slot + 4) > smem_raw + dyn) {
            if (threadIdx.x == 0) zlm_report_status((TC_FAMILY << 8) | 0x40);
            return;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blocks are numbered so that the tiles with the most pages (the last rows of the longest
    // prompts) start first and the short ones fill the gaps at the end
    const int n_hb = nq / HPC;                 // head groups
    const int rank = blockIdx.x / n_hb;        // 0 = the last tile of a sequence
    const int b = tiles_per_seq - 1 - rank / R, r = rank % R;
    const int head0 = (blockIdx.x % n_hb) * HPC;   // the block's first query head; its heads share a kv head
    if (!ZLM_CHK(cu_seqlens + r, 8) || !ZLM_CHK(seq_start + r, 4) || !ZLM_CHK(seq_slot + r, 4)) return;   // block-uniform
    const int tok0 = cu_seqlens[r], n_new = cu_seqlens[r + 1] - tok0;
    const int row0 = b * FA_BM;
    if (row0 >= n_new) return;
    const int rows = min(FA_BM, n_new - row0);
    const int kvh = head0 / (nq / nkv);
    const int start = seq_start[r];
    const int* pages = block_table + (size_t)seq_slot[r] * table_stride;
    const int first_pos = start + row0, last_pos = start + row0 + rows - 1;
    const int blk_lo = (window != 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
    const int page_lo = blk_lo / ZLM_PAGE, page_hi = last_pos / ZLM_PAGE + 1;
    const int NP = page_hi - page_lo;
    const int NS = (NP + 1) / 2;               // steps of two pages

    // K and V of step j into their stages (the producer thread; false if a wait gave up)
    int k_issued = 0, v_issued = 0;
    auto load_step = [&](int j) -> bool {
        int page[2];
#pragma unroll
        for (int pg = 0; pg < 2; ++pg) {
            // an odd last page comes twice: its second copy's keys are beyond every row's position
            const int lp = min(page_lo + 2 * j + pg, page_hi - 1);
            page[pg] = ZLM_CHK(pages + lp, 4) ? pages[lp] : 0;
        }
        const int sk = j % KST, sv = j % VST;
        if (!mbar_wait(&k_empty[sk], ((j / KST) & 1) ^ 1, abort_flag, 1)) return false;
        mbar_expect_tx(&k_full[sk], KV_BYTES);
#pragma unroll
        for (int pg = 0; pg < 2; ++pg) {
            // K: [half][page][64 keys][64 dims]: the 128 keys of a half are one operand tile
            const int krow = ((page[pg] * 2 + 0) * nkv + kvh) * ZLM_PAGE;
            tma_load_2d(sK + sk * KV_BYTES + pg * (PAGE_BYTES / 2), &map_kv, 0, krow, &k_full[sk]);
            tma_load_2d(sK + sk * KV_BYTES + KV_BYTES / 2 + pg * (PAGE_BYTES / 2), &map_kv, 64, krow, &k_full[sk]);
        }
        k_issued = j + 1;
        if (!mbar_wait(&v_empty[sv], ((j / VST) & 1) ^ 1, abort_flag, 1)) return false;
        mbar_expect_tx(&v_full[sv], KV_BYTES);
#pragma unroll
        for (int pg = 0; pg < 2; ++pg) {
            // V: [page][half][64 keys][64 dims]
            const int vrow = ((page[pg] * 2 + 1) * nkv + kvh) * ZLM_PAGE;
            tma_load_2d(sV + sv * KV_BYTES + pg * PAGE_BYTES, &map_kv, 0, vrow, &v_full[sv]);
            tma_load_2d(sV + sv * KV_BYTES + pg * PAGE_BYTES + PAGE_BYTES / 2, &map_kv, 64, vrow, &v_full[sv]);
        }
        v_issued = j + 1;
        return true;
    };
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_kv) : "memory");
        mbar_init(q_full, 1);
        for (int s = 0; s < KST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < VST; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int i = 0; i < HPC; ++i) {
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&p_full[i], 4); mbar_init(&pv_done[i], 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // this thread is the producer: the Q tiles and the first step's keys and values are on
        // their way before the block has met (they arrive at barriers this thread has just set
        // up; their stages are free, so nothing waits).  Q and this step's keys and values come
        // from the kernel before: as a dependent launch the block is set up while that kernel
        // drains, and waits for it here.
        pdl_launch_dependents();
        pdl_wait();
        mbar_expect_tx(q_full, HPC * Q_BYTES);
        for (int h = 0; h < HPC; ++h) {
            // Q: two 64-column halves per head, 128 token rows
            tma_load_2d(sQ + h * Q_BYTES, &map_q, (head0 + h) * FA_HD, tok0 + row0, q_full);
            tma_load_2d(sQ + h * Q_BYTES + Q_BYTES / 2, &map_q, (head0 + h) * FA_HD + 64, tok0 + row0, q_full);
        }
        if (NS > 0) load_step(0);
    }
    if (warp == 1) {
        // columns per head: S [0,128), O [128,256)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(256u * HPC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();              // (thread 0 has waited before the block met; for the others this returns at once)
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int j = 1; j < NS; ++j)
                if (!load_step(j)) break;
            if (*abort_flag) {
                mbar_drain(q_full, 0);
                for (int j = max(0, k_issued - KST); j < k_issued; ++j) mbar_drain(&k_full[j % KST], (j / KST) & 1);
                for (int j = max(0, v_issued - VST); j < v_issued; ++j) mbar_drain(&v_full[j % VST], (j / VST) & 1);
            }
        }
    } else if (warp == 1) {
        // S: M 128, N 128, both operands K-major.  O: M 128, N 128, A (P) K-major, B (V) MN-major.
        const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FA_BK >> 3) << 17) | (8u << 24);
        const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(FA_HD >> 3) << 17) | (8u << 24);
        bool ok = mbar_wait_warp(q_full, 0, abort_flag, 2);
        // S of step j for every head: the keys are there, and the head's softmax warps have taken
        // S of step j - 1 into registers
        auto issue_s = [&](int j) -> bool {
            const int s = j % KST;
            if (!mbar_wait_warp(&k_full[s], (j / KST) & 1, abort_flag, 2)) return false;
            const uint64_t kd = make_desc(smem_u32(sK + s * KV_BYTES));
#pragma unroll
            for (int h = 0; h < HPC; ++h) {
                if (j > 0 && !mbar_wait_warp(&s_empty[h], (j - 1) & 1, abort_flag, 5)) return false;
                tc_fence_after();
                fa_issue_s8(tmem_base + h * 256, make_desc(smem_u32(sQ + h * Q_BYTES)), kd, idesc_s);
                fa_commit(&s_full[h]);
            }
            fa_commit(&k_empty[s]);                // the keys' stage is free when the heads' S have retired
            return true;
        };
        if (ok && NS > 0) ok = issue_s(0);
        for (int j = 0; j < NS && ok; ++j) {
            if (j + 1 < NS) { ok = issue_s(j + 1); if (!ok) break; }
            const int s = j % VST;
            ok = mbar_wait_warp(&v_full[s], (j / VST) & 1, abort_flag, 2);
            if (!ok) break;
            // a V page: [64 keys][128 bytes] for dims 0..63, then the same for dims 64..127:
            // 16 keys a product = 2048 bytes; next 64 dims 8192 bytes on; 8-key groups 1024 bytes apart
            const uint64_t vd = make_desc_ex(smem_u32(sV + s * KV_BYTES), PAGE_BYTES / 2, 1024);
#pragma unroll
            for (int h = 0; h < HPC; ++h) {
                ok = mbar_wait_warp(&p_full[h], j & 1, abort_flag, 6);
                if (!ok) break;
                tc_fence_after();
                fa_issue_pv8(tmem_base + h * 256 + 128, make_desc(smem_u32(sP + h * P_BYTES)), vd, idesc_o, j != 0);
                fa_commit(&pv_done[h]);
            }
            if (!ok) break;
            fa_commit(&v_empty[s]);                // the values' stage is free when the heads' products have retired
        }
        if (!ok) {
            for (int h = 0; h < HPC; ++h) {        // let the softmax warps out
                fa_commit(&s_full[h]);
                fa_commit(&pv_done[h]);
            }
        }
    } else {
        const int hh = (warp - 2) >> 2;                 // which of the block's heads this warp serves
        const int head = head0 + hh;
        const unsigned tmem_s = tmem_base + hh * 256, tmem_o = tmem_s + 128;
        unsigned char* const sP_h = sP + hh * P_BYTES;
        const int lg = warp & 3;
        const int i = lg * 32 + lane;                   // row of the tile = lane of tensor memory
        const bool row_ok = i < rows;
        const int pos = start + row0 + i;
        const int lo = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
        const unsigned lane_addr = (unsigned)(lg * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < NS; ++j) {
            ok = mbar_wait_warp(&s_full[hh], j & 1, abort_flag, 3);
            tc_fence_after();
            if (!ok || *abort_flag) { ok = false; break; }
            const int kbase = (page_lo + 2 * j) * ZLM_PAGE;
            // a step that every row of the tile sees whole needs no mask (block-uniform test)
            const bool inner = rows == FA_BM && kbase + FA_BK - 1 <= first_pos &&
                               (window == 0 || kbase >= last_pos + 1 - window);
            // the row's 128 scores into registers in one round trip to tensor memory; then S is free
            float sv[FA_BK];
#pragma unroll
            for (int c = 0; c < FA_BK; c += 16) tc_ld16_nowait(tmem_s + lane_addr + c, sv + c);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[hh]);
            // four independent chains of maxima (raw scores; the scale is positive)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (inner) {
#pragma unroll
                for (int e = 0; e < FA_BK; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], sv[e]);
            } else {
#pragma unroll
                for (int e = 0; e < FA_BK; ++e) {
                    const int key = kbase + e;
                    const bool vis = row_ok && key <= pos && key >= lo;
                    sv[e] = vis ? sv[e] : -INFINITY;
                    mx4[e & 3] = fmaxf(mx4[e & 3], sv[e]);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // -inf stays -inf
            // lazy reference: move it only when the maximum grew by more than 2^8
            const bool grow = mx > m_ref + FA_RESCALE;              // also true for the first real maximum
            const float m_new = grow ? mx : m_ref;
            const float alpha = (grow && m_ref != -INFINITY) ? exp2f(m_ref - m_new) : 1.0f;
            const bool need_rescale = grow && m_ref != -INFINITY && j > 0;
            // the product of step j - 1 has retired: its P may be overwritten, and O is at rest
            // (step j's cannot have been issued, it waits for this warp)
            if (j > 0) {
                ok = mbar_wait_warp(&pv_done[hh], (j - 1) & 1, abort_flag, 7);
                tc_fence_after();
                if (!ok) break;
            }
            if (__any_sync(0xffffffffu, need_rescale)) {
#pragma unroll 1
                for (int c = 0; c < FA_HD; c += 16) {
                    float ov[16];
                    tc_ld16(tmem_o + lane_addr + c, ov);
#pragma unroll
                    for (int e = 0; e < 16; ++e) ov[e] *= alpha;
                    tc_st16(tmem_o + lane_addr + c, ov);
                }
                tc_wait_st();
                tc_fence_before();
            }
            l *= alpha;
            m_ref = m_new;
            const float ref = m_ref == -INFINITY ? 0.f : m_ref;
            // P = 2^(s * scale - ref) (2^-inf = 0 for masked keys) -> shared memory: two halves of 64
            // keys, 128 bytes a row, 16-byte chunks swizzled by (row % 8)
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ch = 0; ch < FA_BK / 8; ++ch) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = fa_ex2(fmaf(sv[ch * 8 + e], scale_log2, -ref));
                    ps4[e & 3] += p[e];
                }
                uint4 pk;
                pk.x = fa_pack(p[0], p[1]); pk.y = fa_pack(p[2], p[3]);
                pk.z = fa_pack(p[4], p[5]); pk.w = fa_pack(p[6], p[7]);
                *(uint4*)(sP_h + (ch >> 3) * (P_BYTES / 2) + i * 128 + (((ch & 7) ^ (i & 7)) << 4)) = pk;
            }
            l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[hh]);
        }
        if (ok && NS > 0) ok = mbar_wait_warp(&pv_done[hh], (NS - 1) & 1, abort_flag, 8);
        tc_fence_after();
        if (ok && !*abort_flag) {
            const float inv = row_ok ? 1.0f / l : 0.f;
            __nv_bfloat16* orow = out + (size_t)(tok0 + row0 + i) * out_stride + (size_t)head * FA_HD;
#pragma unroll 1
            for (int c = 0; c < FA_HD; c += 16) {
                float ov[16];
                tc_ld16(tmem_o + lane_addr + c, ov);
                if (row_ok && ZLM_CHK(orow + c, 32)) {
                    uint4 a, bq;
                    a.x = fa_pack(ov[0] * inv, ov[1] * inv); a.y = fa_pack(ov[2] * inv, ov[3] * inv);
                    a.z = fa_pack(ov[4] * inv, ov[5] * inv); a.w = fa_pack(ov[6] * inv, ov[7] * inv);
                    bq.x = fa_pack(ov[8] * inv, ov[9] * inv); bq.y = fa_pack(ov[10] * inv, ov[11] * inv);
                    bq.z = fa_pack(ov[12] * inv, ov[13] * inv); bq.w = fa_pack(ov[14] * inv, ov[15] * inv);
                    *(uint4*)(orow + c) = a;
                    *(uint4*)(orow + c + 8) = bq;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256u * HPC) : "memory");
    }
}

extern "C" int zlm_attention_prefill_tc_supported(int nq, int nkv, int hd, int q_stride, int out_stride) {
    return (hd == FA_HD && nkv > 0 && nq % nkv == 0 && q_stride % 8 == 0 && out_stride % 8 == 0) ? 1 : 0;
}

// pool_rows: pages * 2 * nkv * 64 (all rows of the layer's pool, head size 128 each)
static int g_fa_heads = 0;

// Heads of a kv group per block.  Two heads can share a block (they share its keys and values,
// and one head's softmax runs beside the other's: a step of 128 keys takes the two about 4,000
// cycles against 2,500 for one alone), but the blocks are then half as many and the longest
// 1.6 times as long.  The step takes about as long as the larger of its longest block (the last
// tile of the longest prompt) and its whole work spread over the SMs; the form for which that is
// smaller runs (2,048 tokens, 16 heads over 8: 38 us with one head a block, 46 with two; 32 over
// 8: 73 and 54).  Odd groups take one.
extern "C" int zlm_attention_prefill_tc_heads(int R, int max_new, int nq, int nkv) {
    if (nkv <= 0 || nq % nkv != 0 || (nq / nkv) % 2 != 0) return 1;
    if (g_fa_heads) return g_fa_heads;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const int tiles = (max_new + FA_BM - 1) / FA_BM;
    const double pairs_cost = 1.6;                                          // a block of two heads, per step, against one head
    const double work = (double)R * tiles * (tiles + 1) / 2 / sms;          // tiles' pages summed, per SM and head
    const double two = fmax(tiles * pairs_cost, work * (nq / 2) * pairs_cost), one = fmax((double)tiles, work * nq);
    return two <= one ? 2 : 1;
}

extern "C" int zlm_attention_prefill_tc(void* out, int out_stride, const void* q, int q_stride, int T,
                                        const void* pool, long long pool_pages, const int* block_table,
                                        int table_stride, const int* cu_seqlens, const int* seq_slot,
                                        const int* seq_start, int R, int max_new, int nq, int nkv, int hd,
                                        float scale, int window, cudaStream_t st) {
    if (R == 0 || max_new == 0) return ZLM_OK;
    ZLM_REQUIRE(zlm_attention_prefill_tc_supported(nq, nkv, hd, q_stride, out_stride),
                "attention_prefill_tc: %d heads over %d kv heads of size %d (strides %d, %d) is not a shape this kernel takes",
                nq, nkv, hd, q_stride, out_stride);
    ZLM_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)pool % 16 == 0),
                "attention_prefill_tc: q, out and the pool must be 16-byte aligned");
    ZLM_REQUIRE(pool_pages * 2 * nkv * ZLM_PAGE < 2147483647LL, "attention_prefill_tc: the pool has too many rows for a tensor map coordinate");
    CUtensorMap mq, mkv;
    int rc = zlm_make_map_2d(&mq, q, T, nq * hd, q_stride, FA_BM, 64);
    if (rc) return rc;
    rc = zlm_make_map_2d(&mkv, pool, pool_pages * 2 * nkv * ZLM_PAGE, hd, hd, ZLM_PAGE, 64);
    if (rc) return rc;
    const int tiles = (max_new + FA_BM - 1) / FA_BM;
    const int hpc = zlm_attention_prefill_tc_heads(R, max_new, nq, nkv);
    ZLM_REQUIRE((long long)R * tiles * nq < 2147483647LL, "attention_prefill_tc: too many tiles");
    // seven tiles of 32 KB (Q and P per head, the K and V stages), barriers, and what is left of a kilobyte for rounding the base up
    size_t smem = (size_t)7 * FA_BK * FA_HD * 2 + 256 + 1024;
    if (smem > 232448) smem = 232448;
#define ZLM_FA_LAUNCH(H)                                                                                          \
    {                                                                                                             \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                     \
        if (!attr_set) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<H>,                                  \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
            if (e != cudaSuccess) {                                                                               \
                zlm_set_error("attention_prefill_tc: cannot reserve %zu bytes of shared memory: %s", smem,        \
                              cudaGetErrorString(e));                                                             \
                return ZLM_ERR_CUDA;                                                                              \
            }                                                                                                     \
            attr_set = true;                                                                                      \
        }                                                                                                         \
        zlm_launch(attention_prefill_tc_kernel<H>, dim3(R * tiles * (nq / H)), dim3(FA_THREADS(H)), smem, st, mq, mkv,    \
                   (__nv_bfloat16*)out, out_stride, block_table, table_stride, cu_seqlens, seq_slot, seq_start,   \
                   R, tiles, nq, nkv, scale * 1.4426950408889634f, window);                                       \
    }
    if (hpc == 2) ZLM_FA_LAUNCH(2)
    else ZLM_FA_LAUNCH(1)
#undef ZLM_FA_LAUNCH
    return zlm_check_launch("attention_prefill_tc");
}

// heads of a kv group per block: 0 lets the dispatcher choose; 1 or 2 force that many where the kv
// groups are even (odd groups always take one).  For tests and measurements.
extern "C" int zlm_attention_prefill_tc_set_heads(int heads) {
    ZLM_REQUIRE(heads >= 0 && heads <= 2, "attention_prefill_tc: %d heads per block cannot be forced", heads);
    g_fa_heads = heads;
    return ZLM_OK;
}

ZLM_TRANSLATION_UNIT(attention_prefill_tc)
