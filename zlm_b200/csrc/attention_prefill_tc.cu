// Prefill attention on the 5th-generation tensor cores, head size 128, bf16 paged cache.
//
// A block owns 128 query tokens of one sequence and HPC (1 or 2) query heads of one kv
// group, and walks the sequence's pages (64 keys each) that these tokens may see; the
// heads of a block share the K and V tiles in shared memory, and while the softmax
// warps of one head work, the tensor cores serve the other.
//   warp 0      TMA producer: the Q tiles once, then a ring of (K page, V page) tiles
//   1 warp per head: one thread of it issues that head's S = Q K^T (128 x 64, fp32 in
//               tensor memory, two S buffers) and O += P V (128 x 128 in tensor memory)
//               with tcgen05.mma (issuing a product costs one thread about 70 cycles, so
//               the heads do not share an issuer)
//   4 warps per head: softmax, thread = query row.  They read S from tensor memory, mask by the
//               row's own position and window, keep a running maximum and sum in fp32,
//               write P as bf16 into shared memory in the layout the second product
//               wants, and at the end scale O by 1/sum and store it.
// The running maximum is lazy: O is only rescaled (read from tensor memory, scaled,
// written back) when a row's maximum grows by more than 2^8; otherwise the old
// reference stays, which changes nothing in exact arithmetic (the same reference is
// used for P and for the sum) and keeps P below 2^8.
// While the softmax warps work on page j, the product warp already computes S for
// page j+1 into the other S buffer.  Every wait is bounded (see gemm_tcgen05.cu).
//
// Formula: s_t = (q . k_t) / sqrt(hd) for t in [t_start, pos], softmax, o = sum p_t v_t
// (src/kernels/transformer/attention.zig:86-164; per-row bound in block prefill:
// src/runtime/executor.zig:565-584; window start: :93-98).
#define TC_FAMILY 2
#include "tc_common.cuh"
#include <math.h>

#define FA_BM 128          // query rows per block
#define FA_HD 128          // head size this kernel is built for
#define FA_STAGES 3
#define FA_RESCALE 8.0f    // log2 units


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

template <int HPC>
__global__ void __launch_bounds__(32 + 160 * HPC, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_start, int R, int tiles_per_seq, int nq, int nkv,
                            float scale_log2, int window) {
    constexpr unsigned Q_BYTES = FA_BM * FA_HD * 2;                 // two halves of [128][64]
    constexpr unsigned KV_BYTES = ZLM_PAGE * FA_HD * 2;             // K or V: two halves of [64][64]
    constexpr unsigned P_BYTES = FA_BM * ZLM_PAGE * 2;              // [128][64]
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                                       // [HPC] Q tiles
    unsigned char* sK = sQ + HPC * Q_BYTES;
    unsigned char* sV = sK + FA_STAGES * KV_BYTES;
    unsigned char* sP = sV + FA_STAGES * KV_BYTES;                  // [HPC][2] P buffers
    uint64_t* q_full = (uint64_t*)(sP + HPC * 2 * P_BYTES);
    uint64_t* kv_full = q_full + 1;            // [STAGES]   TMA bytes landed
    uint64_t* kv_empty = kv_full + FA_STAGES;  // [STAGES]   every head's O += P V of that page retired
    uint64_t* s_full = kv_empty + FA_STAGES;   // [HPC][2]   S = Q K^T retired
    uint64_t* s_empty = s_full + 2 * HPC;      // [HPC][2]   softmax has read S
    uint64_t* p_full = s_empty + 2 * HPC;      // [HPC][2]   P written (and O rescaled if needed)
    uint64_t* pv_done = p_full + 2 * HPC;      // [HPC]      an O += P V of that head retired
    unsigned* tmem_slot = (unsigned*)(pv_done + HPC);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

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

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < FA_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], HPC); }
        for (int i = 0; i < 2 * HPC; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&p_full[i], 4); }
        for (int i = 0; i < HPC; ++i) mbar_init(&pv_done[i], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        // columns per head: S0 [0,64), S1 [64,128), O [128,256)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(256u * HPC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // Q: two 64-column halves per head, 128 token rows
            mbar_expect_tx(q_full, HPC * Q_BYTES);
            for (int h = 0; h < HPC; ++h) {
                tma_load_2d(sQ + h * Q_BYTES, &map_q, (head0 + h) * FA_HD, tok0 + row0, q_full);
                tma_load_2d(sQ + h * Q_BYTES + Q_BYTES / 2, &map_q, (head0 + h) * FA_HD + 64, tok0 + row0, q_full);
            }
            int issued = 0;
            for (int j = 0; j < NP; ++j) {
                const int s = j % FA_STAGES;
                if (!mbar_wait(&kv_empty[s], ((j / FA_STAGES) & 1) ^ 1, abort_flag, 1)) break;
                const int page = ZLM_CHK(pages + page_lo + j, 4) ? pages[page_lo + j] : 0;
                const int krow = ((page * 2 + 0) * nkv + kvh) * ZLM_PAGE;
                const int vrow = ((page * 2 + 1) * nkv + kvh) * ZLM_PAGE;
                mbar_expect_tx(&kv_full[s], 2 * KV_BYTES);
                tma_load_2d(sK + s * KV_BYTES, &map_kv, 0, krow, &kv_full[s]);
                tma_load_2d(sK + s * KV_BYTES + KV_BYTES / 2, &map_kv, 64, krow, &kv_full[s]);
                tma_load_2d(sV + s * KV_BYTES, &map_kv, 0, vrow, &kv_full[s]);
                tma_load_2d(sV + s * KV_BYTES + KV_BYTES / 2, &map_kv, 64, vrow, &kv_full[s]);
                issued = j + 1;
            }
            if (*abort_flag) {
                mbar_drain(q_full, 0);
                for (int j = max(0, issued - FA_STAGES); j < issued; ++j)
                    mbar_drain(&kv_full[j % FA_STAGES], (j / FA_STAGES) & 1);
            }
        }
    } else if (warp <= HPC) {
        if (lane == 0) {
            const int h = warp - 1;             // the head this thread issues products for
            // S: M 128, N 64, both operands K-major.  O: M 128, N 128, A (P) K-major, B (V) MN-major.
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(ZLM_PAGE >> 3) << 17) | (8u << 24);
            const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(FA_HD >> 3) << 17) | (8u << 24);
            bool ok = mbar_wait(q_full, 0, abort_flag, 2);
            // Descriptors differ only in their start address (in units of 16 bytes, a 14-bit field
            // that never carries here), so they are built once and advanced by constants.
            const uint64_t qd = make_desc(smem_u32(sQ + h * Q_BYTES));
            const unsigned tmem_h = tmem_base + h * 256;
            auto issue_s = [&](int j) -> bool {
                const int s = j % FA_STAGES, sb = j & 1;
                if (!mbar_wait(&kv_full[s], (j / FA_STAGES) & 1, abort_flag, 2)) return false;
                if (!mbar_wait(&s_empty[h * 2 + sb], ((j >> 1) & 1) ^ 1, abort_flag, 5)) return false;
                tc_fence_after();
                const uint64_t kd = make_desc(smem_u32(sK + s * KV_BYTES));
#pragma unroll
                for (int ks = 0; ks < FA_HD / 16; ++ks) {
                    const unsigned qoff = ((ks >> 2) * (Q_BYTES / 2) + (ks & 3) * 32) >> 4;
                    const unsigned koff = ((ks >> 2) * (KV_BYTES / 2) + (ks & 3) * 32) >> 4;
                    tc_mma(tmem_h + sb * ZLM_PAGE, qd + qoff, kd + koff, idesc_s, ks != 0);
                }
                tc_commit(&s_full[h * 2 + sb]);
                return true;
            };
            if (ok && NP > 0) ok = issue_s(0);
            for (int j = 0; j < NP && ok; ++j) {
                if (j + 1 < NP) { ok = issue_s(j + 1); if (!ok) break; }
                const int s = j % FA_STAGES, sb = j & 1;
                ok = mbar_wait(&p_full[h * 2 + sb], (j >> 1) & 1, abort_flag, 6);
                if (!ok) break;
                tc_fence_after();
                // V tile: [64 keys][128 bytes] for dims 0..63, then the same for dims 64..127:
                // 16 keys a step = 2048 bytes; next 64 dims 8192 bytes on; 8-key groups 1024 bytes apart
                const uint64_t vd = make_desc_ex(smem_u32(sV + s * KV_BYTES), KV_BYTES / 2, 1024);
                const uint64_t pd = make_desc(smem_u32(sP + (h * 2 + sb) * P_BYTES));
#pragma unroll
                for (int kk = 0; kk < ZLM_PAGE / 16; ++kk)
                    tc_mma(tmem_h + 128, pd + ((kk * 32) >> 4), vd + ((kk * 2048) >> 4), idesc_o, (j | kk) != 0);
                tc_commit(&pv_done[h]);
                tc_commit(&kv_empty[s]);           // one arrival per head: the page is free when all have retired
            }
            if (!ok) {
                tc_commit(&s_full[h * 2]);
                tc_commit(&s_full[h * 2 + 1]);
                tc_commit(&pv_done[h]);
            }
        }
    } else {
        const int hh = (warp - 1 - HPC) >> 2;           // which of the block's heads this warp serves
        const int head = head0 + hh;
        uint64_t* const s_full_h = s_full + hh * 2;
        uint64_t* const s_empty_h = s_empty + hh * 2;
        uint64_t* const p_full_h = p_full + hh * 2;
        uint64_t* const pv_done_h = pv_done + hh;
        const unsigned tmem_s = tmem_base + hh * 256, tmem_o = tmem_base + hh * 256 + 128;
        unsigned char* const sP_h = sP + hh * 2 * P_BYTES;
        const int lg = warp & 3;
        const int i = lg * 32 + lane;                   // row of the tile = lane of tensor memory
        const bool row_ok = i < rows;
        const int pos = start + row0 + i;
        const int lo = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
        const unsigned lane_addr = (unsigned)(lg * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < NP; ++j) {
            const int sb = j & 1;
            ok = mbar_wait(&s_full_h[sb], (j >> 1) & 1, abort_flag, 3);
            tc_fence_after();
            if (!ok || *abort_flag) { ok = false; break; }
            float sv[ZLM_PAGE];
#pragma unroll
            for (int c = 0; c < ZLM_PAGE; c += 16) tc_ld16_nowait(tmem_s + lane_addr + sb * ZLM_PAGE + c, sv + c);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty_h[sb]);          // S may be overwritten by page j + 2
            const int kbase = (page_lo + j) * ZLM_PAGE;
            float mx = -INFINITY;
            // a page that every row of the tile sees whole needs no mask (block-uniform test)
            const bool inner = rows == FA_BM && kbase + ZLM_PAGE - 1 <= first_pos &&
                               (window == 0 || kbase >= last_pos + 1 - window);
            // four independent chains: one warp per scheduler has no other warp to hide a chain's latency
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (inner) {
#pragma unroll
                for (int c = 0; c < ZLM_PAGE; ++c) {
                    sv[c] *= scale_log2;
                    mx4[c & 3] = fmaxf(mx4[c & 3], sv[c]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < ZLM_PAGE; ++c) {
                    const int key = kbase + c;
                    const bool vis = row_ok && key <= pos && key >= lo;
                    sv[c] = vis ? sv[c] * scale_log2 : -INFINITY;
                    mx4[c & 3] = fmaxf(mx4[c & 3], sv[c]);
                }
            }
            mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // lazy reference: move it only when the maximum grew by more than 2^8
            const bool grow = mx > m_ref + FA_RESCALE;              // also true for the first real maximum
            const float m_new = grow ? mx : m_ref;
            const float alpha = (grow && m_ref != -INFINITY) ? exp2f(m_ref - m_new) : 1.0f;
            const bool need_rescale = grow && m_ref != -INFINITY && j > 0;
            if (__any_sync(0xffffffffu, need_rescale)) {
                // O must be at rest: the product of page j-1 has retired (page j's cannot have been
                // issued, it waits for this warp)
                ok = mbar_wait(pv_done_h, (j - 1) & 1, abort_flag, 7);
                tc_fence_after();
                if (!ok) break;
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
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
            // P row -> shared memory, 128 bytes a row, 16-byte chunks swizzled by (row % 8)
            unsigned char* prow = sP_h + sb * P_BYTES + i * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = fa_ex2(sv[ch * 8 + e] - ref);          // 2^-inf = 0 for masked keys
                    ps4[e & 3] += p[e];
                }
                uint4 pk;
                pk.x = fa_pack(p[0], p[1]); pk.y = fa_pack(p[2], p[3]);
                pk.z = fa_pack(p[4], p[5]); pk.w = fa_pack(p[6], p[7]);
                *(uint4*)(prow + ((ch ^ (i & 7)) << 4)) = pk;
            }
            l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full_h[sb]);
        }
        // the last two products: this warp only knows that the third last has retired, and a
        // parity can tell two phases apart, not three; so wait for them one after the other
        if (ok && NP > 1) ok = mbar_wait(pv_done_h, (NP - 2) & 1, abort_flag, 8);
        if (ok && NP > 0) ok = mbar_wait(pv_done_h, (NP - 1) & 1, abort_flag, 8);
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
// and one head's softmax runs under the other's products: measured 1.46 times the throughput per
// head), but the blocks are then half as many and the longest twice as long.  The step takes about
// as long as the larger of its longest block (the last tile of the longest prompt) and its whole
// work spread over the SMs; the form for which that is smaller runs (2,048 tokens, 16 heads over
// 8: 40 us with one head per block, 50 with two; 32 over 8: 76 and 57).  Odd groups take one.
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
    const double pairs_cost = 2.0 / 1.46;                                   // a block of two heads, per page, against one head
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
    const size_t smem = (size_t)hpc * FA_BM * FA_HD * 2 + 2 * FA_STAGES * ZLM_PAGE * FA_HD * 2 +
                        (size_t)hpc * 2 * FA_BM * ZLM_PAGE * 2 + 1024 + 256;
#define ZLM_FA_LAUNCH(H)                                                                                          \
    {                                                                                                             \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                                                                             \
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
        zlm_launch(attention_prefill_tc_kernel<H>, dim3(R * tiles * (nq / H)), dim3(32 + 160 * H), smem, st, mq, mkv,    \
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
