// Prefill attention over the paged bf16 cache: tiles of 64 query tokens of one
// sequence and one query head attend the sequence's keys page by page (a page is
// the 64-key tile), with the keys and values of the step's own tokens already in
// the cache.  S = Q K^T and O += P V run on the warp-level tensor cores; the
// running maximum and sum of the softmax are fp32; pages are staged with cp.async,
// double buffered.  Causality and the window are bounds on the key index per
// query row, so a chunk of a prompt attends the earlier chunks exactly as a whole
// prompt would.
//
// Formula: s_t = (q . k_t) / sqrt(hd) for t in [t_start, pos], softmax, o = sum
// p_t v_t (src/kernels/transformer/attention.zig:86-164); per-row bound in block
// prefill: src/runtime/executor.zig:565-584; window start: :93-98.
#include "attn_common.cuh"

#define PRE_BM 64
#define PRE_WARPS 4
#define PRE_THREADS (PRE_WARPS * 32)

template <int HD>
__global__ void __launch_bounds__(PRE_THREADS)
attention_prefill_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const __nv_bfloat16* __restrict__ q,
                         int q_stride, const __nv_bfloat16* __restrict__ pool,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_start, int tiles_per_seq, int nq, int nkv,
                         float scale_log2, int window) {
    constexpr int KS = HD / 16;
    constexpr int CH = HD / 8;
    constexpr int TILE = ZLM_PAGE * HD;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Ks = (__nv_bfloat16*)smem_raw;          // [2][TILE]
    __nv_bfloat16* Vs = Ks + 2 * TILE;                     // [2][TILE]

    const int r = blockIdx.x / tiles_per_seq, b = blockIdx.x % tiles_per_seq;
    const int head = blockIdx.y;
    if (!ZLM_CHK(cu_seqlens + r, 8) || !ZLM_CHK(seq_start + r, 4) || !ZLM_CHK(seq_slot + r, 4)) return;   // block-uniform
    const int tok0 = cu_seqlens[r], n_new = cu_seqlens[r + 1] - tok0;
    const int row0 = b * PRE_BM;
    if (row0 >= n_new) return;
    const int rows = min(PRE_BM, n_new - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, qd = lane & 3;
    const int kvh = head / (nq / nkv);
    const int start = seq_start[r];
    const int* pages = block_table + (size_t)seq_slot[r] * table_stride;
    const size_t page_stride = (size_t)2 * nkv * TILE;
    const size_t v_off = (size_t)nkv * TILE;

    // positions of this thread's two rows; rows beyond the tile's tokens are idle
    const int i0 = warp * 16 + g, i1 = i0 + 8;
    bool ok0 = i0 < rows, ok1 = i1 < rows;
#ifdef ZLM_BOUNDS_CHECK
    // a row whose query or output lies outside the tensors passed is treated as idle
    ok0 = ok0 && ZLM_CHK(q + (size_t)(tok0 + row0 + i0) * q_stride + (size_t)head * HD, HD * 2) &&
          ZLM_CHK(out + (size_t)(tok0 + row0 + i0) * out_stride + (size_t)head * HD, HD * 2);
    ok1 = ok1 && ZLM_CHK(q + (size_t)(tok0 + row0 + i1) * q_stride + (size_t)head * HD, HD * 2) &&
          ZLM_CHK(out + (size_t)(tok0 + row0 + i1) * out_stride + (size_t)head * HD, HD * 2);
#endif
    const int pos0 = start + row0 + i0, pos1 = start + row0 + i1;
    const int lo0 = (window != 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int lo1 = (window != 0 && pos1 + 1 > window) ? pos1 + 1 - window : 0;
    // keys the block and this warp can need
    const int blk_first = start + row0, blk_last = start + row0 + rows - 1;
    const int blk_lo = (window != 0 && blk_first + 1 > window) ? blk_first + 1 - window : 0;
    const int page_lo = blk_lo / ZLM_PAGE, page_hi = blk_last / ZLM_PAGE + 1;
    const int w_first = start + row0 + warp * 16;
    const int w_last = min(blk_last, w_first + 15);
    const int w_lo = (window != 0 && w_first + 1 > window) ? w_first + 1 - window : 0;
    const bool warp_idle = warp * 16 >= rows;

    unsigned qf[KS][4];
    {
        const __nv_bfloat16* q0 = q + (size_t)(tok0 + row0 + i0) * q_stride + (size_t)head * HD;
        const __nv_bfloat16* q1 = q + (size_t)(tok0 + row0 + i1) * q_stride + (size_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 16 + qd * 2;
            qf[ks][0] = ok0 ? *(const unsigned*)(q0 + c) : 0u;
            qf[ks][1] = ok1 ? *(const unsigned*)(q1 + c) : 0u;
            qf[ks][2] = ok0 ? *(const unsigned*)(q0 + c + 8) : 0u;
            qf[ks][3] = ok1 ? *(const unsigned*)(q1 + c + 8) : 0u;
        }
    }
    float o[2 * KS][4];
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    auto load_page = [&](int p, int stage) {
        if (!ZLM_CHK(pages + p, 4)) return;
        const __nv_bfloat16* kb = pool + (size_t)pages[p] * page_stride + (size_t)kvh * TILE;
        const __nv_bfloat16* vb = kb + v_off;
        __nv_bfloat16* ks_ = Ks + stage * TILE;
        __nv_bfloat16* vs_ = Vs + stage * TILE;
        for (int id = tid; id < ZLM_PAGE * CH; id += PRE_THREADS) {
            const int rr = id / CH, c = id % CH;
            dec_cp_async16(ks_ + tile_off<HD>(rr, c), kb + rr * HD + c * 8);
            dec_cp_async16(vs_ + tile_off<HD>(rr, c), vb + rr * HD + c * 8);
        }
    };

    load_page(page_lo, 0);
    dec_commit();
    for (int p = page_lo; p < page_hi; ++p) {
        const int stage = (p - page_lo) & 1;
        dec_wait<0>();
        __syncthreads();
        if (p + 1 < page_hi) load_page(p + 1, stage ^ 1);
        dec_commit();
        const int kbase = p * ZLM_PAGE;
        if (warp_idle || kbase > w_last || kbase + ZLM_PAGE - 1 < w_lo) continue;   // warp-uniform
        const __nv_bfloat16* kt = Ks + stage * TILE;
        const __nv_bfloat16* vt = Vs + stage * TILE;

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {           // pairs of key tiles
                const int mi = lane >> 3;
                const int row = np * 16 + (mi >> 1) * 8 + (lane & 7);
                const int chunk = ks * 2 + (mi & 1);
                unsigned b00, b01, b10, b11;
                dec_ldsm4(b00, b01, b10, b11, kt + tile_off<HD>(row, chunk));
                dec_mma(s[2 * np], qf[ks], b00, b01);
                dec_mma(s[2 * np + 1], qf[ks], b10, b11);
            }
        }
        // scale, mask by each row's own bounds, running maximum
        const bool edge = kbase + ZLM_PAGE - 1 > w_first || kbase < ((window != 0) ? w_last + 1 - window : 0);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kbase + nt * 8 + qd * 2 + e;
                const bool a = !edge || (key <= pos0 && key >= lo0);
                const bool c = !edge || (key <= pos1 && key >= lo1);
                s[nt][e] = (a && ok0) ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][2 + e] = (c && ok1) ? s[nt][2 + e] * scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a row that has seen no key yet keeps max = -inf; use 0 as its reference
        const float r0 = mn0 == -INFINITY ? 0.f : mn0, r1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = m0 == -INFINITY ? 0.f : exp2f(m0 - r0);
        const float a1 = m1 == -INFINITY ? 0.f : exp2f(m1 - r1);
        m0 = mn0;
        m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nt][e] = exp2f(s[nt][e] - r0);             // exp2(-inf) = 0 for masked keys
                s[nt][2 + e] = exp2f(s[nt][2 + e] - r1);
                ps0 += s[nt][e];
                ps1 += s[nt][2 + e];
            }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int i = 0; i < 2 * KS; ++i) {
            o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {               // 16 keys at a time
            unsigned pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dn = 0; dn < KS; ++dn) {
                const int mi = lane >> 3;
                const int row = kk * 16 + (mi & 1) * 8 + (lane & 7);
                const int chunk = dn * 2 + (mi >> 1);
                unsigned b0, b1, b2, b3;
                dec_ldsm4t(b0, b1, b2, b3, vt + tile_off<HD>(row, chunk));
                dec_mma(o[2 * dn], pa, b0, b1);
                dec_mma(o[2 * dn + 1], pa, b2, b3);
            }
        }
    }
    dec_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = ok0 ? 1.0f / l0 : 0.f, inv1 = ok1 ? 1.0f / l1 : 0.f;
    __nv_bfloat16* o0 = out + (size_t)(tok0 + row0 + i0) * out_stride + (size_t)head * HD;
    __nv_bfloat16* o1 = out + (size_t)(tok0 + row0 + i1) * out_stride + (size_t)head * HD;
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
        const int d = i * 8 + qd * 2;
        if (ok0) *(unsigned*)(o0 + d) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (ok1) *(unsigned*)(o1 + d) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

template <int HD>
static int launch_prefill(__nv_bfloat16* out, int out_stride, const __nv_bfloat16* q, int q_stride,
                          const __nv_bfloat16* pool, const int* block_table, int table_stride,
                          const int* cu_seqlens, const int* seq_slot, const int* seq_start, int R, int max_new,
                          int nq, int nkv, float scale, int window, cudaStream_t st) {
    const size_t smem = (size_t)4 * ZLM_PAGE * HD * sizeof(__nv_bfloat16);
    auto kern = attention_prefill_kernel<HD>;
    static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            zlm_set_error("attention_prefill: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        attr_set = true;
    }
    const int tiles = (max_new + PRE_BM - 1) / PRE_BM;
    ZLM_REQUIRE((long long)R * tiles < 2147483647LL && nq <= 65535, "attention_prefill: too many tiles");
    dim3 grid(R * tiles, nq);
    kern<<<grid, PRE_THREADS, smem, st>>>(out, out_stride, q, q_stride, pool, block_table, table_stride, cu_seqlens,
                                         seq_slot, seq_start, tiles, nq, nkv, scale * 1.4426950408889634f, window);
    return zlm_check_launch("attention_prefill");
}

extern "C" int zlm_attention_prefill_supported(int nq, int nkv, int hd) {
    return (nkv > 0 && nq % nkv == 0 && hd % 16 == 0 && hd >= 16 && hd <= 128) ? 1 : 0;
}

// q tokens are packed by sequence: sequence r owns tokens cu_seqlens[r] .. cu_seqlens[r+1]-1 at positions
// seq_start[r] .. of slot seq_slot[r]; max_new is the largest token count of a sequence
extern "C" int zlm_attention_prefill(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                     const int* block_table, int table_stride, const int* cu_seqlens,
                                     const int* seq_slot, const int* seq_start, int R, int max_new, int nq,
                                     int nkv, int hd, float scale, int window, cudaStream_t st) {
    if (R == 0 || max_new == 0) return ZLM_OK;
    ZLM_REQUIRE(zlm_attention_prefill_supported(nq, nkv, hd),
                "attention_prefill: %d heads over %d kv heads of size %d is not a shape this kernel takes", nq, nkv, hd);
    ZLM_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 4 == 0) && ((uintptr_t)out % 4 == 0),
                "attention_prefill: q and out must be 4-byte aligned");
#define ZLM_PRE_CASE(H)                                                                                         \
    case H:                                                                                                     \
        return launch_prefill<H>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,            \
                                 (const __nv_bfloat16*)pool, block_table, table_stride, cu_seqlens, seq_slot,   \
                                 seq_start, R, max_new, nq, nkv, scale, window, st);
    switch (hd) {
        ZLM_PRE_CASE(16) ZLM_PRE_CASE(32) ZLM_PRE_CASE(48) ZLM_PRE_CASE(64) ZLM_PRE_CASE(80) ZLM_PRE_CASE(96)
        ZLM_PRE_CASE(112) ZLM_PRE_CASE(128)
    }
#undef ZLM_PRE_CASE
    ZLM_REQUIRE(false, "attention_prefill: head_dim=%d", hd);
}

ZLM_TRANSLATION_UNIT(attention_prefill)
