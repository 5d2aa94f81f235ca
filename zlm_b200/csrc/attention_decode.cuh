// The bodies of the decode attention kernels as functions of a group of warps (the kernels
// in attention_decode.cu run them with the block as the group).  What they compute is
// described in attention_decode.cu.
#pragma once
#include "common.cuh"
#include "attn_common.cuh"

#define DEC_THREADS 128
#define DEC_WARPS 4

// One (token, kv head, split) by a group of DEC_THREADS threads (`tid` counts inside the
// group, `gs` is its barrier, `smem_raw` its 4 * 64 * HD * 2 bytes of shared memory, 16-byte
// aligned).  PDL: the stand-alone kernel's launch hooks.
template <int HD, bool PDL>
__device__ __forceinline__ void attention_decode_item(
    unsigned char* smem_raw, const int tid, const GroupSync gs, const int t, const int kvh, const int split,
    __nv_bfloat16* out, int out_stride, const __nv_bfloat16* q, int q_stride, const __nv_bfloat16* pool,
    const int* block_table, int table_stride, const int* token_pos, const int* token_slot, int nq, int nkv,
    float scale_log2, int window, int splits, int per, float* part_o, float* part_ml, int fresh) {
    constexpr int KS = HD / 16;            // k-steps of Q K^T; pairs of output n-tiles of P V
    constexpr int CH = HD / 8;             // 16-byte chunks per row
    constexpr int TILE = ZLM_PAGE * HD;    // elements of one K or V page of one kv head
    __nv_bfloat16* Ks = (__nv_bfloat16*)smem_raw;          // [2][TILE]
    __nv_bfloat16* Vs = Ks + 2 * TILE;                     // [2][TILE]

    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, qd = lane & 3;
    const int G = nq / nkv;
    if (PDL) pdl_launch_dependents();
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4)) return;      // block-uniform
    const int pos = token_pos[t];
    const int slot = token_slot[t];
    const int seq = pos + 1;
    const int t_start = (window != 0 && seq > window) ? seq - window : 0;
    const int* pages = block_table + (size_t)slot * table_stride;
    const size_t page_stride = (size_t)2 * nkv * TILE;
    const size_t v_off = (size_t)nkv * TILE;

    // this split's pages
    const int page_lo = t_start / ZLM_PAGE, page_hi = pos / ZLM_PAGE + 1;
    const int p_begin = page_lo + split * per;
    const int p_end = min(page_hi, p_begin + per);
    if (p_begin >= p_end && splits > 1) return;      // the combine kernel skips this split too

    // q and this step's keys and values come from the kernel before; pages that hold only positions
    // from earlier steps do not, and their loads start before the wait for that kernel.  `fresh`
    // is how many of a sequence's newest positions this step may have written (0: not known,
    // nothing is read early).
    const int old_pages = fresh > 0 ? max(0, pos + 1 - fresh) / ZLM_PAGE : 0;
    const bool early0 = PDL && p_begin < p_end && p_begin < old_pages;
    const bool early1 = early0 && p_begin + 1 < p_end && p_begin + 1 < old_pages;
    auto load_page = [&](int p, int stage) {
        if (!ZLM_CHK(pages + p, 4)) return;
        const __nv_bfloat16* kb = pool + (size_t)pages[p] * page_stride + (size_t)kvh * TILE;
        const __nv_bfloat16* vb = kb + v_off;
        __nv_bfloat16* ks_ = Ks + stage * TILE;
        __nv_bfloat16* vs_ = Vs + stage * TILE;
        for (int id = tid; id < ZLM_PAGE * CH; id += DEC_THREADS) {
            const int r = id / CH, c = id % CH;
            dec_cp_async16(ks_ + tile_off<HD>(r, c), kb + r * HD + c * 8);
            dec_cp_async16(vs_ + tile_off<HD>(r, c), vb + r * HD + c * 8);
        }
    };

    if (early0) {
        load_page(p_begin, 0);
        dec_commit();
        if (early1) {
            load_page(p_begin + 1, 1);
            dec_commit();
        }
    }
    if (PDL) pdl_wait();
    // the other pages do not depend on q either: they land while q is fetched
    if (!early0) {
        if (p_begin < p_end) load_page(p_begin, 0);
        dec_commit();
    }
    if (!early1) {
        if (p_begin + 1 < p_end) load_page(p_begin + 1, 1);
        dec_commit();
    }
    // Q fragments: row i of the 16-row tile is head kvh*G + i (zero beyond the group)
    unsigned qf[KS][4] = {};
    {
        const __nv_bfloat16* qt = q + (size_t)t * q_stride + (size_t)kvh * G * HD;
        const bool q_ok = ZLM_CHK(qt, (size_t)G * HD * 2);
#pragma unroll
        for (int ks = 0; ks < KS && q_ok; ++ks) {
            const int c = ks * 16 + qd * 2;
            qf[ks][0] = g < G ? *(const unsigned*)(qt + (size_t)g * HD + c) : 0u;
            qf[ks][1] = g + 8 < G ? *(const unsigned*)(qt + (size_t)(g + 8) * HD + c) : 0u;
            qf[ks][2] = g < G ? *(const unsigned*)(qt + (size_t)g * HD + c + 8) : 0u;
            qf[ks][3] = g + 8 < G ? *(const unsigned*)(qt + (size_t)(g + 8) * HD + c + 8) : 0u;
        }
    }

    float o[2 * KS][4];
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) o[i][r] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g+8

    for (int p = p_begin; p < p_end; ++p) {
        const int stage = (p - p_begin) & 1;
        dec_wait<1>();                       // everything but the newest group has landed: page p is there
        gs.sync();
        const int kbase = p * ZLM_PAGE + warp * 16;
        const bool busy = !(kbase > pos || kbase + 15 < t_start);       // warp-uniform
        if (busy) {
        const __nv_bfloat16* kt = Ks + stage * TILE;
        const __nv_bfloat16* vt = Vs + stage * TILE;

        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int r = 0; r < 4; ++r) s[i][r] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int mi = lane >> 3;
            const int row = warp * 16 + (mi >> 1) * 8 + (lane & 7);
            const int chunk = ks * 2 + (mi & 1);
            unsigned b00, b01, b10, b11;
            dec_ldsm4(b00, b01, b10, b11, kt + tile_off<HD>(row, chunk));
            dec_mma(s[0], qf[ks], b00, b01);
            dec_mma(s[1], qf[ks], b10, b11);
        }
        // scale (to base-2 exponent) and mask by position
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kbase + nt * 8 + qd * 2 + e;
                const bool ok = key <= pos && key >= t_start;
                s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][2 + e] = ok ? s[nt][2 + e] * scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float a0 = m0 == -INFINITY ? 0.f : exp2f(m0 - mn0);
        const float a1 = m1 == -INFINITY ? 0.f : exp2f(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nt][e] = s[nt][e] == -INFINITY ? 0.f : exp2f(s[nt][e] - mn0);
                s[nt][2 + e] = s[nt][2 + e] == -INFINITY ? 0.f : exp2f(s[nt][2 + e] - mn1);
                ps0 += s[nt][e];
                ps1 += s[nt][2 + e];
            }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int i = 0; i < 2 * KS; ++i) {
            o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
        }
        unsigned pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dn = 0; dn < KS; ++dn) {
            const int mi = lane >> 3;
            const int row = warp * 16 + (mi & 1) * 8 + (lane & 7);
            const int chunk = dn * 2 + (mi >> 1);
            unsigned b0, b1, b2, b3;
            dec_ldsm4t(b0, b1, b2, b3, vt + tile_off<HD>(row, chunk));
            dec_mma(o[2 * dn], pa, b0, b1);
            dec_mma(o[2 * dn + 1], pa, b2, b3);
        }
        }
        gs.sync();                     // every warp is done with this stage
        if (p + 2 < p_end) load_page(p + 2, stage);
        dec_commit();
    }
    dec_wait<0>();
    gs.sync();

    // merge the 4 warps (fixed order), reusing the staging memory
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* so = (float*)smem_raw;                 // [DEC_WARPS][16][HD]
    float* sm_ = so + DEC_WARPS * 16 * HD;        // [DEC_WARPS][16]
    float* sl_ = sm_ + DEC_WARPS * 16;            // [DEC_WARPS][16]
    if (qd == 0) {
        sm_[warp * 16 + g] = m0; sm_[warp * 16 + g + 8] = m1;
        sl_[warp * 16 + g] = l0; sl_[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
        const int d = i * 8 + qd * 2;
        float* r0 = so + ((size_t)warp * 16 + g) * HD + d;
        float* r1 = so + ((size_t)warp * 16 + g + 8) * HD + d;
        r0[0] = o[i][0]; r0[1] = o[i][1];
        r1[0] = o[i][2]; r1[1] = o[i][3];
    }
    gs.sync();
    for (int idx = tid; idx < G * HD; idx += DEC_THREADS) {
        const int row = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_[w * 16 + row]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = sm_[w * 16 + row];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += sl_[w * 16 + row] * f;
            O += so[((size_t)w * 16 + row) * HD + d] * f;
        }
        const int head = kvh * G + row;
        if (splits == 1) {
            if (ZLM_CHK(out + (size_t)t * out_stride + (size_t)head * HD + d, 2))
                out[(size_t)t * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(O / L);
        } else {
            const size_t pi = ((size_t)t * nq + head) * splits + split;
            if (ZLM_CHK(part_o + pi * HD + d, 4)) part_o[pi * HD + d] = O;
            if (d == 0 && ZLM_CHK(part_ml + pi * 2, 8)) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
}

// combines the splits of one (token, head) in the order 0 .. used-1: the maxima and sums
// of the splits are read by one thread each and reduced by the block, then every thread
// sums one output dimension over the splits (independent loads, one latency deep)
#define COMB_THREADS 128
#define COMB_MAX_SPLITS 1024
// `fs` holds COMB_MAX_SPLITS floats, `red` 32
__device__ __forceinline__ void attention_decode_combine_item(
    float* fs, float* red, const int tid, const GroupSync gs, const int t, const int head, __nv_bfloat16* out,
    int out_stride, const float* part_o, const float* part_ml, const int* token_pos, int nq, int hd, int splits,
    int per, int window) {
    if (!ZLM_CHK(token_pos + t, 4)) return;
    const int pos = token_pos[t];
    const int t_start = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int pages = pos / ZLM_PAGE + 1 - t_start / ZLM_PAGE;
    const int used = min(splits, (pages + per - 1) / per);
    const size_t base = ((size_t)t * nq + head) * splits;
    if (!ZLM_CHK(part_ml + base * 2, (size_t)used * 8) || !ZLM_CHK(part_o + base * hd, (size_t)used * hd * 4) ||
        !ZLM_CHK(out + (size_t)t * out_stride + (size_t)head * hd, (size_t)hd * 2))
        return;
    float m = -INFINITY;
    for (int s = tid; s < used; s += COMB_THREADS) m = fmaxf(m, part_ml[(base + s) * 2]);
    const float M = group_max(m, red, tid, gs);
    float l = 0.f;
    for (int s = tid; s < used; s += COMB_THREADS) {
        const float ms = part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
        fs[s] = f;
        l += part_ml[(base + s) * 2 + 1] * f;
    }
    const float L = group_sum(l, red, tid, gs);        // fixed order for a given number of splits
    gs.sync();
    const float inv = 1.0f / L;
    for (int d = tid; d < hd; d += COMB_THREADS) {
        float O = 0.f;
#pragma unroll 8
        for (int s = 0; s < used; ++s) O = fmaf(part_o[(base + s) * hd + d], fs[s], O);
        out[(size_t)t * out_stride + (size_t)head * hd + d] = __float2bfloat16_rn(O * inv);
    }
}

