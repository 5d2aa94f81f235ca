// The body of the q/k norm + rotation + cache write kernel as a function of a group of
// warps (see rope_kv.cu for what it computes; its kernel runs it with the block as the group).
#pragma once
#include "common.cuh"

#define ROPE_MAX_PER_LANE 16   // head_dim <= 512
#define ROPE_WARPS 4

// One block per token.  The token's rotation table (cos and sin of pos * inv_freq[i]) is
// computed once into shared memory and shared by all heads; then the warps take the
// heads in turn: heads 0..nq-1 are q, then nkv k heads, then nkv v heads.  NPL is the
// number of elements a lane holds (head_dim <= 32 * NPL).
// The work of one block of the kernel below, token t and head chunk `chunk`, by a group of
// ROPE_WARPS warps; `sm` holds n_rot + ROPE_WARPS * hd floats.
// NPL contiguous elements of a head (NPL = 2, 4 or 8) from or to 4-, 8-, 16- or 32-byte aligned memory
template <typename TA, int NPL> __device__ __forceinline__ void rope_load_vec(float* v, const TA* p) {
    if constexpr (sizeof(TA) == 4) {
        if constexpr (NPL == 2) { const float2 a = *(const float2*)p; v[0] = a.x; v[1] = a.y; }
        else {
#pragma unroll
            for (int i = 0; i < NPL; i += 4) {
                const float4 a = *(const float4*)(p + i);
                v[i] = a.x; v[i + 1] = a.y; v[i + 2] = a.z; v[i + 3] = a.w;
            }
        }
    } else {
        unsigned u[NPL / 2];
        if constexpr (NPL == 2) u[0] = *(const unsigned*)p;
        else if constexpr (NPL == 4) { const uint2 a = *(const uint2*)p; u[0] = a.x; u[1] = a.y; }
        else { const uint4 a = *(const uint4*)p; u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w; }
#pragma unroll
        for (int i = 0; i < NPL / 2; ++i) {
            v[2 * i] = __uint_as_float(u[i] << 16);
            v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
}
template <typename TA, int NPL> __device__ __forceinline__ void rope_store_vec(TA* p, const float* v) {
    if constexpr (sizeof(TA) == 4) {
        if constexpr (NPL == 2) *(float2*)p = make_float2(v[0], v[1]);
        else {
#pragma unroll
            for (int i = 0; i < NPL; i += 4) *(float4*)(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    } else {
        unsigned u[NPL / 2];
#pragma unroll
        for (int i = 0; i < NPL / 2; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            u[i] = *(unsigned*)&h;
        }
        if constexpr (NPL == 2) *(unsigned*)p = u[0];
        else if constexpr (NPL == 4) *(uint2*)p = make_uint2(u[0], u[1]);
        else *(uint4*)p = make_uint4(u[0], u[1], u[2], u[3]);
    }
}

// VEC: head_dim is exactly 32 * NPL and the rows are aligned for it: a lane holds NPL
// neighbouring elements (one vector load and store per head) and the rotation's partner,
// half a head away, is 16 lanes away (a shuffle); otherwise a lane holds every 32nd element
// and the partners meet in shared memory.
template <typename TA, int NPL, bool PDL, bool VEC = false>
__device__ __forceinline__ void qk_norm_rope_write_item(
    float* sm, const int tid, const GroupSync gs, const int t, const int chunk,
    TA* qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
    const float* inv_freq, int n_rot, const int* token_pos,
    const int* token_slot, const int* block_table, int table_stride,
    TA* pool, int nq, int nkv, int hd, int writes_kv, int heads_per_block) {
    const int ang = n_rot / 2, half = hd / 2;
    float* cs = sm;                       // [ang]
    float* sn = sm + ang;                 // [ang]
    float* bufs = sm + 2 * ang;           // [ROPE_WARPS][hd]
    const int lane = tid & 31, warp = tid >> 5;
    if (PDL) pdl_trigger();
    // bounds-check build: the step's integers and tables first (the same answer in every thread)
    if (!ZLM_CHK(token_pos + t, 4) || (ang > 0 && !ZLM_CHK(inv_freq, (size_t)ang * 4)) ||
        (writes_kv && !ZLM_CHK(token_slot + t, 4)))
        return;
    const int pos = token_pos[t];
    for (int i = tid; i < ang; i += ROPE_WARPS * 32) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        sn[i] = s;
    }
    gs.sync();
    const int heads = nq + 2 * nkv;
    float* buf = bufs + warp * hd;
    int page = 0;
    if (writes_kv) {
        const int* entry = block_table + (size_t)token_slot[t] * table_stride + pos / ZLM_PAGE;
        if (!ZLM_CHK(entry, 4)) return;
        page = *entry;
    }
    if (has_norm && (!ZLM_CHK(qw.p, (size_t)hd * (qw.dtype == ZLM_DTYPE_F32 ? 4 : 2)) ||
                     (nkv > 0 && !ZLM_CHK(kw.p, (size_t)hd * (kw.dtype == ZLM_DTYPE_F32 ? 4 : 2)))))
        return;
    if (!ZLM_CHK(qkv + (size_t)t * row_stride, (size_t)(nq + (writes_kv ? 2 : 1) * nkv) * hd * sizeof(TA))) return;
    if (PDL) pdl_wait();    // the table above is the step's own; qkv comes from the kernel before
    const int j_end = min(heads, (chunk + 1) * heads_per_block);
    if constexpr (VEC) {
        // a warp's heads one after the other, the loads of the next two already on their way
        // (a warp with one 256-byte load in flight at a time leaves the memory idle)
        const int j0 = chunk * heads_per_block + warp;
        const int j_stop = writes_kv ? j_end : min(j_end, nq + nkv);     // v is only ever copied to the cache
        TA* base = qkv + (size_t)t * row_stride + lane * NPL;
        float nxt[2][NPL];
#pragma unroll
        for (int a = 0; a < 2; ++a)
            if (j0 + a * ROPE_WARPS < j_stop) rope_load_vec<TA, NPL>(nxt[a], base + (size_t)(j0 + a * ROPE_WARPS) * hd);
        // what a lane needs of the token's rotation and of the norm weights is the same for every
        // head: into registers once (at many tokens this kernel is bound by its instructions)
        float rc[NPL], rs[NPL], wq[NPL], wk[NPL];
        const bool low = lane * NPL < half;              // a lane's elements are all in one half of the head
#pragma unroll
        for (int r = 0; r < NPL; ++r) {
            const int e = lane * NPL + r;
            const int i = low ? e : e - half;
            rc[r] = i < ang ? cs[i] : 1.f;
            rs[r] = i < ang ? sn[i] : 0.f;
            wq[r] = has_norm ? qw[e] : 1.f;
            wk[r] = (has_norm && nkv > 0) ? kw[e] : 1.f;
        }
        for (int j = j0; j < j_stop; j += ROPE_WARPS) {
            float v[NPL];
#pragma unroll
            for (int r = 0; r < NPL; ++r) { v[r] = nxt[0][r]; nxt[0][r] = nxt[1][r]; }
            if (j + 2 * ROPE_WARPS < j_stop) rope_load_vec<TA, NPL>(nxt[1], base + (size_t)(j + 2 * ROPE_WARPS) * hd);
            const int kind = j < nq ? 0 : (j < nq + nkv ? 1 : 2);
            if (kind != 2) {
                if (has_norm) {
                    float ss = 0.f;
#pragma unroll
                    for (int r = 0; r < NPL; ++r) ss = fmaf(v[r], v[r], ss);
                    ss = warp_sum(ss);
                    const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
                    for (int r = 0; r < NPL; ++r) v[r] = (v[r] * inv) * (kind == 0 ? wq[r] : wk[r]);
                }
                if (ang > 0) {
#pragma unroll
                    for (int r = 0; r < NPL; ++r) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[r], 16);
                        const int i = low ? lane * NPL + r : lane * NPL + r - half;
                        if (i < ang) {
                            const float x0 = low ? v[r] : other, x1 = low ? other : v[r];
                            v[r] = low ? (x0 * rc[r] - x1 * rs[r]) : (x0 * rs[r] + x1 * rc[r]);
                        }
                    }
                }
            }
            TA* dst;
            if (kind == 0 || !writes_kv) {
                dst = base + (size_t)j * hd;             // q (and k when nothing is written) in place
            } else {
                const int kvh = kind == 1 ? j - nq : j - nq - nkv;
                const size_t page_stride = (size_t)2 * nkv * ZLM_PAGE * hd;
                dst = pool + (size_t)page * page_stride + (size_t)(kind - 1) * nkv * ZLM_PAGE * hd +
                      ((size_t)kvh * ZLM_PAGE + (pos % ZLM_PAGE)) * hd + lane * NPL;
            }
            if (ZLM_CHK(dst, NPL * sizeof(TA))) rope_store_vec<TA, NPL>(dst, v);
        }
    } else {
    for (int j = chunk * heads_per_block + warp; j < j_end; j += ROPE_WARPS) {
        const int kind = j < nq ? 0 : (j < nq + nkv ? 1 : 2);
        if (kind == 2 && !writes_kv) break;     // v is only ever copied to the cache (warp-uniform)
        TA* src = qkv + (size_t)t * row_stride + (size_t)j * hd;
        float v[NPL];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < NPL; ++r) {
            const int e = lane + 32 * r;
            v[r] = e < hd ? to_f32(src[e]) : 0.f;
            ss = fmaf(v[r], v[r], ss);
        }
        if (kind != 2) {
            if (has_norm) {
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
                const VecW& w = kind == 0 ? qw : kw;
#pragma unroll
                for (int r = 0; r < NPL; ++r) {
                    const int e = lane + 32 * r;
                    if (e < hd) v[r] = (v[r] * inv) * w[e];
                }
            }
            if (ang > 0) {
                __syncwarp();
#pragma unroll
                for (int r = 0; r < NPL; ++r) {
                    const int e = lane + 32 * r;
                    if (e < hd) buf[e] = v[r];
                }
                __syncwarp();
#pragma unroll
                for (int r = 0; r < NPL; ++r) {
                    const int e = lane + 32 * r;
                    if (e < hd) {
                        const int i = e < half ? e : e - half;
                        if (i < ang) {
                            const float x0 = buf[i], x1 = buf[i + half];
                            v[r] = e < half ? (x0 * cs[i] - x1 * sn[i]) : (x0 * sn[i] + x1 * cs[i]);
                        }
                    }
                }
            }
        }
        TA* dst;
        if (kind == 0 || !writes_kv) {
            dst = src;                               // q (and k when nothing is written) in place
        } else {
            const int kvh = kind == 1 ? j - nq : j - nq - nkv;
            const size_t page_stride = (size_t)2 * nkv * ZLM_PAGE * hd;
            dst = pool + (size_t)page * page_stride + (size_t)(kind - 1) * nkv * ZLM_PAGE * hd +
                  ((size_t)kvh * ZLM_PAGE + (pos % ZLM_PAGE)) * hd;
        }
#pragma unroll
        for (int r = 0; r < NPL; ++r) {
            const int e = lane + 32 * r;
            if (e < hd && ZLM_CHK(dst + e, sizeof(TA))) dst[e] = from_f32<TA>(v[r]);
        }
    }
    }
}
