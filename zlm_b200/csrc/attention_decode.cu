// Decode attention over the paged bf16 cache: one query token per sequence, all
// query heads of a kv group share one pass over that group's keys and values.
//
// grid (token, kv head, split).  A block takes `per` consecutive pages of the
// sequence; a page (64 keys) is staged in shared memory with cp.async, two stages,
// the first two loads in flight together; each
// of the 4 warps takes 16 keys of the page: S = Q K^T and O += P V on the
// warp-level tensor cores (the group's heads are the rows of a 16-row tile), with
// an fp32 running maximum and sum per head.  The warps' partial results are
// merged in a fixed order; with more than one split the merged (max, sum, O) go
// to scratch and a second kernel combines the splits, again in a fixed order.
//
// Formula: s_t = (q . k_t) / sqrt(hd), softmax over t in [t_start, pos],
// o = sum p_t v_t (src/kernels/transformer/attention.zig:86-164); kv head =
// q head / group; window start as src/runtime/executor.zig:93-98.
#include "common.cuh"

#include "attn_common.cuh"

#define DEC_THREADS 128
#define DEC_WARPS 4

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const __nv_bfloat16* __restrict__ q,
                        int q_stride, const __nv_bfloat16* __restrict__ pool,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ token_pos, const int* __restrict__ token_slot, int nq, int nkv,
                        float scale_log2, int window, int splits, int per, float* __restrict__ part_o,
                        float* __restrict__ part_ml) {
    constexpr int KS = HD / 16;            // k-steps of Q K^T; pairs of output n-tiles of P V
    constexpr int CH = HD / 8;             // 16-byte chunks per row
    constexpr int TILE = ZLM_PAGE * HD;    // elements of one K or V page of one kv head
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Ks = (__nv_bfloat16*)smem_raw;          // [2][TILE]
    __nv_bfloat16* Vs = Ks + 2 * TILE;                     // [2][TILE]

    const int t = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, qd = lane & 3;
    const int G = nq / nkv;
    pdl_launch_dependents();
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

    pdl_wait();          // q and this step's keys and values come from the kernel before
    // the pages do not depend on q: start them now, they land while q is fetched
    auto load_page = [&](int p, int stage) {
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

    if (p_begin < p_end) load_page(p_begin, 0);
    dec_commit();
    if (p_begin + 1 < p_end) load_page(p_begin + 1, 1);
    dec_commit();
    // Q fragments: row i of the 16-row tile is head kvh*G + i (zero beyond the group)
    unsigned qf[KS][4];
    {
        const __nv_bfloat16* qt = q + (size_t)t * q_stride + (size_t)kvh * G * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
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
        __syncthreads();
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
        __syncthreads();                     // every warp is done with this stage
        if (p + 2 < p_end) load_page(p + 2, stage);
        dec_commit();
    }
    dec_wait<0>();
    __syncthreads();

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
    __syncthreads();
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
            out[(size_t)t * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(O / L);
        } else {
            const size_t pi = ((size_t)t * nq + head) * splits + split;
            part_o[pi * HD + d] = O;
            if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
}

// combines the splits of one (token, head) in the order 0 .. used-1: the maxima and sums
// of the splits are read by one thread each and reduced by the block, then every thread
// sums one output dimension over the splits (independent loads, one latency deep)
#define COMB_THREADS 128
#define COMB_MAX_SPLITS 1024
__global__ void __launch_bounds__(COMB_THREADS)
attention_decode_combine_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const float* __restrict__ part_o,
                                const float* __restrict__ part_ml, const int* __restrict__ token_pos, int nq,
                                int hd, int splits, int per, int window) {
    __shared__ float fs[COMB_MAX_SPLITS];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int pos = token_pos[t];
    const int t_start = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int pages = pos / ZLM_PAGE + 1 - t_start / ZLM_PAGE;
    const int used = min(splits, (pages + per - 1) / per);
    const size_t base = ((size_t)t * nq + head) * splits;
    float m = -INFINITY;
    for (int s = tid; s < used; s += COMB_THREADS) m = fmaxf(m, part_ml[(base + s) * 2]);
    const float M = block_max(m, red);
    float l = 0.f;
    for (int s = tid; s < used; s += COMB_THREADS) {
        const float ms = part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
        fs[s] = f;
        l += part_ml[(base + s) * 2 + 1] * f;
    }
    const float L = block_sum(l, red);        // fixed order for a given number of splits
    __syncthreads();
    const float inv = 1.0f / L;
    for (int d = tid; d < hd; d += COMB_THREADS) {
        float O = 0.f;
#pragma unroll 8
        for (int s = 0; s < used; ++s) O = fmaf(part_o[(base + s) * hd + d], fs[s], O);
        out[(size_t)t * out_stride + (size_t)head * hd + d] = __float2bfloat16_rn(O * inv);
    }
}

template <int HD>
static int launch_decode(__nv_bfloat16* out, int out_stride, const __nv_bfloat16* q, int q_stride,
                         const __nv_bfloat16* pool, const int* block_table, int table_stride,
                         const int* token_pos, const int* token_slot, int T, int nq, int nkv, float scale,
                         int window, int splits, int per, float* part_o, float* part_ml, cudaStream_t st) {
    const size_t stage_bytes = (size_t)4 * ZLM_PAGE * HD * sizeof(__nv_bfloat16);
    const size_t merge_bytes = (size_t)DEC_WARPS * 16 * (HD + 2) * sizeof(float);
    const size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    auto kern = attention_decode_kernel<HD>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            zlm_set_error("attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        attr_set = true;
    }
    dim3 grid(T, nkv, splits);
    const float scale_log2 = scale * 1.4426950408889634f;
    zlm_launch(kern, grid, dim3(DEC_THREADS), smem, st, out, out_stride, q, q_stride, pool, block_table, table_stride,
               token_pos, token_slot, nq, nkv, scale_log2, window, splits, per, part_o, part_ml);
    int rc = zlm_check_launch("attention_decode");
    if (rc) return rc;
    if (splits > 1) {
        zlm_launch(attention_decode_combine_kernel, dim3(T, nq), dim3(COMB_THREADS), 0, st, out, out_stride,
                   (const float*)part_o, (const float*)part_ml, token_pos, nq, HD, splits, per, window);
        rc = zlm_check_launch("attention_decode_combine");
    }
    return rc;
}

// 1 if this kernel takes the shape, 0 if the caller has to use the generic kernel
extern "C" int zlm_attention_decode_supported(int nq, int nkv, int hd) {
    return (nkv > 0 && nq % nkv == 0 && nq / nkv <= 16 && hd % 16 == 0 && hd >= 16 && hd <= 128) ? 1 : 0;
}

// every split takes `per` pages; splits * per pages must cover the longest sequence.
// scratch: part_o needs T*nq*splits*hd floats, part_ml T*nq*splits*2 floats (unused if splits == 1)
extern "C" int zlm_attention_decode(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                    const int* block_table, int table_stride, const int* token_pos,
                                    const int* token_slot, int T, int nq, int nkv, int hd, float scale,
                                    int window, int splits, int per, float* part_o, float* part_ml,
                                    cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(zlm_attention_decode_supported(nq, nkv, hd),
                "attention_decode: %d heads over %d kv heads of size %d is not a shape this kernel takes", nq, nkv, hd);
    ZLM_REQUIRE(splits >= 1 && splits <= COMB_MAX_SPLITS && nkv <= 65535 && per >= 1,
                "attention_decode: splits=%d (at most %d) of %d pages", splits, COMB_MAX_SPLITS, per);
    ZLM_REQUIRE(splits == 1 || (part_o && part_ml), "attention_decode: scratch missing for %d splits", splits);
    ZLM_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0), "attention_decode: q must be 4-byte aligned");
#define ZLM_DEC_CASE(H)                                                                                       \
    case H:                                                                                                   \
        return launch_decode<H>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,           \
                                (const __nv_bfloat16*)pool, block_table, table_stride, token_pos, token_slot, \
                                T, nq, nkv, scale, window, splits, per, part_o, part_ml, st);
    switch (hd) {
        ZLM_DEC_CASE(16) ZLM_DEC_CASE(32) ZLM_DEC_CASE(48) ZLM_DEC_CASE(64) ZLM_DEC_CASE(80) ZLM_DEC_CASE(96)
        ZLM_DEC_CASE(112) ZLM_DEC_CASE(128)
    }
#undef ZLM_DEC_CASE
    ZLM_REQUIRE(false, "attention_decode: head_dim=%d", hd);
}

// ---------------------------------------------------------------------------
// The same decode attention for callers that must not allocate (declared in
// zlm_no_alloc.h).  The split partials go to a fixed array that is part of the
// library's image on every GPU that loads it, instead of to scratch that the
// caller allocates.
// ---------------------------------------------------------------------------
#include "zlm_no_alloc.h"

static __device__ __align__(256) float g_decode_scratch[ZLM_NO_ALLOC_SCRATCH_FLOATS];

#define ZLM_MAX_DEVICES 64
static float* g_decode_scratch_ptr[ZLM_MAX_DEVICES];     // device address of the array, per device

extern "C" int zlm_attention_decode_static(void* out, int out_stride, const void* q, int q_stride,
                                           const void* pool, const int* block_table, int table_stride,
                                           const int* token_pos, const int* token_slot, int T, int nq,
                                           int nkv, int hd, float scale, int window, int splits, int per,
                                           cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && nq > 0 && hd > 0 && splits >= 1, "attention_decode_static: bad sizes T=%d nq=%d hd=%d splits=%d",
                T, nq, hd, splits);
    const unsigned long long need = (unsigned long long)T * nq * splits * ((unsigned long long)hd + 2);
    ZLM_REQUIRE(splits == 1 || need <= (unsigned long long)ZLM_NO_ALLOC_SCRATCH_FLOATS,
                "attention_decode_static: T*heads*splits*(head_dim+2) = %llu floats of split partials exceed the "
                "built-in scratch of %llu floats; use fewer splits or tokens, or zlm_attention_decode with your own scratch",
                need, (unsigned long long)ZLM_NO_ALLOC_SCRATCH_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= ZLM_MAX_DEVICES) {
        zlm_set_error("attention_decode_static: cannot tell the current device (%s)", cudaGetErrorString(e));
        return ZLM_ERR_CUDA;
    }
    if (!g_decode_scratch_ptr[dev]) {
        // once per device, with that device current: in host code the array's name is
        // only a handle; the address a kernel can use has to be asked for
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
        if (e != cudaSuccess || !p) {
            zlm_set_error("attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                          cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        g_decode_scratch_ptr[dev] = p;
    }
    float* part_o = g_decode_scratch_ptr[dev];
    float* part_ml = part_o + (size_t)T * nq * splits * hd;
    return zlm_attention_decode(out, out_stride, q, q_stride, pool, block_table, table_stride, token_pos,
                                token_slot, T, nq, nkv, hd, scale, window, splits, per, part_o, part_ml, st);
}
