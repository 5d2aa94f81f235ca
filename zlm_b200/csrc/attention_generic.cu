// Attention of packed query tokens over the paged cache, any head size up to 512,
// fp32 or bf16 storage, fp32 arithmetic.  One block per (query head, token); the
// keys are walked in chunks of 32 that are aligned to absolute positions and
// dealt round-robin to the 4 warps, so the order of every sum depends only on
// the query's own position and window, never on the batch or on how the
// sequence was cut into steps.
// Formula: s_t = (q . k_t) * scale, softmax over t in [t_start, pos],
// o = sum p_t v_t with a running maximum and sum
// (src/kernels/transformer/attention.zig:86-164); kv head = q head / group
// (:104-105); window start: seq = pos + 1, t_start = seq - w if w and seq > w
// (src/runtime/executor.zig:93-98).
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_PER_LANE 16   // head_dim <= 512

template <typename TA>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_generic_kernel(TA* __restrict__ out, int out_stride, const TA* __restrict__ q,
                         int q_stride, const TA* __restrict__ pool,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ token_pos, const int* __restrict__ token_slot,
                         int nq, int nkv, int hd, float scale, int window) {
    extern __shared__ float sm[];
    float* qs = sm;                         // [hd]
    float* accs = sm + hd;                  // [ATT_WARPS][hd]
    __shared__ float ms[ATT_WARPS], ls[ATT_WARPS];

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / (nq / nkv);
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4)) return;
    const int pos = token_pos[t];
    const int slot = token_slot[t];
    const int seq = pos + 1;
    const int t_start = (window != 0 && seq > window) ? seq - window : 0;
    const int* pages = block_table + (size_t)slot * table_stride;
    const size_t page_stride = (size_t)2 * nkv * ZLM_PAGE * hd;
    const size_t v_off = (size_t)nkv * ZLM_PAGE * hd;

    const TA* qp = q + (size_t)t * q_stride + (size_t)h * hd;
    if (!ZLM_CHK(qp, (size_t)hd * sizeof(TA)) ||
        !ZLM_CHK(out + (size_t)t * out_stride + (size_t)h * hd, (size_t)hd * sizeof(TA)))
        return;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) qs[e] = to_f32(qp[e]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_PER_LANE];
#pragma unroll
    for (int r = 0; r < ATT_MAX_PER_LANE; ++r) acc[r] = 0.f;

    const int c0 = t_start / 32, c1 = pos / 32;
    for (int c = c0 + ((warp - c0 % ATT_WARPS + ATT_WARPS) % ATT_WARPS); c <= c1; c += ATT_WARPS) {
        // chunk c holds keys [32c, 32c+32); chunk c belongs to warp c % ATT_WARPS
        const int key = c * 32 + lane;
        const bool valid = key >= t_start && key <= pos;
        if (!ZLM_CHK(pages + (c * 32) / ZLM_PAGE, 4)) continue;
        const int page = pages[(c * 32) / ZLM_PAGE];
        const TA* kbase = pool + (size_t)page * page_stride + (size_t)kvh * ZLM_PAGE * hd;
        // this head's 64 keys and 64 values of the page
        if (!ZLM_CHK(kbase, (size_t)ZLM_PAGE * hd * sizeof(TA)) || !ZLM_CHK(kbase + v_off, (size_t)ZLM_PAGE * hd * sizeof(TA)))
            continue;
        float s = -INFINITY;
        if (valid) {
            const TA* kr = kbase + (size_t)(key % ZLM_PAGE) * hd;
            float d = 0.f;
            for (int e = 0; e < hd; ++e) d = fmaf(qs[e], to_f32(kr[e]), d);
            s = d * scale;
        }
        const float cm = warp_max(s);          // the chunk holds at least one valid key
        const float mn = fmaxf(m, cm);
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - mn);
        const float p = valid ? expf(s - mn) : 0.f;
        l = l * alpha + warp_sum(p);
        m = mn;
#pragma unroll
        for (int r = 0; r < ATT_MAX_PER_LANE; ++r) acc[r] *= alpha;
        const TA* vbase = kbase + v_off;
        const int nvalid_hi = min(31, pos - c * 32);
        const int lo = max(0, t_start - c * 32);
        for (int jk = lo; jk <= nvalid_hi; ++jk) {
            const float pj = __shfl_sync(0xffffffffu, p, jk);
            const TA* vr = vbase + (size_t)((c * 32 + jk) % ZLM_PAGE) * hd;
#pragma unroll
            for (int r = 0; r < ATT_MAX_PER_LANE; ++r) {
                const int e = lane + 32 * r;
                if (e < hd) acc[r] = fmaf(pj, to_f32(vr[e]), acc[r]);
            }
        }
    }
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int r = 0; r < ATT_MAX_PER_LANE; ++r) {
        const int e = lane + 32 * r;
        if (e < hd) accs[warp * hd + e] = acc[r];
    }
    __syncthreads();
    // merge the warps in the fixed order 0..3
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, ms[w]);
    float L = 0.f;
    float f[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        f[w] = (ms[w] == -INFINITY) ? 0.f : expf(ms[w] - M);
        L += ls[w] * f[w];
    }
    const float invL = 1.0f / L;
    TA* op = out + (size_t)t * out_stride + (size_t)h * hd;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += accs[w * hd + e] * f[w];
        op[e] = from_f32<TA>(o * invL);
    }
}

extern "C" int zlm_attention_generic(void* out, int out_stride, const void* q, int q_stride,
                                     int dtype, const void* pool, const int* block_table,
                                     int table_stride, const int* token_pos,
                                     const int* token_slot, int T, int nq, int nkv, int hd,
                                     float scale, int window, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(hd > 0 && hd <= 32 * ATT_MAX_PER_LANE, "attention: head_dim=%d must be at most %d", hd,
                32 * ATT_MAX_PER_LANE);
    ZLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads over %d kv heads", nq, nkv);
    ZLM_REQUIRE(window >= 0, "attention: window=%d", window);
    ZLM_REQUIRE(nq <= 65535, "attention: more than 65535 query heads");
    dim3 grid(T, nq);
    const size_t smem = (size_t)(1 + ATT_WARPS) * hd * sizeof(float);
    zlm_count_launch();
    if (dtype == ZLM_DTYPE_F32)
        attention_generic_kernel<float><<<grid, ATT_WARPS * 32, smem, st>>>(
            (float*)out, out_stride, (const float*)q, q_stride, (const float*)pool, block_table,
            table_stride, token_pos, token_slot, nq, nkv, hd, scale, window);
    else if (dtype == ZLM_DTYPE_BF16)
        attention_generic_kernel<__nv_bfloat16><<<grid, ATT_WARPS * 32, smem, st>>>(
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)pool, block_table, table_stride, token_pos, token_slot, nq, nkv,
            hd, scale, window);
    else
        ZLM_REQUIRE(false, "attention: unsupported dtype %d", dtype);
    return zlm_check_launch("attention_generic");
}

ZLM_TRANSLATION_UNIT(attention_generic)
