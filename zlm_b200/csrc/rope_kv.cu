// Per-head RMSNorm of q and k, rotary position encoding of q and k, and the write
// of k and v into the paged cache, in one pass over the fused qkv activations.
// Order as the reference: norm, then rotation, then the cache write; v is written
// as it is (src/architectures/impl/qwen3/block.zig:26-30,
// src/kernels/transformer/norm.zig:128-166, src/kernels/transformer/rope.zig:161-206,
// src/kernels/transformer/attention.zig:6-28).  All arithmetic in fp32.
#include "common.cuh"

#define ROPE_MAX_PER_LANE 16   // head_dim <= 512

// one warp per (token, head); heads 0..nq-1 are q, then nkv k heads, then nkv v heads
template <typename TA>
__global__ void qk_norm_rope_write_kernel(
    TA* __restrict__ qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
    const float* __restrict__ inv_freq, int n_rot, const int* __restrict__ token_pos,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int table_stride,
    TA* __restrict__ pool, int nq, int nkv, int hd, int writes_kv, int T) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x, wy = threadIdx.y;
    const int heads = nq + 2 * nkv;
    const long long item = (long long)blockIdx.x * blockDim.y + wy;
    if (item >= (long long)T * heads) return;
    const int t = (int)(item / heads);
    const int j = (int)(item - (long long)t * heads);
    const int kind = j < nq ? 0 : (j < nq + nkv ? 1 : 2);
    if (kind == 2 && !writes_kv) return;     // v is only ever copied to the cache
    float* buf = sm + wy * hd;
    TA* src = qkv + (size_t)t * row_stride + (size_t)j * hd;
    const int pos = token_pos[t];

    float v[ROPE_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < ROPE_MAX_PER_LANE; ++r) {
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
            for (int r = 0; r < ROPE_MAX_PER_LANE; ++r) {
                const int e = lane + 32 * r;
                if (e < hd) v[r] = (v[r] * inv) * w[e];
            }
        }
        if (n_rot > 0) {
#pragma unroll
            for (int r = 0; r < ROPE_MAX_PER_LANE; ++r) {
                const int e = lane + 32 * r;
                if (e < hd) buf[e] = v[r];
            }
            __syncwarp();
            const int half = hd / 2, ang = n_rot / 2;
#pragma unroll
            for (int r = 0; r < ROPE_MAX_PER_LANE; ++r) {
                const int e = lane + 32 * r;
                if (e < hd) {
                    const int i = e < half ? e : e - half;
                    if (i < ang) {
                        const float a = (float)pos * inv_freq[i];
                        float s, c;
                        sincosf(a, &s, &c);
                        const float x0 = buf[i], x1 = buf[i + half];
                        v[r] = e < half ? (x0 * c - x1 * s) : (x0 * s + x1 * c);
                    }
                }
            }
        }
    }
    TA* dst;
    if (kind == 0 || !writes_kv) {
        dst = src;                               // q (and k when nothing is written) in place
    } else {
        const int slot = token_slot[t];
        const int page = block_table[(size_t)slot * table_stride + pos / ZLM_PAGE];
        const int kvh = kind == 1 ? j - nq : j - nq - nkv;
        const size_t page_stride = (size_t)2 * nkv * ZLM_PAGE * hd;
        dst = pool + (size_t)page * page_stride + (size_t)(kind - 1) * nkv * ZLM_PAGE * hd +
              ((size_t)kvh * ZLM_PAGE + (pos % ZLM_PAGE)) * hd;
    }
#pragma unroll
    for (int r = 0; r < ROPE_MAX_PER_LANE; ++r) {
        const int e = lane + 32 * r;
        if (e < hd) dst[e] = from_f32<TA>(v[r]);
    }
}

extern "C" int zlm_qk_norm_rope_write(void* qkv, int dtype, int row_stride, const void* q_w,
                                      const void* k_w, int w_dtype, int has_norm, float eps,
                                      const float* inv_freq, int n_rot, const int* token_pos,
                                      const int* token_slot, const int* block_table,
                                      int table_stride, void* pool, int nq, int nkv, int hd,
                                      int writes_kv, int T, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(hd > 0 && hd <= 32 * ROPE_MAX_PER_LANE && hd % 2 == 0,
                "qk_norm_rope_write: head_dim=%d must be even and at most %d", hd, 32 * ROPE_MAX_PER_LANE);
    ZLM_REQUIRE(n_rot >= 0 && n_rot <= hd && n_rot % 2 == 0, "qk_norm_rope_write: n_rot=%d with head_dim=%d", n_rot, hd);
    ZLM_REQUIRE(nq > 0 && nkv >= 0, "qk_norm_rope_write: bad head counts %d/%d", nq, nkv);
    ZLM_REQUIRE(!has_norm || (q_w && (k_w || nkv == 0)), "qk_norm_rope_write: norm weights missing");
    const int wpb = 4;
    const long long items = (long long)T * (nq + 2 * nkv);
    const long long blocks = (items + wpb - 1) / wpb;
    ZLM_REQUIRE(blocks < 2147483647LL, "qk_norm_rope_write: too many tokens");
    dim3 block(32, wpb);
    const size_t smem = (size_t)wpb * hd * sizeof(float);
    VecW qw{q_w, w_dtype}, kw{k_w, w_dtype};
    if (dtype == ZLM_DTYPE_F32)
        qk_norm_rope_write_kernel<float><<<(unsigned)blocks, block, smem, st>>>(
            (float*)qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos, token_slot,
            block_table, table_stride, (float*)pool, nq, nkv, hd, writes_kv, T);
    else if (dtype == ZLM_DTYPE_BF16)
        qk_norm_rope_write_kernel<__nv_bfloat16><<<(unsigned)blocks, block, smem, st>>>(
            (__nv_bfloat16*)qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos,
            token_slot, block_table, table_stride, (__nv_bfloat16*)pool, nq, nkv, hd, writes_kv, T);
    else
        ZLM_REQUIRE(false, "qk_norm_rope_write: unsupported dtype %d", dtype);
    return zlm_check_launch("qk_norm_rope_write");
}
