// Per-head RMSNorm of q and k, rotary position encoding of q and k, and the write
// of k and v into the paged cache, in one pass over the fused qkv activations.
// Order as the reference: norm, then rotation, then the cache write; v is written
// as it is (src/architectures/impl/qwen3/block.zig:26-30,
// src/kernels/transformer/norm.zig:128-166, src/kernels/transformer/rope.zig:161-206,
// src/kernels/transformer/attention.zig:6-28).  All arithmetic in fp32.
#include "common.cuh"

#define ROPE_MAX_PER_LANE 16   // head_dim <= 512
#define ROPE_WARPS 4

// One block per token.  The token's rotation table (cos and sin of pos * inv_freq[i]) is
// computed once into shared memory and shared by all heads; then the warps take the
// heads in turn: heads 0..nq-1 are q, then nkv k heads, then nkv v heads.  NPL is the
// number of elements a lane holds (head_dim <= 32 * NPL).
template <typename TA, int NPL>
__global__ void __launch_bounds__(ROPE_WARPS * 32)
qk_norm_rope_write_kernel(
    TA* __restrict__ qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
    const float* __restrict__ inv_freq, int n_rot, const int* __restrict__ token_pos,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int table_stride,
    TA* __restrict__ pool, int nq, int nkv, int hd, int writes_kv, int heads_per_block) {
    extern __shared__ float sm[];
    const int ang = n_rot / 2, half = hd / 2;
    float* cs = sm;                       // [ang]
    float* sn = sm + ang;                 // [ang]
    float* bufs = sm + 2 * ang;           // [ROPE_WARPS][hd]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = blockIdx.x;
    pdl_launch_dependents();
    const int pos = token_pos[t];
    for (int i = tid; i < ang; i += ROPE_WARPS * 32) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        sn[i] = s;
    }
    __syncthreads();
    const int heads = nq + 2 * nkv;
    float* buf = bufs + warp * hd;
    int page = 0;
    if (writes_kv) page = block_table[(size_t)token_slot[t] * table_stride + pos / ZLM_PAGE];
    pdl_wait();             // the table above is the step's own; qkv comes from the kernel before
    const int j_end = min(heads, (int)(blockIdx.y + 1) * heads_per_block);
    for (int j = blockIdx.y * heads_per_block + warp; j < j_end; j += ROPE_WARPS) {
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
            if (e < hd) dst[e] = from_f32<TA>(v[r]);
        }
    }
}

template <typename TA, int NPL>
static void launch_rope(void* qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
                        const float* inv_freq, int n_rot, const int* token_pos, const int* token_slot,
                        const int* block_table, int table_stride, void* pool, int nq, int nkv, int hd,
                        int writes_kv, int T, cudaStream_t st) {
    const size_t smem = (size_t)(n_rot + ROPE_WARPS * hd) * sizeof(float);
    // a long step: one block per token does all heads and computes the token's rotation table
    // once; a short step (decode): blocks of 4 heads, so that the GPU has something to spread
    const int heads = nq + 2 * nkv;
    const int hpb = T >= 512 ? heads : ROPE_WARPS;
    dim3 grid(T, (heads + hpb - 1) / hpb);
    zlm_launch(qk_norm_rope_write_kernel<TA, NPL>, grid, dim3(ROPE_WARPS * 32), smem, st,
        (TA*)qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos, token_slot, block_table,
        table_stride, (TA*)pool, nq, nkv, hd, writes_kv, hpb);
}

template <typename TA>
static void dispatch_rope(int hd, void* qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
                          const float* inv_freq, int n_rot, const int* token_pos, const int* token_slot,
                          const int* block_table, int table_stride, void* pool, int nq, int nkv,
                          int writes_kv, int T, cudaStream_t st) {
#define ZLM_ROPE(N) launch_rope<TA, N>(qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos, \
                                       token_slot, block_table, table_stride, pool, nq, nkv, hd, writes_kv, T, st)
    if (hd <= 32) ZLM_ROPE(1);
    else if (hd <= 64) ZLM_ROPE(2);
    else if (hd <= 128) ZLM_ROPE(4);
    else if (hd <= 256) ZLM_ROPE(8);
    else ZLM_ROPE(16);
#undef ZLM_ROPE
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
    ZLM_REQUIRE(n_rot == 0 || inv_freq, "qk_norm_rope_write: the frequency table is missing");
    ZLM_REQUIRE(nq + 2 * nkv <= 65535 * ROPE_WARPS, "qk_norm_rope_write: too many heads");
    VecW qw{q_w, w_dtype}, kw{k_w, w_dtype};
    if (dtype == ZLM_DTYPE_F32)
        dispatch_rope<float>(hd, qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos, token_slot,
                             block_table, table_stride, pool, nq, nkv, writes_kv, T, st);
    else if (dtype == ZLM_DTYPE_BF16)
        dispatch_rope<__nv_bfloat16>(hd, qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos,
                                     token_slot, block_table, table_stride, pool, nq, nkv, writes_kv, T, st);
    else
        ZLM_REQUIRE(false, "qk_norm_rope_write: unsupported dtype %d", dtype);
    return zlm_check_launch("qk_norm_rope_write");
}
