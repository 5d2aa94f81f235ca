// Per-head RMSNorm of q and k, rotary position encoding of q and k, and the write
// of k and v into the paged cache, in one pass over the fused qkv activations.
// Order as the reference: norm, then rotation, then the cache write; v is written
// as it is (src/architectures/impl/qwen3/block.zig:26-30,
// src/kernels/transformer/norm.zig:128-166, src/kernels/transformer/rope.zig:161-206,
// src/kernels/transformer/attention.zig:6-28).  All arithmetic in fp32.
#include "common.cuh"
#include "rope_kv.cuh"

template <typename TA, int NPL, bool VEC>
__global__ void __launch_bounds__(ROPE_WARPS * 32)
qk_norm_rope_write_kernel(
    TA* __restrict__ qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
    const float* __restrict__ inv_freq, int n_rot, const int* __restrict__ token_pos,
    const int* __restrict__ token_slot, const int* __restrict__ block_table, int table_stride,
    TA* __restrict__ pool, int nq, int nkv, int hd, int writes_kv, int heads_per_block,
    const float* __restrict__ shares, int ks, size_t share_elems) {
    extern __shared__ float sm[];
    if (shares) {
        // the projection still lies in shares (fp32 [ks][T][heads * hd], the cut of K that a few-token
        // product leaves): this block adds up its own heads of its token, rounds them as the
        // product's second kernel would, and goes on with what it has just written
        pdl_trigger();
        pdl_wait();
        const int heads = nq + 2 * nkv, width = heads * hd;
        const int e0 = blockIdx.y * heads_per_block * hd, e1 = min(width, e0 + heads_per_block * hd);
        const float* sr = shares + (size_t)blockIdx.x * width;
        TA* row = qkv + (size_t)blockIdx.x * row_stride;
        for (int e = e0 + threadIdx.x; e < e1; e += ROPE_WARPS * 32) {
            if (!ZLM_CHK(sr + e, 4) || !ZLM_CHK(sr + (size_t)(ks - 1) * share_elems + e, 4) || !ZLM_CHK(row + e, sizeof(TA))) continue;
            float sum = 0.f;
            for (int s = 0; s < ks; ++s) sum += sr[(size_t)s * share_elems + e];
            row[e] = from_f32<TA>(sum);
        }
        __syncthreads();
    }
    qk_norm_rope_write_item<TA, NPL, true, VEC>(sm, threadIdx.x, GroupSync{0, ROPE_WARPS * 32}, blockIdx.x, blockIdx.y,
                                                qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos,
                                                token_slot, block_table, table_stride, pool, nq, nkv, hd, writes_kv,
                                                heads_per_block);
}

template <typename TA, int NPL, bool VEC>
static void launch_rope(void* qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
                        const float* inv_freq, int n_rot, const int* token_pos, const int* token_slot,
                        const int* block_table, int table_stride, void* pool, int nq, int nkv, int hd,
                        int writes_kv, int T, const float* shares, int ks, cudaStream_t st) {
    const size_t smem = (size_t)(n_rot + ROPE_WARPS * hd) * sizeof(float);
    // a long step: one block per token does all heads and computes the token's rotation table
    // once; a short step (decode): blocks of 4 heads, so that the GPU has something to spread
    const int heads = nq + 2 * nkv;
    const int hpb = T >= 512 ? heads : ROPE_WARPS;
    const size_t share_elems = (size_t)T * heads * hd;
    dim3 grid(T, (heads + hpb - 1) / hpb);
    zlm_launch(qk_norm_rope_write_kernel<TA, NPL, VEC>, grid, dim3(ROPE_WARPS * 32), smem, st,
        (TA*)qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos, token_slot, block_table,
        table_stride, (TA*)pool, nq, nkv, hd, writes_kv, hpb, shares, ks, share_elems);
}

// 1 if the vector form takes these heads: head_dim 64, 128 or 256 and rows (and the pool) aligned
// for a lane's head_dim / 32 elements
extern "C" int zlm_rope_vector_form(int hd, int elem_bytes, int row_stride, const void* qkv, const void* pool) {
    if (hd != 64 && hd != 128 && hd != 256) return 0;
    const size_t bytes = (size_t)(hd / 32) * elem_bytes;
    return ((uintptr_t)qkv % bytes == 0 && (uintptr_t)pool % bytes == 0 && ((size_t)row_stride * elem_bytes) % bytes == 0) ? 1 : 0;
}

template <typename TA>
static void dispatch_rope(int hd, void* qkv, int row_stride, VecW qw, VecW kw, int has_norm, float eps,
                          const float* inv_freq, int n_rot, const int* token_pos, const int* token_slot,
                          const int* block_table, int table_stride, void* pool, int nq, int nkv,
                          int writes_kv, int T, const float* shares, int ks, cudaStream_t st) {
#define ZLM_ROPE(N, V) launch_rope<TA, N, V>(qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos, \
                                             token_slot, block_table, table_stride, pool, nq, nkv, hd, writes_kv, T, shares, ks, st)
    if (zlm_rope_vector_form(hd, (int)sizeof(TA), row_stride, qkv, pool)) {
        if (hd == 64) ZLM_ROPE(2, true);
        else if (hd == 128) ZLM_ROPE(4, true);
        else ZLM_ROPE(8, true);
        return;
    }
    if (hd <= 32) ZLM_ROPE(1, false);
    else if (hd <= 64) ZLM_ROPE(2, false);
    else if (hd <= 128) ZLM_ROPE(4, false);
    else if (hd <= 256) ZLM_ROPE(8, false);
    else ZLM_ROPE(16, false);
#undef ZLM_ROPE
}

// With `shares` (fp32 [ks][T][(nq + 2 nkv) hd], what zlm_gemm_tc_shares left of the projection) the
// kernel first adds them up into qkv, each block its own heads; without, qkv holds the projection.
static int rope_entry(void* qkv, int dtype, int row_stride, const void* q_w,
                      const void* k_w, int w_dtype, int has_norm, float eps,
                      const float* inv_freq, int n_rot, const int* token_pos,
                      const int* token_slot, const int* block_table,
                      int table_stride, void* pool, int nq, int nkv, int hd,
                      int writes_kv, int T, const float* shares, int ks, cudaStream_t st) {
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
                             block_table, table_stride, pool, nq, nkv, writes_kv, T, shares, ks, st);
    else if (dtype == ZLM_DTYPE_BF16)
        dispatch_rope<__nv_bfloat16>(hd, qkv, row_stride, qw, kw, has_norm, eps, inv_freq, n_rot, token_pos,
                                     token_slot, block_table, table_stride, pool, nq, nkv, writes_kv, T, shares, ks, st);
    else
        ZLM_REQUIRE(false, "qk_norm_rope_write: unsupported dtype %d", dtype);
    return zlm_check_launch("qk_norm_rope_write");
}

extern "C" int zlm_qk_norm_rope_write(void* qkv, int dtype, int row_stride, const void* q_w,
                                      const void* k_w, int w_dtype, int has_norm, float eps,
                                      const float* inv_freq, int n_rot, const int* token_pos,
                                      const int* token_slot, const int* block_table,
                                      int table_stride, void* pool, int nq, int nkv, int hd,
                                      int writes_kv, int T, cudaStream_t st) {
    return rope_entry(qkv, dtype, row_stride, q_w, k_w, w_dtype, has_norm, eps, inv_freq, n_rot, token_pos, token_slot,
                      block_table, table_stride, pool, nq, nkv, hd, writes_kv, T, nullptr, 0, st);
}
extern "C" int zlm_qk_norm_rope_write_shares(void* qkv, int dtype, int row_stride, const void* q_w,
                                             const void* k_w, int w_dtype, int has_norm, float eps,
                                             const float* inv_freq, int n_rot, const int* token_pos,
                                             const int* token_slot, const int* block_table,
                                             int table_stride, void* pool, int nq, int nkv, int hd,
                                             int writes_kv, int T, const float* shares, int ks, cudaStream_t st) {
    ZLM_REQUIRE(shares && ks > 1 && T < 512, "qk_norm_rope_write_shares: %d shares at %d tokens", ks, T);
    return rope_entry(qkv, dtype, row_stride, q_w, k_w, w_dtype, has_norm, eps, inv_freq, n_rot, token_pos, token_slot,
                      block_table, table_stride, pool, nq, nkv, hd, writes_kv, T, shares, ks, st);
}

ZLM_TRANSLATION_UNIT(rope_kv)
