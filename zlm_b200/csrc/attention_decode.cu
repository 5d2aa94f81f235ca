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
#include "attention_decode.cuh"

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const __nv_bfloat16* __restrict__ q,
                        int q_stride, const __nv_bfloat16* __restrict__ pool,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ token_pos, const int* __restrict__ token_slot, int nq, int nkv,
                        float scale_log2, int window, int splits, int per, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int fresh) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    attention_decode_item<HD, true>(smem_raw, threadIdx.x, GroupSync{0, DEC_THREADS}, blockIdx.x, blockIdx.y,
                                    blockIdx.z, out, out_stride, q, q_stride, pool, block_table, table_stride,
                                    token_pos, token_slot, nq, nkv, scale_log2, window, splits, per, part_o, part_ml, fresh);
}

__global__ void __launch_bounds__(COMB_THREADS)
attention_decode_combine_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const float* __restrict__ part_o,
                                const float* __restrict__ part_ml, const int* __restrict__ token_pos, int nq,
                                int hd, int splits, int per, int window) {
    __shared__ float fs[COMB_MAX_SPLITS];
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    attention_decode_combine_item(fs, red, threadIdx.x, GroupSync{0, COMB_THREADS}, blockIdx.x, blockIdx.y, out,
                                  out_stride, part_o, part_ml, token_pos, nq, hd, splits, per, window);
}

template <int HD>
static int launch_decode(__nv_bfloat16* out, int out_stride, const __nv_bfloat16* q, int q_stride,
                         const __nv_bfloat16* pool, const int* block_table, int table_stride,
                         const int* token_pos, const int* token_slot, int T, int nq, int nkv, float scale,
                         int window, int splits, int per, float* part_o, float* part_ml, int fresh, cudaStream_t st) {
    const size_t stage_bytes = (size_t)4 * ZLM_PAGE * HD * sizeof(__nv_bfloat16);
    const size_t merge_bytes = (size_t)DEC_WARPS * 16 * (HD + 2) * sizeof(float);
    const size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    auto kern = attention_decode_kernel<HD>;
    static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];
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
               token_pos, token_slot, nq, nkv, scale_log2, window, splits, per, part_o, part_ml, fresh);
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
// scratch: part_o needs T*nq*splits*hd floats, part_ml T*nq*splits*2 floats (unused if splits == 1).
// fresh: how many of each sequence's newest positions the kernels of this step may have written
// (1 for a decode step); pages that hold older positions only are read before the wait for the
// kernel before this one.  0: not known, nothing is read early.
extern "C" int zlm_attention_decode_fresh(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                          const int* block_table, int table_stride, const int* token_pos,
                                          const int* token_slot, int T, int nq, int nkv, int hd, float scale,
                                          int window, int splits, int per, float* part_o, float* part_ml,
                                          int fresh, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(zlm_attention_decode_supported(nq, nkv, hd),
                "attention_decode: %d heads over %d kv heads of size %d is not a shape this kernel takes", nq, nkv, hd);
    ZLM_REQUIRE(splits >= 1 && splits <= COMB_MAX_SPLITS && nkv <= 65535 && per >= 1,
                "attention_decode: splits=%d (at most %d) of %d pages", splits, COMB_MAX_SPLITS, per);
    ZLM_REQUIRE(splits == 1 || (part_o && part_ml), "attention_decode: scratch missing for %d splits", splits);
    ZLM_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0), "attention_decode: q must be 4-byte aligned");
    ZLM_REQUIRE(fresh >= 0, "attention_decode: fresh=%d", fresh);
#define ZLM_DEC_CASE(H)                                                                                       \
    case H:                                                                                                   \
        return launch_decode<H>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,           \
                                (const __nv_bfloat16*)pool, block_table, table_stride, token_pos, token_slot, \
                                T, nq, nkv, scale, window, splits, per, part_o, part_ml, fresh, st);
    switch (hd) {
        ZLM_DEC_CASE(16) ZLM_DEC_CASE(32) ZLM_DEC_CASE(48) ZLM_DEC_CASE(64) ZLM_DEC_CASE(80) ZLM_DEC_CASE(96)
        ZLM_DEC_CASE(112) ZLM_DEC_CASE(128)
    }
#undef ZLM_DEC_CASE
    ZLM_REQUIRE(false, "attention_decode: head_dim=%d", hd);
}

extern "C" int zlm_attention_decode(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                    const int* block_table, int table_stride, const int* token_pos,
                                    const int* token_slot, int T, int nq, int nkv, int hd, float scale,
                                    int window, int splits, int per, float* part_o, float* part_ml,
                                    cudaStream_t st) {
    return zlm_attention_decode_fresh(out, out_stride, q, q_stride, pool, block_table, table_stride, token_pos,
                                      token_slot, T, nq, nkv, hd, scale, window, splits, per, part_o, part_ml, 0, st);
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
    // one split needs no partials: nothing to look up, and the call may then be a device's first
    // even inside a stream capture
    if (splits > 1 && !g_decode_scratch_ptr[dev]) {
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
    float* part_o = splits > 1 ? g_decode_scratch_ptr[dev] : nullptr;
    float* part_ml = splits > 1 ? part_o + (size_t)T * nq * splits * hd : nullptr;
    return zlm_attention_decode(out, out_stride, q, q_stride, pool, block_table, table_stride, token_pos,
                                token_slot, T, nq, nkv, hd, scale, window, splits, per, part_o, part_ml, st);
}

ZLM_TRANSLATION_UNIT(attention_decode)
