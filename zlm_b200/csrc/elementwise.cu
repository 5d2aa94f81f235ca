// Embedding gather, RMSNorm over rows of the fp32 residual stream, and SwiGLU.
// Formulas: src/runtime/executor.zig:714-764 (row lookup, no scale),
// src/kernels/transformer/norm.zig:4-37 (eps inside the root, x*inv then *w),
// src/kernels/transformer/activation.zig:8-13 (g / (1 + e^-g) * u).
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>

// ---------------------------------------------------------------- error channel
static thread_local char g_err[512] = "";

void zlm_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int zlm_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        zlm_set_error("%s: %s", what, cudaGetErrorString(e));
        return ZLM_ERR_CUDA;
    }
    return ZLM_OK;
}

static int g_pdl = 0;
int zlm_pdl_enabled() { return g_pdl; }
// 1: launch the decode-path kernels with programmatic dependent launch; 0: plain stream order
extern "C" void zlm_set_pdl(int on) { g_pdl = on ? 1 : 0; }

extern "C" const char* zlm_last_error() { return g_err; }
extern "C" int zlm_page_tokens() { return ZLM_PAGE; }

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table,
                             const int* __restrict__ ids, int H, int V) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    pdl_wait();                 // the ids may be what the previous step's sampler wrote
    int id = ids[t];
    // ids are validated on the host; clamp so that a bad id can never read
    // outside the table
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const TW* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    if (sizeof(TW) == 2 && H % 8 == 0) {
        // 16-byte loads, two 16-byte stores
        for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
            const uint4 v = *(const uint4*)((const __nv_bfloat16*)row + c * 8);
            float4 lo, hi;
            lo.x = __uint_as_float(v.x << 16); lo.y = __uint_as_float(v.x & 0xffff0000u);
            lo.z = __uint_as_float(v.y << 16); lo.w = __uint_as_float(v.y & 0xffff0000u);
            hi.x = __uint_as_float(v.z << 16); hi.y = __uint_as_float(v.z & 0xffff0000u);
            hi.z = __uint_as_float(v.w << 16); hi.w = __uint_as_float(v.w & 0xffff0000u);
            *(float4*)(o + c * 8) = lo;
            *(float4*)(o + c * 8 + 4) = hi;
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int zlm_embed(float* out, const void* table, int table_dtype, const int* ids, int T,
                         int H, int V, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && H > 0 && V > 0, "embed: bad sizes T=%d H=%d V=%d", T, H, V);
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (table_dtype == ZLM_DTYPE_F32)
        zlm_launch(embed_kernel<float>, T, threads, 0, st, out, (const float*)table, ids, H, V);
    else if (table_dtype == ZLM_DTYPE_BF16)
        zlm_launch(embed_kernel<__nv_bfloat16>, T, threads, 0, st, out, (const __nv_bfloat16*)table, ids, H, V);
    else
        ZLM_REQUIRE(false, "embed: unsupported table dtype %d", table_dtype);
    return zlm_check_launch("embed");
}

// ---------------------------------------------------------------- rmsnorm
// one block per output row; rows[r] (optional) selects the input row.  The block
// size is a function of H alone, so the order of the sum never depends on the batch.
// With H a multiple of 4 every thread keeps its float4s in registers between the
// sum and the scaling, so the row is read once and the latency is one load deep.
#define NORM_MAX_V4 4
template <typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, VecW w,
                               const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float* xr = x + (size_t)src * H;
    pdl_wait();
    TO* o = out + (size_t)r * H;
    const int nv = H / 4;
    if (H % 4 == 0 && nv <= NORM_MAX_V4 * (int)blockDim.x) {
        float4 v[NORM_MAX_V4];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            v[j] = c < nv ? *(const float4*)(xr + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            s = fmaf(v[j].x, v[j].x, s); s = fmaf(v[j].y, v[j].y, s);
            s = fmaf(v[j].z, v[j].z, s); s = fmaf(v[j].w, v[j].w, s);
        }
        s = block_sum(s, red);
        const float inv = 1.0f / sqrtf(s / (float)H + eps);
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c < nv) {
                const int i = c * 4;
                o[i] = from_f32<TO>((v[j].x * inv) * w[i]);
                o[i + 1] = from_f32<TO>((v[j].y * inv) * w[i + 1]);
                o[i + 2] = from_f32<TO>((v[j].z * inv) * w[i + 2]);
                o[i + 3] = from_f32<TO>((v[j].w * inv) * w[i + 3]);
            }
        }
        return;
    }
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i];
        s = fmaf(v, v, s);
    }
    s = block_sum(s, red);
    const float inv = 1.0f / sqrtf(s / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>((xr[i] * inv) * w[i]);
}

extern "C" int zlm_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype,
                           const int* rows, int R, int H, float eps, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
    ZLM_REQUIRE(w_dtype == ZLM_DTYPE_F32 || w_dtype == ZLM_DTYPE_BF16, "rmsnorm: weight dtype %d", w_dtype);
    VecW vw{w, w_dtype};
    // 32-bit output (the 32-bit path): a function of H only, so that the order of the sum
    // never depends on the batch.  bf16 output: rows of a long step share an SM better
    // with 256 threads each; the difference is in the last bit of the sum.
    int threads = 128;
    while (threads < 1024 && threads * 4 < H) threads *= 2;
    if (out_dtype == ZLM_DTYPE_BF16 && R >= 512 && H % 4 == 0 && H <= 256 * 4 * NORM_MAX_V4 && threads > 256) threads = 256;
    if (out_dtype == ZLM_DTYPE_F32)
        zlm_launch(rmsnorm_kernel<float>, R, threads, 0, st, (float*)out, x, vw, rows, H, eps);
    else if (out_dtype == ZLM_DTYPE_BF16)
        zlm_launch(rmsnorm_kernel<__nv_bfloat16>, R, threads, 0, st, (__nv_bfloat16*)out, x, vw, rows, H, eps);
    else
        ZLM_REQUIRE(false, "rmsnorm: unsupported output dtype %d", out_dtype);
    return zlm_check_launch("rmsnorm");
}

// ---------------------------------------------------------------- swiglu
// gu is [T, 2I]: gate in columns [0, I), up in [I, 2I)
template <typename TA>
__global__ void swiglu_kernel(TA* __restrict__ out, const TA* __restrict__ gu, int T, int I) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)T * I;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n;
         e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / I;
        const int i = (int)(e - t * I);
        const float g = to_f32(gu[t * 2 * I + i]);
        const float u = to_f32(gu[t * 2 * I + I + i]);
        out[e] = from_f32<TA>((g / (1.0f + expf(-g))) * u);
    }
}

extern "C" int zlm_swiglu(void* out, const void* gu, int dtype, int T, int I, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && I > 0, "swiglu: bad sizes T=%d I=%d", T, I);
    const size_t n = (size_t)T * I;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(swiglu_kernel<float>, blocks, 256, 0, st, (float*)out, (const float*)gu, T, I);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(swiglu_kernel<__nv_bfloat16>, blocks, 256, 0, st, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, T, I);
    else
        ZLM_REQUIRE(false, "swiglu: unsupported dtype %d", dtype);
    return zlm_check_launch("swiglu");
}

