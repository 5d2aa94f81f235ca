// Embedding gather, RMSNorm over rows of the fp32 residual stream, and SwiGLU.
// Formulas: src/runtime/executor.zig:714-764 (row lookup, no scale),
// src/kernels/transformer/norm.zig:4-37 (eps inside the root, x*inv then *w),
// src/kernels/transformer/activation.zig:8-13 (g / (1 + e^-g) * u).
#include "common.cuh"
#include "elementwise.cuh"
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

static long long g_launches = 0;
void zlm_count_launch() { ++g_launches; }
// kernels launched by the library so far (also those captured into a graph: they are counted when captured)
extern "C" long long zlm_launch_count() { return g_launches; }
extern "C" const char* zlm_last_error() { return g_err; }
extern "C" int zlm_page_tokens() { return ZLM_PAGE; }

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table,
                             const int* __restrict__ ids, int H, int V) {
    pdl_trigger();
    const int t = blockIdx.x;
    pdl_wait();                 // the ids may be what the previous step's sampler wrote
    if (!ZLM_CHK(ids + t, 4) || !ZLM_CHK(out + (size_t)t * H, (size_t)H * 4)) return;
    embed_row(out + (size_t)t * H, table, ids[t], H, V, threadIdx.x, blockDim.x);
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
template <typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, VecW w,
                               const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    pdl_trigger();
    const int r = blockIdx.x;
    if (rows && !ZLM_CHK(rows + r, 4)) return;
    const int src = rows ? rows[r] : r;
    pdl_wait();
    if (!ZLM_CHK(x + (size_t)src * H, (size_t)H * 4) || !ZLM_CHK(out + (size_t)r * H, (size_t)H * sizeof(TO)) ||
        !ZLM_CHK(w.p, (size_t)H * (w.dtype == ZLM_DTYPE_F32 ? 4 : 2)))
        return;
    rmsnorm_row<TO, 1>(out + (size_t)r * H, x + (size_t)src * H, w, H, eps, red, threadIdx.x,
                       GroupSync{0, (int)blockDim.x}, blockDim.x);
}

// The same for a stream whose last product still lies in shares (fp32 [ks][R][H], the cut of K that
// a few-token product leaves): the row's block adds them in first, x[r] += (s0 + s1 + ...) as the
// product's own second kernel would, writes the row back, and norms it: one kernel instead of two.
template <typename TO>
__global__ void rmsnorm_shares_kernel(TO* __restrict__ out, float* __restrict__ x, VecW w,
                                      const float* __restrict__ shares, int ks, size_t share_elems, int H, float eps) {
    __shared__ float red[32];
    pdl_trigger();
    const int r = blockIdx.x;
    pdl_wait();
    float* xr = x + (size_t)r * H;
    const float* sr = shares + (size_t)r * H;
    if (!ZLM_CHK(xr, (size_t)H * 4) || !ZLM_CHK(out + (size_t)r * H, (size_t)H * sizeof(TO)) ||
        !ZLM_CHK(w.p, (size_t)H * (w.dtype == ZLM_DTYPE_F32 ? 4 : 2)) || !ZLM_CHK(sr, (size_t)H * 4) ||
        !ZLM_CHK(sr + (size_t)(ks - 1) * share_elems, (size_t)H * 4))
        return;
    if (H % 4 == 0) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < ks; ++s) {
                const float4 p = *(const float4*)(sr + (size_t)s * share_elems + i);
                sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
            }
            float4 a = *(const float4*)(xr + i);
            a.x += sum.x; a.y += sum.y; a.z += sum.z; a.w += sum.w;
            *(float4*)(xr + i) = a;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float sum = 0.f;
            for (int s = 0; s < ks; ++s) sum += sr[(size_t)s * share_elems + i];
            xr[i] += sum;
        }
    }
    __syncthreads();          // the row as the block has just written it
    rmsnorm_row<TO, 1>(out + (size_t)r * H, xr, w, H, eps, red, threadIdx.x, GroupSync{0, (int)blockDim.x}, blockDim.x);
}

// Many rows, bf16 output: a block of 256 threads walks rows r, r + gridDim.x, ... and has the
// next row's loads in flight while it reduces and stores the current one.  (One block per row,
// all blocks of a wave starting together, loads and then reduces in step across the whole GPU:
// the memory system idles while they reduce, 14 us for the 50 MB of 2,048 rows of 4,096.)
// The order of a row's sum depends on H alone.
#define NORM_ROWS_THREADS 256
template <int NV4>
__global__ void __launch_bounds__(NORM_ROWS_THREADS)
rmsnorm_rows_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ x, VecW w, int R, int H, float eps) {
    __shared__ float red[2][NORM_ROWS_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nv = H / 4;
    pdl_launch_dependents();
    float4 wv[NV4];
#pragma unroll
    for (int k = 0; k < NV4; ++k) {
        const int c = tid + k * NORM_ROWS_THREADS;
        wv[k] = (c < nv && ZLM_CHK((const char*)w.p + (size_t)c * 4 * (w.dtype == ZLM_DTYPE_F32 ? 4 : 2), 4 * (w.dtype == ZLM_DTYPE_F32 ? 4 : 2)))
                    ? w.load4(c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    auto load_row = [&](int r, float4* v) {
        const float* xr = x + (size_t)r * H;
#pragma unroll
        for (int k = 0; k < NV4; ++k) {
            const int c = tid + k * NORM_ROWS_THREADS;
            v[k] = (c < nv && ZLM_CHK(xr + c * 4, 16)) ? *(const float4*)(xr + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    float4 cur[NV4], nxt[NV4];
    int row = blockIdx.x;
    if (row < R) load_row(row, cur);
    for (int it = 0; row < R; row += gridDim.x, ++it) {
        const int nrow = row + gridDim.x;
        if (nrow < R) load_row(nrow, nxt);
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < NV4; ++k) {
            s = fmaf(cur[k].x, cur[k].x, s); s = fmaf(cur[k].y, cur[k].y, s);
            s = fmaf(cur[k].z, cur[k].z, s); s = fmaf(cur[k].w, cur[k].w, s);
        }
        s = warp_sum(s);
        float* rd = red[it & 1];            // two sets: the next row's partial sums do not wait for this row's readers
        if (lane == 0) rd[warp] = s;
        __syncthreads();
        float tot = lane < NORM_ROWS_THREADS / 32 ? rd[lane] : 0.f;
        tot = warp_sum(tot);
        const float inv = 1.0f / sqrtf(tot / (float)H + eps);
        __nv_bfloat16* o = out + (size_t)row * H;
#pragma unroll
        for (int k = 0; k < NV4; ++k) {
            const int c = tid + k * NORM_ROWS_THREADS;
            if (c < nv && ZLM_CHK(o + c * 4, 8))
                store4(o + c * 4, (cur[k].x * inv) * wv[k].x, (cur[k].y * inv) * wv[k].y, (cur[k].z * inv) * wv[k].z,
                       (cur[k].w * inv) * wv[k].w);
        }
#pragma unroll
        for (int k = 0; k < NV4; ++k) cur[k] = nxt[k];
    }
}

// threads of the block that norms one row.  32-bit output (the 32-bit path): a function of H
// only, so that the order of the sum never depends on the batch.  bf16 output: rows of a long
// step share an SM better with 256 threads each; the difference is in the last bit of the sum.
extern "C" int zlm_rmsnorm_threads(int out_dtype, int R, int H) {
    int threads = 128;
    while (threads < 1024 && threads * 4 < H) threads *= 2;
    if (out_dtype == ZLM_DTYPE_BF16 && R >= 512 && H % 4 == 0 && H <= 256 * 4 * NORM_MAX_V4 && threads > 256) threads = 256;
    return threads;
}

// 1 if a step of R rows of width H with bf16 output takes the row-walking kernel
extern "C" int zlm_rmsnorm_walks_rows(int out_dtype, int R, int H, int has_rows) {
    return (out_dtype == ZLM_DTYPE_BF16 && !has_rows && R >= 512 && H % 4 == 0 && H <= NORM_ROWS_THREADS * 4 * 8) ? 1 : 0;
}

extern "C" int zlm_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype,
                           const int* rows, int R, int H, float eps, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
    ZLM_REQUIRE(w_dtype == ZLM_DTYPE_F32 || w_dtype == ZLM_DTYPE_BF16, "rmsnorm: weight dtype %d", w_dtype);
    ZLM_REQUIRE(H % 4 != 0 || ((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0),
                "rmsnorm: input, weight and output must be 16-byte aligned");
    VecW vw{w, w_dtype};
    if (zlm_rmsnorm_walks_rows(out_dtype, R, H, rows != nullptr)) {
        static int sms = 0;
        if (!sms && (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, zlm_device_index()) != cudaSuccess || sms <= 0)) sms = 148;
        const int nv4 = (H / 4 + NORM_ROWS_THREADS - 1) / NORM_ROWS_THREADS;
        const int blocks = R < sms * 4 ? R : sms * 4;
        __nv_bfloat16* o = (__nv_bfloat16*)out;
        if (nv4 <= 1) zlm_launch(rmsnorm_rows_kernel<1>, blocks, NORM_ROWS_THREADS, 0, st, o, x, vw, R, H, eps);
        else if (nv4 <= 2) zlm_launch(rmsnorm_rows_kernel<2>, blocks, NORM_ROWS_THREADS, 0, st, o, x, vw, R, H, eps);
        else if (nv4 <= 4) zlm_launch(rmsnorm_rows_kernel<4>, blocks, NORM_ROWS_THREADS, 0, st, o, x, vw, R, H, eps);
        else zlm_launch(rmsnorm_rows_kernel<8>, blocks, NORM_ROWS_THREADS, 0, st, o, x, vw, R, H, eps);
        return zlm_check_launch("rmsnorm_rows");
    }
    const int threads = zlm_rmsnorm_threads(out_dtype, R, H);
    if (out_dtype == ZLM_DTYPE_F32)
        zlm_launch(rmsnorm_kernel<float>, R, threads, 0, st, (float*)out, x, vw, rows, H, eps);
    else if (out_dtype == ZLM_DTYPE_BF16)
        zlm_launch(rmsnorm_kernel<__nv_bfloat16>, R, threads, 0, st, (__nv_bfloat16*)out, x, vw, rows, H, eps);
    else
        ZLM_REQUIRE(false, "rmsnorm: unsupported output dtype %d", out_dtype);
    return zlm_check_launch("rmsnorm");
}

extern "C" int zlm_rmsnorm_shares(void* out, int out_dtype, float* x, const void* w, int w_dtype, int R, int H, float eps,
                                  const float* shares, int ks, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && H > 0 && ks > 1 && shares, "rmsnorm_shares: bad sizes R=%d H=%d shares=%d", R, H, ks);
    VecW vw{w, w_dtype};
    // the same block as zlm_rmsnorm takes for a short step, so that the row's sum has the same order
    int threads = 128;
    while (threads < 1024 && threads * 4 < H) threads *= 2;
    const size_t share_elems = (size_t)R * H;
    if (out_dtype == ZLM_DTYPE_F32)
        zlm_launch(rmsnorm_shares_kernel<float>, R, threads, 0, st, (float*)out, x, vw, shares, ks, share_elems, H, eps);
    else if (out_dtype == ZLM_DTYPE_BF16)
        zlm_launch(rmsnorm_shares_kernel<__nv_bfloat16>, R, threads, 0, st, (__nv_bfloat16*)out, x, vw, shares, ks, share_elems, H, eps);
    else
        ZLM_REQUIRE(false, "rmsnorm_shares: unsupported output dtype %d", out_dtype);
    return zlm_check_launch("rmsnorm_shares");
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
        if (!ZLM_CHK(&gu[t * 2 * I + i], sizeof(TA)) || !ZLM_CHK(&gu[t * 2 * I + I + i], sizeof(TA)) ||
            !ZLM_CHK(&out[e], sizeof(TA)))
            continue;
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


ZLM_TRANSLATION_UNIT(elementwise)
