// Weight-streaming bf16 matrix-vector product for decode steps of up to 8 tokens:
// Y[t, n] = sum_k X[t, k] W[n, k].  Each warp owns ROWS rows of W and streams them
// once with 16-byte loads that bypass L1; the few activation rows stay in L1/L2.
// Products and sums are fp32; the warp reduction is a fixed butterfly.
// (src/kernels/linear/matvec/kernels/bfloat.zig:43-67: bf16 widened by a 16-bit
// shift, fp32 accumulate; src/gpu/kernels/shaders/matvec_bf16.comp:56-121: rows
// per group, lanes stride over K, subgroup reduction.)
#include "common.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

#define GEMV_WARPS 4

// MODE 0: Y bf16 = acc; MODE 1: Y fp32 += acc; MODE 2: Y fp32 = acc
template <int TT, int ROWS, int MODE>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_bf16_kernel(void* __restrict__ Y, const __nv_bfloat16* __restrict__ X,
                 const __nv_bfloat16* __restrict__ W, int T, int N, int K, int ldx, int ldy) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n0 = (blockIdx.x * GEMV_WARPS + warp) * ROWS;
    if (n0 >= N) return;
    float acc[ROWS][TT];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) acc[r][t] = 0.f;

    const __nv_bfloat16* wrow[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) wrow[r] = W + (size_t)min(n0 + r, N - 1) * K;

    for (int k = lane * 8; k < K; k += 32 * 8) {
        uint4 wv[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) wv[r] = ld_stream16(wrow[r] + k);
        float wf[ROWS][8];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) unpack8(wv[r], wf[r]);
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            if (t < T) {
                const uint4 xv = __ldg((const uint4*)(X + (size_t)t * ldx + k));
                float xf[8];
                unpack8(xv, xf);
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[r][t] = fmaf(wf[r][e], xf[e], acc[r][t]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) acc[r][t] = warp_sum(acc[r][t]);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int n = n0 + r;
            if (n >= N) continue;
#pragma unroll
            for (int t = 0; t < TT; ++t) {
                if (t >= T) continue;
                const size_t idx = (size_t)t * ldy + n;
                if (MODE == 0) ((__nv_bfloat16*)Y)[idx] = __float2bfloat16_rn(acc[r][t]);
                else if (MODE == 1) ((float*)Y)[idx] += acc[r][t];
                else ((float*)Y)[idx] = acc[r][t];
            }
        }
    }
}

template <int TT, int ROWS>
static int launch_gemv(void* Y, const __nv_bfloat16* X, const __nv_bfloat16* W, int T, int N, int K,
                       int ldx, int ldy, int mode, cudaStream_t st) {
    const int rows_per_block = GEMV_WARPS * ROWS;
    const int blocks = (N + rows_per_block - 1) / rows_per_block;
    if (mode == 0) gemv_bf16_kernel<TT, ROWS, 0><<<blocks, GEMV_WARPS * 32, 0, st>>>(Y, X, W, T, N, K, ldx, ldy);
    else if (mode == 1) gemv_bf16_kernel<TT, ROWS, 1><<<blocks, GEMV_WARPS * 32, 0, st>>>(Y, X, W, T, N, K, ldx, ldy);
    else gemv_bf16_kernel<TT, ROWS, 2><<<blocks, GEMV_WARPS * 32, 0, st>>>(Y, X, W, T, N, K, ldx, ldy);
    return zlm_check_launch("gemv_bf16");
}

extern "C" int zlm_gemv_bf16(void* Y, const void* X, const void* W, int T, int N, int K, int ldx,
                             int ldy, int mode, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && T <= 8, "gemv_bf16: takes 1 to 8 tokens, got %d", T);
    ZLM_REQUIRE(N > 0 && K > 0, "gemv_bf16: bad sizes N=%d K=%d", N, K);
    ZLM_REQUIRE(K % 8 == 0 && ldx % 8 == 0,
                "gemv_bf16: the inner size K=%d (row stride %d) must be a multiple of 8 for bf16 kernels", K, ldx);
    ZLM_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemv_bf16: operands must be 16-byte aligned");
    ZLM_REQUIRE(mode >= 0 && mode <= 2, "gemv_bf16: mode %d", mode);
    const __nv_bfloat16* x = (const __nv_bfloat16*)X;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    if (T == 1) return launch_gemv<1, 4>(Y, x, w, T, N, K, ldx, ldy, mode, st);
    if (T == 2) return launch_gemv<2, 4>(Y, x, w, T, N, K, ldx, ldy, mode, st);
    if (T <= 4) return launch_gemv<4, 4>(Y, x, w, T, N, K, ldx, ldy, mode, st);
    return launch_gemv<8, 2>(Y, x, w, T, N, K, ldx, ldy, mode, st);
}
