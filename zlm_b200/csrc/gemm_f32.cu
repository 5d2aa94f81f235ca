// True 32-bit matrix product Y[T,N] = X[T,K] . W[N,K]^T on the FFMA pipe: no
// tensor cores, no reduced-precision mode.  Every output element is one chain of
// FMAs over k = 0..K-1 in ascending order, so a token's result is bit-identical
// whatever the batch around it and however the step was cut.
// out_i = sum_j W[i,j] x_j with fp32 accumulation, row-major [out][in] weights
// (src/kernels/linear/matvec/kernels/float.zig:69-80).
#include "common.cuh"

#define F32_BM 64
#define F32_BN 64
#define F32_BK 16

// mode 0: Y = acc (fp32); mode 1: Y += acc (fp32 residual stream)
template <int MODE>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ Y, const float* __restrict__ X, const float* __restrict__ W,
                int T, int N, int K, int ldy) {
    __shared__ float Xs[F32_BK][F32_BM + 4];
    __shared__ float Ws[F32_BK][F32_BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * F32_BM, n0 = blockIdx.x * F32_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile: row = id / 16 (+16 per pass), k = id % 16
    const int lk = threadIdx.x & 15, lr = threadIdx.x >> 4;
    for (int k0 = 0; k0 < K; k0 += F32_BK) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int r = lr + 16 * p;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + lk;
            Xs[lk][r] = (gm < T && gk < K && ZLM_CHK(X + (size_t)gm * K + gk, 4)) ? X[(size_t)gm * K + gk] : 0.f;
            Ws[lk][r] = (gn < N && gk < K && ZLM_CHK(W + (size_t)gn * K + gk, 4)) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < F32_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N || !ZLM_CHK(Y + (size_t)gm * ldy + gn, 4)) continue;
            float* y = Y + (size_t)gm * ldy + gn;
            if (MODE == 0) *y = acc[i][j];
            else *y = *y + acc[i][j];
        }
    }
}

extern "C" int zlm_gemm_f32(float* Y, const float* X, const float* W, int T, int N, int K, int ldy,
                            int accumulate, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && N > 0 && K > 0 && ldy >= N, "gemm_f32: bad sizes T=%d N=%d K=%d ldy=%d", T, N, K, ldy);
    dim3 grid((N + F32_BN - 1) / F32_BN, (T + F32_BM - 1) / F32_BM);
    ZLM_REQUIRE(grid.y <= 65535, "gemm_f32: more than %d tokens in one step", 65535 * F32_BM);
    zlm_count_launch();
    if (accumulate) gemm_f32_kernel<1><<<grid, 256, 0, st>>>(Y, X, W, T, N, K, ldy);
    else gemm_f32_kernel<0><<<grid, 256, 0, st>>>(Y, X, W, T, N, K, ldy);
    return zlm_check_launch("gemm_f32");
}

ZLM_TRANSLATION_UNIT(gemm_f32)
