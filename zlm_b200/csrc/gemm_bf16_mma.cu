// bf16 matrix product Y[T,N] = X[T,K] . W[N,K]^T with fp32 accumulation on the
// warp-level tensor-core path (mma.sync m16n8k16) behind a 4-stage cp.async
// pipeline.  This is the kernel that takes every shape (any T and N, K a multiple
// of 8); the tcgen05 kernel takes over the large aligned shapes.
// out_i = sum_j W[i,j] x_j, bf16 widened to fp32 products, fp32 sum
// (src/kernels/linear/matvec/kernels/bfloat.zig:43-67).
#include "common.cuh"

#define MMA_BK 32
#define MMA_PAD 8
#define MMA_LD (MMA_BK + MMA_PAD)
#define MMA_STAGES 4
#define MMA_THREADS 256

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = (valid && ZLM_CHK(gmem, 16)) ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                            const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MODE 0: Y bf16 = acc; MODE 1: Y fp32 += acc; MODE 2: Y fp32 = acc
template <int MODE>
__device__ __forceinline__ void store_out(void* Y, size_t idx, float v) {
    if (!ZLM_CHK((char*)Y + idx * (MODE == 0 ? 2 : 4), MODE == 0 ? 2 : 4)) return;
    if (MODE == 0) ((__nv_bfloat16*)Y)[idx] = __float2bfloat16_rn(v);
    else if (MODE == 1) ((float*)Y)[idx] += v;
    else if (MODE == 2) ((float*)Y)[idx] = v;
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int MODE>
__global__ void __launch_bounds__(MMA_THREADS)
gemm_bf16_mma_kernel(void* __restrict__ Y, const __nv_bfloat16* __restrict__ X,
                     const __nv_bfloat16* __restrict__ W, int T, int N, int K, int ldx, int ldy) {
    static_assert(WARPS_M * WARPS_N == MMA_THREADS / 32, "8 warps");
    constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    constexpr int MT = WM / 16, NT = WN / 8;
    static_assert(WM % 16 == 0 && WN % 16 == 0, "warp tile");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* As = (__nv_bfloat16*)smem_raw;                       // [STAGES][BM][LD]
    __nv_bfloat16* Bs = As + (size_t)MMA_STAGES * BM * MMA_LD;          // [STAGES][BN][LD]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WARPS_N, wn = warp % WARPS_N;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int KT = (K + MMA_BK - 1) / MMA_BK;

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;

    auto load_tile = [&](int kt, int stage) {
        const int k0 = kt * MMA_BK;
        __nv_bfloat16* a = As + (size_t)stage * BM * MMA_LD;
        __nv_bfloat16* b = Bs + (size_t)stage * BN * MMA_LD;
        for (int id = tid; id < BM * 4; id += MMA_THREADS) {
            const int r = id >> 2, c = (id & 3) * 8;
            const bool ok = (m0 + r < T) && (k0 + c < K);
            const __nv_bfloat16* src = ok ? X + (size_t)(m0 + r) * ldx + k0 + c : X;
            cp_async16(a + r * MMA_LD + c, src, ok);
        }
        for (int id = tid; id < BN * 4; id += MMA_THREADS) {
            const int r = id >> 2, c = (id & 3) * 8;
            const bool ok = (n0 + r < N) && (k0 + c < K);
            const __nv_bfloat16* src = ok ? W + (size_t)(n0 + r) * K + k0 + c : W;
            cp_async16(b + r * MMA_LD + c, src, ok);
        }
    };

#pragma unroll
    for (int s = 0; s < MMA_STAGES - 1; ++s) {
        if (s < KT) load_tile(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<MMA_STAGES - 2>();
        __syncthreads();
        const int nk = kt + MMA_STAGES - 1;
        if (nk < KT) load_tile(nk, nk % MMA_STAGES);
        cp_async_commit();
        const __nv_bfloat16* a = As + (size_t)(kt % MMA_STAGES) * BM * MMA_LD;
        const __nv_bfloat16* b = Bs + (size_t)(kt % MMA_STAGES) * BN * MMA_LD;
#pragma unroll
        for (int ks = 0; ks < MMA_BK; ks += 16) {
            unsigned af[MT][4];
            unsigned bf[NT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int r = wm * WM + i * 16 + (lane & 15);
                const int c = ks + (lane >> 4) * 8;
                ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], a + r * MMA_LD + c);
            }
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                const int mi = lane >> 3;
                const int r = wn * WN + j * 8 + (mi >> 1) * 8 + (lane & 7);
                const int c = ks + (mi & 1) * 8;
                ldmatrix_x4(bf[j][0], bf[j][1], bf[j + 1][0], bf[j + 1][1], b + r * MMA_LD + c);
            }
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_bf16(acc[i][j], af[i], bf[j][0], bf[j][1]);
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, q = lane & 3;
    if constexpr (MODE == 3) {
        // n-tiles come in pairs: 8 gate channels, then the 8 matching up channels
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int m = m0 + wm * WM + i * 16 + g + half * 8;
                if (m >= T) continue;
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    const int n = n0 + wn * WN + j * 8;              // first gate channel of the pair of tiles
                    if (n + 16 > N) continue;
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float gt = acc[i][j][half * 2 + e], up = acc[i][j + 1][half * 2 + e];
                        if (ZLM_CHK((__nv_bfloat16*)Y + (size_t)m * ldy + n / 2 + q * 2 + e, 2))
                            ((__nv_bfloat16*)Y)[(size_t)m * ldy + n / 2 + q * 2 + e] =
                                __float2bfloat16_rn((gt / (1.0f + expf(-gt))) * up);
                    }
                }
            }
    } else {
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + wm * WM + i * 16 + g + half * 8;
            if (m >= T) continue;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int n = n0 + wn * WN + j * 8 + q * 2;
                if (n < N) store_out<MODE>(Y, (size_t)m * ldy + n, acc[i][j][half * 2 + 0]);
                if (n + 1 < N) store_out<MODE>(Y, (size_t)m * ldy + n + 1, acc[i][j][half * 2 + 1]);
            }
        }
    }
    }
}

template <int BM, int BN, int WARPS_M, int WARPS_N>
static int launch_mma(void* Y, const __nv_bfloat16* X, const __nv_bfloat16* W, int T, int N, int K,
                      int ldx, int ldy, int mode, cudaStream_t st) {
    const size_t smem = (size_t)MMA_STAGES * (BM + BN) * MMA_LD * sizeof(__nv_bfloat16);
    dim3 grid((N + BN - 1) / BN, (T + BM - 1) / BM);
    ZLM_REQUIRE(grid.y <= 65535, "gemm_bf16: too many tokens in one step (%d)", T);
#define ZLM_LAUNCH_MODE(M)                                                                           \
    {                                                                                                \
        auto kern = gemm_bf16_mma_kernel<BM, BN, WARPS_M, WARPS_N, M>;                               \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                                                                \
        if (!attr_set) {                                                                             \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                 (int)smem);                                         \
            if (e != cudaSuccess) {                                                                  \
                zlm_set_error("gemm_bf16: cannot reserve %zu bytes of shared memory: %s", smem,      \
                              cudaGetErrorString(e));                                                \
                return ZLM_ERR_CUDA;                                                                 \
            }                                                                                        \
            attr_set = true;                                                                         \
        }                                                                                            \
        kern<<<grid, MMA_THREADS, smem, st>>>(Y, X, W, T, N, K, ldx, ldy);                           \
    }
    if (mode == 0) ZLM_LAUNCH_MODE(0)
    else if (mode == 1) ZLM_LAUNCH_MODE(1)
    else if (mode == 2) ZLM_LAUNCH_MODE(2)
    else ZLM_LAUNCH_MODE(3)
#undef ZLM_LAUNCH_MODE
    return zlm_check_launch("gemm_bf16_mma");
}

// mode 0: Y bf16 = X W^T; mode 1: Y fp32 += X W^T; mode 2: Y fp32 = X W^T;
// mode 3: Y bf16 [T, N/2] = silu(gate) * up with W's rows in groups of 8 gate + 8 up
extern "C" int zlm_gemm_bf16_mma(void* Y, const void* X, const void* W, int T, int N, int K, int ldx,
                                 int ldy, int mode, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && N > 0 && K > 0, "gemm_bf16: bad sizes T=%d N=%d K=%d", T, N, K);
    ZLM_REQUIRE(K % 8 == 0 && ldx % 8 == 0,
                "gemm_bf16: the inner size K=%d (row stride %d) must be a multiple of 8 for bf16 kernels", K, ldx);
    ZLM_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_bf16: operands must be 16-byte aligned");
    ZLM_REQUIRE(mode >= 0 && mode <= 3, "gemm_bf16: mode %d", mode);
    ZLM_REQUIRE(mode != 3 || N % 16 == 0, "gemm_bf16: the fused gate/up product needs N=%d to be a multiple of 16", N);
    const __nv_bfloat16* x = (const __nv_bfloat16*)X;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    if (T > 64) return launch_mma<128, 128, 2, 4>(Y, x, w, T, N, K, ldx, ldy, mode, st);
    if (T > 32) return launch_mma<64, 128, 2, 4>(Y, x, w, T, N, K, ldx, ldy, mode, st);
    if (T > 16) return launch_mma<32, 64, 2, 4>(Y, x, w, T, N, K, ldx, ldy, mode, st);
    return launch_mma<16, 128, 1, 8>(Y, x, w, T, N, K, ldx, ldy, mode, st);
}

ZLM_TRANSLATION_UNIT(gemm_bf16_mma)
