// Weight-streaming bf16 product for decode steps of up to 16 tokens:
// Y[t, n] = sum_k X[t, k] W[n, k], fp32 accumulation.
//
// The step is bound by reading W once.  A block owns 16 rows of W; its 8 warps (or 4:
// zlm_gemv_plan_warps) split K between them (512 columns each of every 4096, or another even split).  Every thread loads 16 bytes (8 consecutive k) of row g
// and of row g+8 straight from global memory into registers, and the 8 matching
// k of token g of X; these registers are, as they are, the A and B fragments of
// two m16n8k16 tensor-core products: a sum over k does not care in which order
// the k are visited, so the k of a fragment are taken where a 16-byte load puts
// them instead of where the instruction's layout would want them.  No shared
// memory is needed for the operands, W is read in whole 32-byte sectors, and the
// activations cost half the weight's load traffic instead of a multiple of it.
// The warps' partial sums are added in a fixed order.
// (src/kernels/linear/matvec/kernels/bfloat.zig:43-67: bf16 widened, fp32 sum;
// src/gpu/kernels/shaders/matvec_bf16.comp:56-121: rows per group, lanes stride
// over K, tree reduction.)
#include "common.cuh"

#define GEMV_WARPS 8
#define GEMV_THREADS (GEMV_WARPS * 32)
#define GEMV_ROWS 16
#ifndef GEMV_UNROLL
#define GEMV_UNROLL 4
#endif

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    if (!ZLM_CHK(p, 16)) return make_uint4(0, 0, 0, 0);
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// 16 bytes of the activations (they stay in L1: every warp of the block reads them)
__device__ __forceinline__ uint4 ld_act16(const __nv_bfloat16* p) {
    if (!ZLM_CHK(p, 16)) return make_uint4(0, 0, 0, 0);
    return __ldg((const uint4*)p);
}
__device__ __forceinline__ void gemv_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MODE 0: Y bf16 = acc; MODE 1: Y fp32 += acc; MODE 2: Y fp32 = acc; MODE 3: the block's 16 rows are
// 8 gate + 8 up channels, Y bf16 [T, N/2] = silu(gate) * up.  NT: token tiles of 8.
//
// The RMSNorm between a product into the stream and the product that reads the normed stream, without
// a kernel of its own (GemvNorm).  MODE 4 is MODE 1 that also leaves what the norm needs: next[t, n] =
// bf16(Y[t, n] * weight[n]), the normed row but for its scale, and for every token the sum of Y^2 over
// this block's 16 outputs (squares[t][block]).  A product that is given such sums for its input adds
// them up in a fixed order, scale[t] = 1 / sqrt(sum / K + eps), and multiplies its sums by it before
// anything else is done with them: sum_k W[n, k] (x[k] w[k] scale) = scale * sum_k W[n, k] (x[k] w[k]).
// Squares, sum and scale are 32-bit (src/kernels/transformer/norm.zig:128-166).
struct GemvNorm {
    const float* in_squares;        // [T][in_blocks], or null: X is what it is
    int in_blocks;
    float in_eps;
    VecW weight;                    // MODE 4: the following norm's weight [N]
    __nv_bfloat16* next;            // MODE 4: [T][N]
    float* squares;                 // MODE 4: [T][blocks of this product]
};
template <int NT, int MODE, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? 4 : 2)
gemv_bf16_kernel(void* __restrict__ Y, const __nv_bfloat16* __restrict__ X,
                 const __nv_bfloat16* __restrict__ W, int T, int N, int K, int ldx, int ldy, int SEG,
                 float* __restrict__ best_v, int* __restrict__ best_i, const GemvNorm nm) {
    __shared__ float red[WARPS][NT][GEMV_ROWS][8];
    __shared__ float scale[NT * 8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int n0 = blockIdx.x * GEMV_ROWS;
    const __nv_bfloat16* w0 = W + (size_t)min(n0 + g, N - 1) * K + q * 8;
    const __nv_bfloat16* w1 = W + (size_t)min(n0 + g + 8, N - 1) * K + q * 8;
    const __nv_bfloat16* xr[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = j * 8 + g < T;
        xr[j] = X + (size_t)(xok[j] ? j * 8 + g : 0) * ldx + q * 8;
    }
    // Four chains of sums per thread, so that four tensor-core products can be in flight
    // (one chain would run at the latency of the instruction).  K is cut into chunks of
    // WARPS x SEG columns; warp w takes the w-th SEG columns of every chunk, as blocks of 32
    // in ascending k; chain 2 * (i & 1) + h takes the h-th 16 k of block i.  The chains are
    // added at the end, (0 + 1) + (2 + 3).  SEG is 512 unless another width spreads K evenly over the
    // warps where 512 would not (gemv_segment below).
    float ch[NT][4][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int r = 0; r < 4; ++r) ch[j][c][r] = 0.f;

    // GEMV_UNROLL blocks in flight.  The weights do not depend on the kernel before this one:
    // their first loads are issued before the wait for it, the activations after.
    const int CHUNK = WARPS * SEG;
    pdl_launch_dependents();
    uint4 a[GEMV_UNROLL], b[GEMV_UNROLL];
    bool have = warp * SEG + GEMV_UNROLL * 32 <= K;
    if (have) {
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; ++u) {
            a[u] = ld_stream16(w0 + warp * SEG + u * 32);
            b[u] = ld_stream16(w1 + warp * SEG + u * 32);
        }
    }
    pdl_wait();
    // What the epilogue would otherwise wait for after the last product: the stream's old values
    // (MODE 1 and 4), the following norm's weight, and the scale of an input whose norm was left to
    // this product.  Asked for now, they arrive under the weights' first loads.
    constexpr int EPI = (NT * GEMV_ROWS * 8 + WARPS * 32 - 1) / (WARPS * 32);
    float y_old[EPI], nw_row = 0.f;
    if constexpr (MODE == 1 || MODE == 4) {
#pragma unroll
        for (int it = 0; it < EPI; ++it) {
            const int idx = tid + it * WARPS * 32;
            const int tok = (idx / (GEMV_ROWS * 8)) * 8 + (idx % (GEMV_ROWS * 8)) / GEMV_ROWS, n = n0 + idx % GEMV_ROWS;
            const float* yp = (const float*)Y + (size_t)tok * ldy + n;
            y_old[it] = (idx < NT * GEMV_ROWS * 8 && tok < T && n < N && ZLM_CHK(yp, 4)) ? *yp : 0.f;
        }
        if (MODE == 4 && n0 + tid % GEMV_ROWS < N) nw_row = nm.weight[n0 + tid % GEMV_ROWS];   // a thread's row is the same in every turn
    }
    if (nm.in_squares) {
        // the scale of a row whose norm is left to this product: a warp a token, the blocks' sums in
        // lanes and then across them, the same order in every block and every run
        for (int tok = warp; tok < T; tok += WARPS) {
            const float* sq = nm.in_squares + (size_t)tok * nm.in_blocks;
            float ss = 0.f;
            for (int i = lane; i < nm.in_blocks; i += 32)
                if (ZLM_CHK(sq + i, 4)) ss += sq[i];
            ss = warp_sum(ss);
            if (lane == 0) scale[tok] = 1.0f / sqrtf(ss / (float)K + nm.in_eps);
        }
    }
    for (int kc = warp * SEG; kc < K; kc += CHUNK) {
        const int kend = min(K, kc + SEG);
        int kb = kc;
        for (; kb + GEMV_UNROLL * 32 <= kend; kb += GEMV_UNROLL * 32) {
            uint4 x[GEMV_UNROLL][NT];
            if (!have) {
#pragma unroll
                for (int u = 0; u < GEMV_UNROLL; ++u) {
                    a[u] = ld_stream16(w0 + kb + u * 32);
                    b[u] = ld_stream16(w1 + kb + u * 32);
                }
            }
            have = false;
#pragma unroll
            for (int u = 0; u < GEMV_UNROLL; ++u)
#pragma unroll
                for (int j = 0; j < NT; ++j)
                    x[u][j] = xok[j] ? ld_act16(xr[j] + kb + u * 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < GEMV_UNROLL; ++u)      // kb - kc is a multiple of 128: block u has parity u & 1
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    gemv_mma(ch[j][2 * (u & 1)], a[u].x, b[u].x, a[u].y, b[u].y, x[u][j].x, x[u][j].y);
                    gemv_mma(ch[j][2 * (u & 1) + 1], a[u].z, b[u].z, a[u].w, b[u].w, x[u][j].z, x[u][j].w);
                }
        }
        for (int par = 0; kb < kend; kb += 32, par ^= 1) {
            // K is a multiple of 8, so a thread's 8 k are all inside or all outside
            const bool in = kb + q * 8 < K;
            const uint4 z = make_uint4(0, 0, 0, 0);
            const uint4 a = in ? ld_stream16(w0 + kb) : z;
            const uint4 b = in ? ld_stream16(w1 + kb) : z;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 x = (in && xok[j]) ? ld_act16(xr[j] + kb) : z;
                if (par == 0) {
                    gemv_mma(ch[j][0], a.x, b.x, a.y, b.y, x.x, x.y);
                    gemv_mma(ch[j][1], a.z, b.z, a.w, b.w, x.z, x.w);
                } else {
                    gemv_mma(ch[j][2], a.x, b.x, a.y, b.y, x.x, x.y);
                    gemv_mma(ch[j][3], a.z, b.z, a.w, b.w, x.z, x.w);
                }
            }
        }
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[j][r] = (ch[j][0][r] + ch[j][1][r]) + (ch[j][2][r] + ch[j][3][r]);
    // acc[j][0..1]: row g, tokens 8j + 2q, 2q+1; acc[j][2..3]: row g + 8
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][j][g][2 * q] = acc[j][0];
        red[warp][j][g][2 * q + 1] = acc[j][1];
        red[warp][j][g + 8][2 * q] = acc[j][2];
        red[warp][j][g + 8][2 * q + 1] = acc[j][3];
    }
    __syncthreads();
    if constexpr (MODE == 3) {
        for (int idx = tid; idx < NT * 8 * 8; idx += WARPS * 32) {
            const int j = idx / 64, rem = idx % 64;
            const int tok = j * 8 + rem / 8, row = rem % 8;
            if (tok >= T || n0 + row + 8 >= N) continue;
            float sg = 0.f, su = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                sg += red[w][j][row][tok & 7];
                su += red[w][j][row + 8][tok & 7];
            }
            if (nm.in_squares) { sg *= scale[tok]; su *= scale[tok]; }
            if (ZLM_CHK((__nv_bfloat16*)Y + (size_t)tok * ldy + n0 / 2 + row, 2))
                ((__nv_bfloat16*)Y)[(size_t)tok * ldy + n0 / 2 + row] = __float2bfloat16_rn((sg / (1.0f + expf(-sg))) * su);
        }
    } else {
#pragma unroll
    for (int it = 0; it < EPI; ++it) {
        const int idx = tid + it * WARPS * 32;
        if (idx >= NT * GEMV_ROWS * 8) break;            // whole warps
        const int j = idx / (GEMV_ROWS * 8), rem = idx % (GEMV_ROWS * 8);
        const int tok = j * 8 + rem / GEMV_ROWS, row = rem % GEMV_ROWS;   // rows fastest: coalesced stores
        const int n = n0 + row;
        const bool live = tok < T && n < N;
        float s = 0.f;
        if (live) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) s += red[w][j][row][tok & 7];
            if (nm.in_squares) s *= scale[tok];
            const size_t o = (size_t)tok * ldy + n;
            if (ZLM_CHK((char*)Y + o * (MODE == 0 ? 2 : 4), MODE == 0 ? 2 : 4)) {
                if (MODE == 0) ((__nv_bfloat16*)Y)[o] = __float2bfloat16_rn(s);
                else if (MODE == 1 || MODE == 4) { s += y_old[it]; ((float*)Y)[o] = s; }     // s: the stream's new value
                else ((float*)Y)[o] = s;
            } else s = 0.f;
        }
        if (MODE == 4) {
            // what the norm after this product needs: the new values times its weight, and the
            // token's sum of squares over this block's outputs (16 neighbouring lanes, whole warps)
            if (live && ZLM_CHK(nm.next + (size_t)tok * N + n, 2))
                nm.next[(size_t)tok * N + n] = __float2bfloat16_rn(s * nw_row);
            float ss = live ? s * s : 0.f;
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
            if (row == 0 && tok < T && ZLM_CHK(nm.squares + (size_t)tok * gridDim.x + blockIdx.x, 4))
                nm.squares[(size_t)tok * gridDim.x + blockIdx.x] = ss;
        }
        if (MODE == 2 && best_v) {
            // The logits' argmax starts here: the best of this block's 16 outputs for every token
            // (16 neighbouring lanes hold a token's 16 rows; every iteration of this loop is taken
            // by whole warps), ties to the lower index; a second kernel picks among the blocks'
            // candidates instead of reading the logits again (src/runtime/sampler.zig:14-21).
            float bv = live ? s : -INFINITY;
            int bi = live ? n : 0x7fffffff;
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o2);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o2);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (row == 0 && tok < T) {
                const size_t c = (size_t)tok * gridDim.x + blockIdx.x;
                if (ZLM_CHK(best_v + c, 4) && ZLM_CHK(best_i + c, 4)) { best_v[c] = bv; best_i[c] = bi; }
            }
        }
    }
    }
}

// The columns a warp takes of every chunk of K.  With 512, a K that is no multiple of 4096 leaves
// warps idle in its last chunk: of K = 5120 two warps would read 1024 columns each and six 512,
// of K = 1024 two warps would do everything.  Where K is a multiple of 1024 but not of 4096 the
// widest of 640, 384, 256 and 128 columns that divides K into whole chunks is taken instead
// (multiples of the 128 columns a warp has in flight).
static int gemv_segment(int K, int warps) {
    if (K % (512 * warps) == 0 || K % 1024 != 0) return 512;
    for (int seg : {640, 384, 256, 128})
        if (K % (warps * seg) == 0) return seg;
    return 512;
}
extern "C" int zlm_gemv_segment(int K) { return gemv_segment(K, GEMV_WARPS); }

// Blocks of 8 warps or of 4.  A block of 8 warps has twice the loads in flight and is done in half
// the time, which is what a product of one round of blocks wants; but two such blocks fill an SM,
// and of 384 blocks the last 88 then run alone, far too few to keep the memory busy, where blocks
// of 4 warps (5 to an SM, 4 with two token tiles) are all resident at once.  The choice is by an
// estimate of both forms' time in microseconds: the blocks run in rounds of all resident places;
// a round takes as long as its bytes at the memory's rate or as a block's own chain of loads
// (a warp has 128 columns in flight, about a microsecond a trip), whichever is longer, and half
// a microsecond around it.  Fitted on products of 300 to 3,000 blocks at K = 1024 and 4096 and
// checked at K = 5120, 8192 and 12288: it names the faster form wherever the two differ by
// more than a twentieth.
static double gemv_estimate(int blocks, int K, int warps, int slots) {
    const double trip_us = 1.0, bytes_per_us = 6.2e6, round_us = 0.5;
    const double block_bytes = (double)GEMV_ROWS * K * 2;
    const double chain = (double)((K + warps * 128 - 1) / (warps * 128)) * trip_us;
    double t = 0;
    for (int rem = blocks; rem > 0; rem -= slots) {
        const double stream = (double)(rem < slots ? rem : slots) * block_bytes / bytes_per_us;
        t += (stream > chain ? stream : chain) + round_us;
    }
    return t;
}
// 8 or 4: the warps of a block for a product of N outputs over K; wide and narrow are the blocks
// of 8 and of 4 warps that an SM holds at once.
extern "C" int zlm_gemv_plan_warps(int N, int K, int sms, int wide, int narrow) {
    const int blocks = (N + GEMV_ROWS - 1) / GEMV_ROWS;
    if (sms <= 0 || wide <= 0 || narrow <= 0 || blocks <= sms * wide) return 8;
    return gemv_estimate(blocks, K, 4, sms * narrow) < gemv_estimate(blocks, K, 8, sms * wide) ? 4 : 8;
}

template <int NT, int WARPS>
static int launch_gemv_w(void* Y, const __nv_bfloat16* X, const __nv_bfloat16* W, int T, int N, int K,
                         int ldx, int ldy, int mode, float* best_v, int* best_i, const GemvNorm& nm, cudaStream_t st) {
    const int blocks = (N + GEMV_ROWS - 1) / GEMV_ROWS;
    const int seg = gemv_segment(K, WARPS);
    float* bv = mode == 2 ? best_v : nullptr;
    int* bi = mode == 2 ? best_i : nullptr;
    if (mode == 0) zlm_launch(gemv_bf16_kernel<NT, 0, WARPS>, blocks, WARPS * 32, 0, st, Y, X, W, T, N, K, ldx, ldy, seg, bv, bi, nm);
    else if (mode == 1) zlm_launch(gemv_bf16_kernel<NT, 1, WARPS>, blocks, WARPS * 32, 0, st, Y, X, W, T, N, K, ldx, ldy, seg, bv, bi, nm);
    else if (mode == 2) zlm_launch(gemv_bf16_kernel<NT, 2, WARPS>, blocks, WARPS * 32, 0, st, Y, X, W, T, N, K, ldx, ldy, seg, bv, bi, nm);
    else if (mode == 3) zlm_launch(gemv_bf16_kernel<NT, 3, WARPS>, blocks, WARPS * 32, 0, st, Y, X, W, T, N, K, ldx, ldy, seg, bv, bi, nm);
    else zlm_launch(gemv_bf16_kernel<NT, 4, WARPS>, blocks, WARPS * 32, 0, st, Y, X, W, T, N, K, ldx, ldy, seg, bv, bi, nm);
    return zlm_check_launch("gemv_bf16");
}

template <int NT>
static int launch_gemv(void* Y, const __nv_bfloat16* X, const __nv_bfloat16* W, int T, int N, int K,
                       int ldx, int ldy, int mode, float* best_v, int* best_i, const GemvNorm& nm, cudaStream_t st) {
    // the head's product (mode 2) is many rounds either way and keeps the wide blocks
    static int sms = 0, wide = 0, narrow = 0;
    if (!sms) {
        int n = 0, w = 0, nw = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, zlm_device_index()) != cudaSuccess || n <= 0) n = 148;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&w, gemv_bf16_kernel<NT, 0, 8>, 8 * 32, 0) != cudaSuccess || w <= 0) w = 2;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nw, gemv_bf16_kernel<NT, 0, 4>, 4 * 32, 0) != cudaSuccess || nw <= 0) nw = 4;
        (void)cudaGetLastError();
        wide = w; narrow = nw; sms = n;
    }
    if (mode != 2 && zlm_gemv_plan_warps(N, K, sms, wide, narrow) == 4)
        return launch_gemv_w<NT, 4>(Y, X, W, T, N, K, ldx, ldy, mode, best_v, best_i, nm, st);
    return launch_gemv_w<NT, 8>(Y, X, W, T, N, K, ldx, ldy, mode, best_v, best_i, nm, st);
}

extern "C" int zlm_gemv_max_tokens() { return 16; }

extern "C" int zlm_gemv_blocks(int N) { return (N + GEMV_ROWS - 1) / GEMV_ROWS; }

static int gemv_entry(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy, int mode,
                      float* best_v, int* best_i, const GemvNorm& nm, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && T <= 16, "gemv_bf16: takes 1 to 16 tokens, got %d", T);
    ZLM_REQUIRE(N > 0 && K > 0, "gemv_bf16: bad sizes N=%d K=%d", N, K);
    ZLM_REQUIRE(K % 8 == 0 && ldx % 8 == 0,
                "gemv_bf16: the inner size K=%d (row stride %d) must be a multiple of 8 for bf16 kernels", K, ldx);
    ZLM_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemv_bf16: operands must be 16-byte aligned");
    ZLM_REQUIRE(mode >= 0 && mode <= 4, "gemv_bf16: mode %d", mode);
    ZLM_REQUIRE(mode != 3 || N % 16 == 0, "gemv_bf16: the fused gate/up product needs N=%d to be a multiple of 16", N);
    ZLM_REQUIRE(mode != 4 || (nm.weight.p && nm.next && nm.squares), "gemv_bf16: the following norm's weight and outputs are missing");
    ZLM_REQUIRE(!nm.in_squares || nm.in_blocks > 0, "gemv_bf16: sums of squares of %d blocks", nm.in_blocks);
    const __nv_bfloat16* x = (const __nv_bfloat16*)X;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    if (T <= 8) return launch_gemv<1>(Y, x, w, T, N, K, ldx, ldy, mode, best_v, best_i, nm, st);
    return launch_gemv<2>(Y, x, w, T, N, K, ldx, ldy, mode, best_v, best_i, nm, st);
}

static GemvNorm gemv_no_norm() { return GemvNorm{nullptr, 0, 0.f, VecW{nullptr, ZLM_DTYPE_F32}, nullptr, nullptr}; }

extern "C" int zlm_gemv_bf16(void* Y, const void* X, const void* W, int T, int N, int K, int ldx,
                             int ldy, int mode, cudaStream_t st) {
    ZLM_REQUIRE(mode != 4, "gemv_bf16: mode 4 is zlm_gemv_bf16_norms'");
    return gemv_entry(Y, X, W, T, N, K, ldx, ldy, mode, nullptr, nullptr, gemv_no_norm(), st);
}

// Y fp32 [T, N] = X W^T, and for every token the best (value, index) of each block's 16 outputs:
// best_v / best_i [T][zlm_gemv_blocks(N)], what zlm_argmax_candidates picks the row's argmax from.
extern "C" int zlm_gemv_bf16_best(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy,
                                  float* best_v, int* best_i, cudaStream_t st) {
    ZLM_REQUIRE(best_v && best_i, "gemv_bf16_best: the candidates' arrays are missing");
    return gemv_entry(Y, X, W, T, N, K, ldx, ldy, 2, best_v, best_i, gemv_no_norm(), st);
}

// The product with an RMSNorm's halves in it (GemvNorm above).  in_squares [T][in_blocks]: X is a
// normed row but for its scale, which is taken from these sums with in_eps (null: X as it is).
// norm_weight (mode 1 only; null: no following norm): Y += acc also leaves next [T][N] bf16 and
// squares [T][zlm_gemv_blocks(N)] for the product after the norm.  best_v / best_i as above
// (mode 2; may be null).
extern "C" int zlm_gemv_bf16_norms(void* Y, const void* X, const void* W, int T, int N, int K, int ldx, int ldy,
                                   int mode, float* best_v, int* best_i, const float* in_squares, int in_blocks,
                                   float in_eps, const void* norm_weight, int norm_weight_dtype, void* next,
                                   float* squares, cudaStream_t st) {
    ZLM_REQUIRE(mode != 4 && (!norm_weight || mode == 1), "gemv_bf16_norms: a following norm goes with mode 1, got %d", mode);
    GemvNorm nm{in_squares, in_blocks, in_eps, VecW{norm_weight, norm_weight_dtype}, (__nv_bfloat16*)next, squares};
    return gemv_entry(Y, X, W, T, N, K, ldx, ldy, norm_weight ? 4 : mode, best_v, best_i, nm, st);
}

ZLM_TRANSLATION_UNIT(gemv_bf16)
