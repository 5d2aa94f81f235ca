// Token selection on the GPU.  argmax: the highest logit, ties to the lowest
// index (src/runtime/sampler.zig:14-21).
#include "common.cuh"

__global__ void __launch_bounds__(1024)
argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || idx == 0x7fffffff) { best = v; idx = i; }
    }
    // (value, index) reduction: higher value wins, equal values keep the lower index
    auto better = [](float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

extern "C" int zlm_argmax(int* out, const float* logits, int R, int V, int ld, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && V > 0 && ld >= V, "argmax: bad sizes R=%d V=%d ld=%d", R, V, ld);
    argmax_kernel<<<R, 1024, 0, st>>>(out, logits, V, ld);
    return zlm_check_launch("argmax");
}
