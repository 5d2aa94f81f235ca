// Token selection on the GPU.  argmax: the highest logit, ties to the lowest
// index (src/runtime/sampler.zig:14-21).
#include "common.cuh"

#define ARGMAX_CHUNKS 64
#define ARGMAX_THREADS 256

__device__ __forceinline__ bool argmax_better(float va, int ia, float vb, int ib) {
    return va > vb || (va == vb && ia < ib);     // higher value wins, equal values keep the lower index
}

// stage 1: block (row, chunk) finds the best of its chunk of the row
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_partial_kernel(float* __restrict__ pv, int* __restrict__ pi, const float* __restrict__ logits, int V, int ld) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = blockIdx.y * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) {
        const float v = row[i];
        if (v > best || idx == 0x7fffffff) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (argmax_better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < ARGMAX_THREADS / 32 ? bv[lane] : -INFINITY;
        idx = lane < ARGMAX_THREADS / 32 ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (argmax_better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) {
            pv[blockIdx.x * ARGMAX_CHUNKS + blockIdx.y] = best;
            pi[blockIdx.x * ARGMAX_CHUNKS + blockIdx.y] = idx;      // 0x7fffffff: the chunk is empty
        }
    }
}

// stage 2: one warp per row picks among the chunks' candidates (an empty chunk's index
// is the largest integer, so it loses every comparison against a real candidate of equal value;
// its value is -inf, so it loses the others)
__global__ void __launch_bounds__(32)
argmax_final_kernel(int* __restrict__ out, const float* __restrict__ pv, const int* __restrict__ pi) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int c = lane; c < ARGMAX_CHUNKS; c += 32) {
        const float v = pv[blockIdx.x * ARGMAX_CHUNKS + c];
        const int i = pi[blockIdx.x * ARGMAX_CHUNKS + c];
        if (argmax_better(v, i, best, idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (argmax_better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
}

// scratch: R * 64 floats and R * 64 ints
extern "C" int zlm_argmax(int* out, const float* logits, int R, int V, int ld, float* scratch_v, int* scratch_i,
                          cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && V > 0 && ld >= V, "argmax: bad sizes R=%d V=%d ld=%d", R, V, ld);
    ZLM_REQUIRE(scratch_v && scratch_i, "argmax: scratch missing");
    ZLM_REQUIRE(R <= 2147483647 / ARGMAX_CHUNKS, "argmax: too many rows");
    zlm_launch(argmax_partial_kernel, dim3(R, ARGMAX_CHUNKS), dim3(ARGMAX_THREADS), 0, st, scratch_v, scratch_i, logits, V, ld);
    int rc = zlm_check_launch("argmax_partial");
    if (rc) return rc;
    zlm_launch(argmax_final_kernel, dim3(R), dim3(32), 0, st, out, (const float*)scratch_v, (const int*)scratch_i);
    return zlm_check_launch("argmax_final");
}

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling, one block per row.
//
// The reference sorts the logits, keeps the k best, weighs them by
// exp((l - max)/T) in 64-bit, cuts the sorted list at the first place where the
// running share reaches top_p, and draws r = U * kept: the first kept element
// whose running sum exceeds r (src/runtime/sampler.zig:30-67).  Here the same
// kept set is found without a sort: a radix select over order-preserving keys
// gives the k-th largest logit, a second select weighted by the 64-bit weights
// gives the logit at which the share reaches top_p; ties at either threshold are
// kept in index order, as a stable sort would keep them.  The draw then walks
// the kept set in index order (same distribution, one uniform per row).  The
// uniform comes from a counter hash of (seed, request, position), so a row's
// draw does not depend on what else is in the batch.
// ---------------------------------------------------------------------------
#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned order_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__host__ __device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// exclusive scan of one double per thread over the block; also returns the total
__device__ double block_excl_scan(double v, double* warp_tot, double* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    double base = 0.0, tot = 0.0;
    const int nw = blockDim.x >> 5;
    for (int w = 0; w < nw; ++w) {
        const double t = warp_tot[w];
        if (w < warp) base += t;
        tot += t;
    }
    *total = tot;
    return base + inc - v;
}

struct Thresh {
    unsigned key;   // keep keys above this
    int cut;        // and keys equal to it at indices <= cut
};
__device__ __forceinline__ bool kept(unsigned key, int i, const Thresh& t) {
    return key > t.key || (key == t.key && i <= t.cut);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld, float temperature,
              int top_k, float top_p, unsigned long long seed, const int* __restrict__ request,
              const int* __restrict__ position) {
    __shared__ float redf[32];
    __shared__ double redd[32];
    __shared__ double hist_w[256];
    __shared__ int hist_c[256];
    __shared__ unsigned sh_prefix;
    __shared__ int sh_krem, sh_int;
    __shared__ double sh_dbl, sh_dbl2;

    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * ld;
    const int seg = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;     // contiguous segment per thread
    const int i0 = min(V, tid * seg), i1 = min(V, i0 + seg);
    const double invT = 1.0 / (double)temperature;

    float mx = -INFINITY;
    for (int i = tid; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, l[i]);
    mx = block_max(mx, redf);
    const double dmx = (double)mx;

    // index of the n-th (1-based) element with key == key0 among those kept by `lim`
    auto nth_equal = [&](unsigned key0, int n, const Thresh& lim) -> int {
        int c = 0;
        for (int i = i0; i < i1; ++i) c += (order_key(l[i]) == key0 && kept(key0, i, lim)) ? 1 : 0;
        double tot;
        const int before = (int)block_excl_scan((double)c, redd, &tot);
        __syncthreads();
        if (tid == 0) sh_int = 0x7fffffff;
        __syncthreads();
        if (before < n && n <= before + c) {
            int seen = before;
            for (int i = i0; i < i1; ++i)
                if (order_key(l[i]) == key0 && kept(key0, i, lim) && ++seen == n) { sh_int = i; break; }
        }
        __syncthreads();
        return sh_int;
    };

    Thresh tk{0u, 0x7fffffff};
    if (top_k > 0 && top_k < V) {
        // k-th largest key by radix select, 8 bits a pass
        if (tid == 0) { sh_prefix = 0u; sh_krem = top_k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist_c[tid] = 0;
            __syncthreads();
            const unsigned prefix = sh_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            // neighbours mostly fall into the same bin: add a run at a time
            int cb = -1, cc = 0;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const unsigned k = order_key(l[i]);
                if ((k & mask) != prefix) continue;
                const int b = (k >> shift) & 255;
                if (b != cb) {
                    if (cc) atomicAdd(&hist_c[cb], cc);
                    cb = b;
                    cc = 0;
                }
                ++cc;
            }
            if (cc) atomicAdd(&hist_c[cb], cc);
            __syncthreads();
            if (tid == 0) {
                int rem = sh_krem, b = 255;
                for (; b > 0; --b) {
                    if (hist_c[b] >= rem) break;
                    rem -= hist_c[b];
                }
                sh_krem = rem;
                sh_prefix = prefix | ((unsigned)b << shift);
            }
            __syncthreads();
        }
        tk.key = sh_prefix;
        const int ties_kept = sh_krem;
        __syncthreads();
        Thresh all{0u, 0x7fffffff};
        tk.cut = nth_equal(tk.key, ties_kept, all);
    }

    // total weight of what top-k keeps
    double part = 0.0;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = l[i];
        if (kept(order_key(v), i, tk)) part += exp(((double)v - dmx) * invT);
    }
    double total;
    block_excl_scan(part, redd, &total);
    __syncthreads();

    Thresh tp = tk;
    if (top_p < 1.0f) {
        const double target = (double)top_p * total;
        if (tid == 0) { sh_prefix = 0u; sh_dbl = 0.0; }      // sh_dbl: weight strictly above the prefix
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) { hist_w[tid] = 0.0; hist_c[tid] = 0; }
            __syncthreads();
            const unsigned prefix = sh_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            int cb = -1, cc = 0;
            double cw = 0.0;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float v = l[i];
                const unsigned k = order_key(v);
                if ((k & mask) != prefix || !kept(k, i, tk)) continue;
                const int b = (k >> shift) & 255;
                if (b != cb) {
                    if (cc) { atomicAdd(&hist_w[cb], cw); atomicAdd(&hist_c[cb], cc); }
                    cb = b;
                    cc = 0;
                    cw = 0.0;
                }
                cw += exp(((double)v - dmx) * invT);
                ++cc;
            }
            if (cc) { atomicAdd(&hist_w[cb], cw); atomicAdd(&hist_c[cb], cc); }
            __syncthreads();
            if (tid == 0) {
                // from the top bin down: the first non-empty bin at which the running weight
                // reaches the target; if rounding lets none reach it, the lowest non-empty bin
                double above = sh_dbl;
                int b = -1, lowest = -1;
                for (int c = 255; c >= 0; --c) {
                    if (hist_c[c] == 0) continue;
                    lowest = c;
                    if (above + hist_w[c] >= target) { b = c; break; }
                    above += hist_w[c];
                }
                if (b < 0) { b = lowest; above -= hist_w[lowest]; }
                sh_dbl = above;
                sh_dbl2 = hist_w[b];
                sh_int = hist_c[b];
                sh_prefix = prefix | ((unsigned)b << shift);
            }
            __syncthreads();
        }
        tp.key = sh_prefix;
        const double above = sh_dbl, tie_w = sh_dbl2;
        const int ties = sh_int;
        __syncthreads();
        // ties at the threshold weigh the same; keep as many as reach the target
        int need = ties;
        if (ties > 1 && tie_w > 0.0) {
            const double each = tie_w / (double)ties;
            need = (int)ceil((target - above) / each);
            need = need < 1 ? 1 : (need > ties ? ties : need);
        }
        tp.cut = nth_equal(tp.key, need, tk);
    }

    // the draw: r = u * kept weight; walk the kept set in index order
    double mine = 0.0;
    for (int i = i0; i < i1; ++i) {
        const float v = l[i];
        if (kept(order_key(v), i, tp)) mine += exp(((double)v - dmx) * invT);
    }
    double kept_sum;
    const double before = block_excl_scan(mine, redd, &kept_sum);
    __syncthreads();
    const unsigned long long h = splitmix64(seed ^ splitmix64(((unsigned long long)(unsigned)request[row] << 32) |
                                                              (unsigned)position[row]));
    const double u = (double)(h >> 40) * (1.0 / 16777216.0);
    const double r = u * kept_sum;
    if (tid == 0) sh_int = -1;
    __syncthreads();
    if (mine > 0.0 && before <= r && r < before + mine) {
        double cum = before;
        int pick = -1, last = -1;
        for (int i = i0; i < i1; ++i) {
            const float v = l[i];
            if (!kept(order_key(v), i, tp)) continue;
            last = i;
            cum += exp(((double)v - dmx) * invT);
            if (r < cum) { pick = i; break; }
        }
        atomicMax(&sh_int, pick >= 0 ? pick : last);
    }
    __syncthreads();
    const int found = sh_int;
    __syncthreads();
    if (found < 0) {
        // rounding left r at or beyond the last running sum: the last kept element
        int last = -1;
        for (int i = i0; i < i1; ++i)
            if (kept(order_key(l[i]), i, tp)) last = i;
        atomicMax(&sh_int, last);
        __syncthreads();
    }
    if (tid == 0) out[row] = sh_int < 0 ? 0 : sh_int;
}

extern "C" int zlm_sample(int* out, const float* logits, int R, int V, int ld, float temperature, int top_k,
                          float top_p, unsigned long long seed, const int* request, const int* position,
                          cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%d", R, V, ld);
    ZLM_REQUIRE(temperature > 0.f, "sample: temperature must be positive (greedy is argmax)");
    ZLM_REQUIRE(top_k >= 0 && top_p > 0.f, "sample: top_k=%d top_p=%f", top_k, top_p);
    zlm_launch(sample_kernel, R, SAMPLE_THREADS, 0, st, out, logits, V, ld, temperature, top_k, top_p, seed, request,
               position);
    return zlm_check_launch("sample");
}

extern "C" unsigned long long zlm_sample_hash(unsigned long long seed, int request, int position) {
    return splitmix64(seed ^ splitmix64(((unsigned long long)(unsigned)request << 32) | (unsigned)position));
}
