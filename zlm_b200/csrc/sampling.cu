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
    if (!ZLM_CHK(row, (size_t)V * 4) || !ZLM_CHK(pv + blockIdx.x * ARGMAX_CHUNKS + blockIdx.y, 4) ||
        !ZLM_CHK(pi + blockIdx.x * ARGMAX_CHUNKS + blockIdx.y, 4))
        return;                                                          // block-uniform
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
    if (!ZLM_CHK(pv + blockIdx.x * ARGMAX_CHUNKS, ARGMAX_CHUNKS * 4) || !ZLM_CHK(pi + blockIdx.x * ARGMAX_CHUNKS, ARGMAX_CHUNKS * 4) ||
        !ZLM_CHK(out + blockIdx.x, 4))
        return;
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

// the row's argmax from `n` candidates (value, index) that the product of the logits left
// (one per block of 16 outputs): one block per row, the same tie rule
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_candidates_kernel(int* __restrict__ out, const float* __restrict__ cv, const int* __restrict__ ci, int n) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* v = cv + (size_t)blockIdx.x * n;
    const int* ix = ci + (size_t)blockIdx.x * n;
    if (!ZLM_CHK(v, (size_t)n * 4) || !ZLM_CHK(ix, (size_t)n * 4) || !ZLM_CHK(out + blockIdx.x, 4)) return;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int c = threadIdx.x; c < n; c += ARGMAX_THREADS)
        if (argmax_better(v[c], ix[c], best, idx)) { best = v[c]; idx = ix[c]; }
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
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}
extern "C" int zlm_argmax_candidates(int* out, const float* cand_v, const int* cand_i, int R, int n, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && n > 0 && cand_v && cand_i, "argmax_candidates: bad sizes R=%d n=%d", R, n);
    zlm_launch(argmax_candidates_kernel, dim3(R), dim3(ARGMAX_THREADS), 0, st, out, cand_v, cand_i, n);
    return zlm_check_launch("argmax_candidates");
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

// Walks a row with 8 loads in flight per thread: a loop whose body branches on the value it
// has just loaded would otherwise wait a whole memory latency per element.
template <typename F>
__device__ __forceinline__ void for_each_strided(const float* __restrict__ l, int V, F f) {
    for (int base = threadIdx.x; base < V; base += 8 * SAMPLE_THREADS) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * SAMPLE_THREADS;
            v[u] = i < V ? l[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * SAMPLE_THREADS;
            if (i < V) f(i, v[u]);
        }
    }
}
// the same over a thread's own contiguous segment [i0, i1), in index order; f returns false to stop
template <typename F>
__device__ __forceinline__ void for_each_segment(const float* __restrict__ l, int i0, int i1, F f) {
    for (int base = i0; base < i1; base += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = base + u < i1 ? l[base + u] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (base + u < i1 && !f(base + u, v[u])) return;
    }
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
    __shared__ unsigned long long hist_w[256];     // weights of a pass's bins in 2^-40 units (exact, order-free sums)
    __shared__ int hist_c[256];
    __shared__ unsigned sh_prefix;
    __shared__ int sh_krem, sh_int;
    __shared__ unsigned long long sh_u64, sh_u64b;
    // one histogram per warp, so that only the 32 lanes of a warp ever meet on an address
    extern __shared__ __align__(16) unsigned char sample_smem[];
    unsigned long long* warp_w = (unsigned long long*)sample_smem;                // [32][256]
    int* warp_c = (int*)(warp_w + 32 * 256);                                      // [32][256]
    const int my_warp = threadIdx.x >> 5;

    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t)row * ld;
    if (!ZLM_CHK(l, (size_t)V * 4) || !ZLM_CHK(out + row, 4) || !ZLM_CHK(request + row, 4) || !ZLM_CHK(position + row, 4))
        return;                                                          // block-uniform
    const int seg = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;     // contiguous segment per thread
    const int i0 = min(V, tid * seg), i1 = min(V, i0 + seg);
    const float invT = 1.0f / temperature;

    float mx = -INFINITY;
    for_each_strided(l, V, [&](int, float v) { mx = fmaxf(mx, v); });
    mx = block_max(mx, redf);

    // index of the n-th (1-based) element with key == key0 among those kept by `lim`
    auto nth_equal = [&](unsigned key0, int n, const Thresh& lim) -> int {
        int c = 0;
        for_each_segment(l, i0, i1, [&](int i, float v) { c += (order_key(v) == key0 && kept(key0, i, lim)) ? 1 : 0; return true; });
        double tot;
        const int before = (int)block_excl_scan((double)c, redd, &tot);
        __syncthreads();
        if (tid == 0) sh_int = 0x7fffffff;
        __syncthreads();
        if (before < n && n <= before + c) {
            int seen = before;
            for_each_segment(l, i0, i1, [&](int i, float v) {
                if (order_key(v) == key0 && kept(key0, i, lim) && ++seen == n) { sh_int = i; return false; }
                return true;
            });
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
            for (int i = tid; i < 32 * 256; i += SAMPLE_THREADS) warp_c[i] = 0;
            __syncthreads();
            const unsigned prefix = sh_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for_each_strided(l, V, [&](int, float v) {
                const unsigned k = order_key(v);
                if ((k & mask) == prefix) atomicAdd(&warp_c[my_warp * 256 + ((k >> shift) & 255)], 1);
            });
            __syncthreads();
            if (tid < 256) {
                int c = 0;
#pragma unroll 8
                for (int w = 0; w < 32; ++w) c += warp_c[w * 256 + tid];
                hist_c[tid] = c;
            }
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

    // total weight of what top-k keeps, in 2^-40 units
    const double FX = 1099511627776.0;
    // a token's weight exp((l - max) / T): 32-bit arithmetic, as the softmax of the model's other
    // kernels; sums of weights are exact (fixed point, or 64-bit floating point for the draw)
    auto weight = [&](float v) -> float { return expf((v - mx) * invT); };
    auto weight_fx = [&](float v) -> unsigned long long { return (unsigned long long)((double)weight(v) * FX + 0.5); };
    Thresh tp = tk;
    if (top_p < 1.0f) {
        unsigned long long part = 0;
        for_each_strided(l, V, [&](int i, float v) {
            if (kept(order_key(v), i, tk)) part += weight_fx(v);
        });
        if (tid == 0) sh_u64 = 0;
        __syncthreads();
        atomicAdd(&sh_u64, part);
        __syncthreads();
        const unsigned long long total = sh_u64;
        const unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        __syncthreads();
        if (tid == 0) { sh_prefix = 0u; sh_u64 = 0; }         // sh_u64: weight strictly above the prefix
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 32 * 256; i += SAMPLE_THREADS) { warp_w[i] = 0; warp_c[i] = 0; }
            __syncthreads();
            const unsigned prefix = sh_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for_each_strided(l, V, [&](int i, float v) {
                const unsigned k = order_key(v);
                if ((k & mask) != prefix || !kept(k, i, tk)) return;
                const int b = my_warp * 256 + ((k >> shift) & 255);
                atomicAdd(&warp_w[b], weight_fx(v));
                atomicAdd(&warp_c[b], 1);
            });
            __syncthreads();
            if (tid < 256) {
                unsigned long long w = 0;
                int c = 0;
#pragma unroll 8
                for (int wi = 0; wi < 32; ++wi) { w += warp_w[wi * 256 + tid]; c += warp_c[wi * 256 + tid]; }
                hist_w[tid] = w;
                hist_c[tid] = c;
            }
            __syncthreads();
            if (tid == 0) {
                // from the top bin down: the first non-empty bin at which the running weight
                // reaches the target; if none reaches it, the lowest non-empty bin
                unsigned long long above = sh_u64;
                int b = -1, lowest = -1;
                for (int c = 255; c >= 0; --c) {
                    if (hist_c[c] == 0) continue;
                    lowest = c;
                    if (above + hist_w[c] >= target) { b = c; break; }
                    above += hist_w[c];
                }
                if (b < 0) { b = lowest; above -= hist_w[lowest]; }
                sh_u64 = above;
                sh_u64b = hist_w[b];
                sh_int = hist_c[b];
                sh_prefix = prefix | ((unsigned)b << shift);
            }
            __syncthreads();
        }
        tp.key = sh_prefix;
        const unsigned long long above = sh_u64, tie_w = sh_u64b;
        const int ties = sh_int;
        __syncthreads();
        // ties at the threshold weigh the same; keep as many as reach the target
        int need = ties;
        if (ties > 1 && tie_w > 0) {
            const unsigned long long each = tie_w / (unsigned long long)ties;
            if (each > 0 && target > above) {
                const unsigned long long n = (target - above + each - 1) / each;
                need = n < 1 ? 1 : (n > (unsigned long long)ties ? ties : (int)n);
            } else {
                need = 1;
            }
        }
        tp.cut = nth_equal(tp.key, need, tk);
    }

    // the draw: r = u * kept weight; walk the kept set in index order
    double mine = 0.0;
    for_each_segment(l, i0, i1, [&](int i, float v) {
        if (kept(order_key(v), i, tp)) mine += (double)weight(v);
        return true;
    });
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
            cum += (double)weight(v);
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

// ---------------------------------------------------------------------------
// The same sampler on a thread-block cluster: 8 blocks per row, each holding an eighth
// of the row in shared memory.  The one-block kernel above walks the row in L2 a dozen
// times with 1,024 threads, every walk a chain of memory latencies; here the row is
// read once, every later walk reads shared memory, and what the blocks have to agree on
// (a maximum, a histogram, a count, a sum) is exchanged through distributed shared
// memory: each block leaves its share in its own shared memory, the cluster meets at a
// barrier, and every block adds up all eight in rank order, so that all decide alike.
// Exchange buffers take turns (parity of the exchange's number): a block can be at most
// one exchange ahead of a block that still reads.
// The kept set, the ties' order and the draw are those of the one-block kernel; sums of
// 64-bit floating point are added in index order block by block instead of thread by
// thread, which moves the draw's boundaries by rounding only.
// ---------------------------------------------------------------------------
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SC_CLUSTER 8

struct SampleExchange {
    float f[2];
    int i[2];
    unsigned long long u[2];
    double d[2];
    int hist_c[2][256];
    unsigned long long hist_w[2][256];
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_cluster_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int ld, float temperature,
                      int top_k, float top_p, unsigned long long seed, const int* __restrict__ request,
                      const int* __restrict__ position, int chunk) {
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int row = blockIdx.x / SC_CLUSTER, tid = threadIdx.x, lane = tid & 31, my_warp = tid >> 5;
    __shared__ SampleExchange X;
    __shared__ float redf[32];
    __shared__ double redd[32];
    __shared__ int tot_c[256];
    __shared__ unsigned long long tot_w[256];
    __shared__ unsigned sh_prefix;
    __shared__ int sh_krem, sh_int;
    __shared__ unsigned long long sh_u64, sh_u64b;
    __shared__ double sh_d[2];
    extern __shared__ __align__(16) unsigned char sample_smem[];
    unsigned long long* warp_w = (unsigned long long*)sample_smem;                // [32][256]
    int* warp_c = (int*)(warp_w + 32 * 256);                                      // [32][256]
    float* seg = (float*)(warp_c + 32 * 256);                                     // [chunk]: this block's part of the row

    pdl_launch_dependents();
    pdl_wait();
    const float* l = logits + (size_t)row * ld;
    if (!ZLM_CHK(l, (size_t)V * 4) || !ZLM_CHK(out + row, 4) || !ZLM_CHK(request + row, 4) || !ZLM_CHK(position + row, 4))
        return;                                                          // the same answer in every block of the cluster
    const int lo = min(V, rank * chunk), n = min(V, lo + chunk) - lo;             // global [lo, lo + n)
    // a thread's own contiguous part, for the walks in index order (an odd length: no bank conflicts)
    const int sseg = ((chunk + SAMPLE_THREADS - 1) / SAMPLE_THREADS) | 1;
    const int t0 = min(n, tid * sseg), t1 = min(n, t0 + sseg);
    const float invT = 1.0f / temperature;
    int par = 0;                                                                  // the next exchange's buffers

    float mx = -INFINITY;
    for (int i = tid; i < n; i += SAMPLE_THREADS) {
        const float v = l[lo + i];
        seg[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, redf);
    if (tid == 0) X.f[par] = mx;
    cluster.sync();
    if (tid < 32) {
        float m = lane < SC_CLUSTER ? cluster.map_shared_rank(&X, lane)->f[par] : -INFINITY;
        m = warp_max(m);
        if (lane == 0) redf[0] = m;
    }
    __syncthreads();
    mx = redf[0];
    par ^= 1;
    __syncthreads();

    // ---- exchanges ------------------------------------------------------------
    // sum of one int / u64 per block over the cluster, and the sum over the lower ranks
    auto exchange_u64 = [&](unsigned long long mine_, unsigned long long* below) -> unsigned long long {
        if (tid == 0) X.u[par] = mine_;
        cluster.sync();
        if (tid == 0) {
            unsigned long long tot = 0, b = 0;
            for (int r = 0; r < SC_CLUSTER; ++r) {
                const unsigned long long v = cluster.map_shared_rank(&X, r)->u[par];
                if (r < rank) b += v;
                tot += v;
            }
            sh_u64 = tot;
            sh_u64b = b;
        }
        __syncthreads();
        const unsigned long long tot = sh_u64;
        if (below) *below = sh_u64b;
        par ^= 1;
        __syncthreads();
        return tot;
    };
    // the smallest / largest int over the cluster
    auto exchange_int = [&](int mine_, bool take_min) -> int {
        if (tid == 0) X.i[par] = mine_;
        cluster.sync();
        if (tid == 0) {
            int best = cluster.map_shared_rank(&X, 0)->i[par];
            for (int r = 1; r < SC_CLUSTER; ++r) {
                const int v = cluster.map_shared_rank(&X, r)->i[par];
                best = take_min ? min(best, v) : max(best, v);
            }
            sh_int = best;
        }
        __syncthreads();
        const int best = sh_int;
        par ^= 1;
        __syncthreads();
        return best;
    };
    // this block's merged histogram lies in X.hist_*[par]: the cluster's total into tot_c / tot_w
    auto exchange_hist = [&](bool weights) {
        cluster.sync();
        if (tid < 256) {
            int c = 0;
            unsigned long long w = 0;
            for (int r = 0; r < SC_CLUSTER; ++r) {
                const SampleExchange* x = cluster.map_shared_rank(&X, r);
                c += x->hist_c[par][tid];
                if (weights) w += x->hist_w[par][tid];
            }
            tot_c[tid] = c;
            tot_w[tid] = w;
        }
        par ^= 1;
        __syncthreads();
    };

    // global index of the n-th (1-based) element with key == key0 among those kept by `lim`
    auto nth_equal = [&](unsigned key0, int nth, const Thresh& lim) -> int {
        int c = 0;
        for (int i = t0; i < t1; ++i) c += (order_key(seg[i]) == key0 && kept(key0, lo + i, lim)) ? 1 : 0;
        double tot;
        const int before_block = (int)block_excl_scan((double)c, redd, &tot);
        __syncthreads();
        unsigned long long below;
        exchange_u64((unsigned long long)tot, &below);
        const int before = (int)below + before_block;
        int found = 0x7fffffff;
        if (before < nth && nth <= before + c) {
            int seen = before;
            for (int i = t0; i < t1; ++i)
                if (order_key(seg[i]) == key0 && kept(key0, lo + i, lim) && ++seen == nth) { found = lo + i; break; }
        }
        if (tid == 0) sh_int = 0x7fffffff;
        __syncthreads();
        if (found != 0x7fffffff) sh_int = found;            // at most one thread of the cluster
        __syncthreads();
        const int mine_ = sh_int;
        __syncthreads();
        return exchange_int(mine_, true);
    };

    Thresh tk{0u, 0x7fffffff};
    if (top_k > 0 && top_k < V) {
        if (tid == 0) { sh_prefix = 0u; sh_krem = top_k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 32 * 256; i += SAMPLE_THREADS) warp_c[i] = 0;
            __syncthreads();
            const unsigned prefix = sh_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < n; i += SAMPLE_THREADS) {
                const unsigned k = order_key(seg[i]);
                if ((k & mask) == prefix) atomicAdd(&warp_c[my_warp * 256 + ((k >> shift) & 255)], 1);
            }
            __syncthreads();
            if (tid < 256) {
                int c = 0;
#pragma unroll 8
                for (int w = 0; w < 32; ++w) c += warp_c[w * 256 + tid];
                X.hist_c[par][tid] = c;
            }
            exchange_hist(false);
            if (tid == 0) {
                int rem = sh_krem, b = 255;
                for (; b > 0; --b) {
                    if (tot_c[b] >= rem) break;
                    rem -= tot_c[b];
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

    const double FX = 1099511627776.0;
    auto weight = [&](float v) -> float { return expf((v - mx) * invT); };
    auto weight_fx = [&](float v) -> unsigned long long { return (unsigned long long)((double)weight(v) * FX + 0.5); };
    Thresh tp = tk;
    if (top_p < 1.0f) {
        unsigned long long part = 0;
        for (int i = tid; i < n; i += SAMPLE_THREADS) {
            const float v = seg[i];
            if (kept(order_key(v), lo + i, tk)) part += weight_fx(v);
        }
        if (tid == 0) sh_u64 = 0;
        __syncthreads();
        atomicAdd(&sh_u64, part);
        __syncthreads();
        const unsigned long long block_total = sh_u64;
        __syncthreads();
        const unsigned long long total = exchange_u64(block_total, nullptr);
        const unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        if (tid == 0) { sh_prefix = 0u; sh_u64 = 0; }
        __syncthreads();
        unsigned long long above_run = 0;            // weight strictly above the prefix (the same in every thread)
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 32 * 256; i += SAMPLE_THREADS) { warp_w[i] = 0; warp_c[i] = 0; }
            __syncthreads();
            const unsigned prefix = sh_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < n; i += SAMPLE_THREADS) {
                const float v = seg[i];
                const unsigned k = order_key(v);
                if ((k & mask) != prefix || !kept(k, lo + i, tk)) continue;
                const int b = my_warp * 256 + ((k >> shift) & 255);
                atomicAdd(&warp_w[b], weight_fx(v));
                atomicAdd(&warp_c[b], 1);
            }
            __syncthreads();
            if (tid < 256) {
                unsigned long long w = 0;
                int c = 0;
#pragma unroll 8
                for (int wi = 0; wi < 32; ++wi) { w += warp_w[wi * 256 + tid]; c += warp_c[wi * 256 + tid]; }
                X.hist_w[par][tid] = w;
                X.hist_c[par][tid] = c;
            }
            exchange_hist(true);
            if (tid == 0) {
                unsigned long long above = above_run;
                int b = -1, lowest = -1;
                for (int c = 255; c >= 0; --c) {
                    if (tot_c[c] == 0) continue;
                    lowest = c;
                    if (above + tot_w[c] >= target) { b = c; break; }
                    above += tot_w[c];
                }
                if (b < 0) { b = lowest; above -= tot_w[lowest]; }
                sh_u64 = above;
                sh_u64b = tot_w[b];
                sh_int = tot_c[b];
                sh_prefix = prefix | ((unsigned)b << shift);
            }
            __syncthreads();
            above_run = sh_u64;
            __syncthreads();
        }
        tp.key = sh_prefix;
        const unsigned long long above = above_run, tie_w = sh_u64b;
        const int ties = sh_int;
        __syncthreads();
        int need = ties;
        if (ties > 1 && tie_w > 0) {
            const unsigned long long each = tie_w / (unsigned long long)ties;
            if (each > 0 && target > above) {
                const unsigned long long nn = (target - above + each - 1) / each;
                need = nn < 1 ? 1 : (nn > (unsigned long long)ties ? ties : (int)nn);
            } else {
                need = 1;
            }
        }
        tp.cut = nth_equal(tp.key, need, tk);
    }

    // the draw: r = u * kept weight; walk the kept set in index order
    double mine = 0.0;
    int last_kept = -1;
    for (int i = t0; i < t1; ++i) {
        const float v = seg[i];
        if (kept(order_key(v), lo + i, tp)) { mine += (double)weight(v); last_kept = lo + i; }
    }
    double block_sum_;
    const double before_block = block_excl_scan(mine, redd, &block_sum_);
    __syncthreads();
    if (tid == 0) X.d[par] = block_sum_;
    cluster.sync();
    if (tid == 0) {
        double tot = 0.0, b = 0.0;
        for (int r = 0; r < SC_CLUSTER; ++r) {
            const double v = cluster.map_shared_rank(&X, r)->d[par];
            if (r < rank) b += v;
            tot += v;
        }
        sh_d[0] = tot;
        sh_d[1] = b;
    }
    __syncthreads();
    const double kept_sum = sh_d[0], before = sh_d[1] + before_block;
    par ^= 1;
    const unsigned long long h = splitmix64(seed ^ splitmix64(((unsigned long long)(unsigned)request[row] << 32) |
                                                              (unsigned)position[row]));
    const double u = (double)(h >> 40) * (1.0 / 16777216.0);
    const double r = u * kept_sum;
    if (tid == 0) sh_int = -1;
    __syncthreads();
    if (mine > 0.0 && before <= r && r < before + mine) {
        double cum = before;
        int pick = -1, last = -1;
        for (int i = t0; i < t1; ++i) {
            const float v = seg[i];
            if (!kept(order_key(v), lo + i, tp)) continue;
            last = lo + i;
            cum += (double)weight(v);
            if (r < cum) { pick = lo + i; break; }
        }
        atomicMax(&sh_int, pick >= 0 ? pick : last);
    }
    __syncthreads();
    const int mine_pick = sh_int;
    __syncthreads();
    int found = exchange_int(mine_pick, false);
    if (found < 0) {
        // rounding left r at or beyond the last running sum: the last kept element of the row
        if (tid == 0) sh_int = -1;
        __syncthreads();
        atomicMax(&sh_int, last_kept);
        __syncthreads();
        const int mine_last = sh_int;
        __syncthreads();
        found = exchange_int(mine_last, false);
    }
    if (rank == 0 && tid == 0) out[row] = found < 0 ? 0 : found;
    cluster.sync();          // no block leaves while another may still read its shared memory
}

// the longest row the cluster form takes: an eighth of it, the per-warp histograms and the
// exchange buffers have to fit a block's shared memory
#define SC_MAX_CHUNK ((232448 - 32 * 256 * 12 - 12 * 1024) / 4)

// form 0: the cluster form where the row fits it and the rows fit the GPU at once, else one block per row;
// 1: one block per row; 2: the cluster form
extern "C" int zlm_sample(int* out, const float* logits, int R, int V, int ld, float temperature, int top_k,
                          float top_p, unsigned long long seed, const int* request, const int* position, int form,
                          cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%d", R, V, ld);
    ZLM_REQUIRE(temperature > 0.f, "sample: temperature must be positive (greedy is argmax)");
    ZLM_REQUIRE(top_k >= 0 && top_p > 0.f, "sample: top_k=%d top_p=%f", top_k, top_p);
    const size_t hist = (size_t)32 * 256 * (sizeof(unsigned long long) + sizeof(int));
    const int chunk = ((V + SC_CLUSTER - 1) / SC_CLUSTER + 3) / 4 * 4;
    // measured at 151,936 logits a row: the cluster form takes 15 / 43 / 140 us (temperature / top-k /
    // top-p) at 8 rows against 72 / 179 / 456 us for one block per row; its blocks need most of an
    // SM's shared memory, so with more rows than fit the GPU at once (8 blocks each) it falls behind
    // (64 rows: 636 us against 458 for top-p)
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const bool fits = chunk <= SC_MAX_CHUNK;
    if (form == 2 ? fits : (form == 0 && fits && R * SC_CLUSTER <= sms)) {
        // the cluster form: 8 blocks per row
        const size_t smem = hist + (size_t)chunk * sizeof(float);
        static size_t reserved = 0;
        if (smem > reserved) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) {
                zlm_set_error("sample: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
                return ZLM_ERR_CUDA;
            }
            reserved = smem;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(R * SC_CLUSTER);
        cfg.blockDim = dim3(SAMPLE_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = SC_CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = zlm_pdl_enabled() ? 2 : 1;
        cudaLaunchKernelEx(&cfg, sample_cluster_kernel, out, logits, V, ld, temperature, top_k, top_p, seed, request, position,
                           chunk);
        return zlm_check_launch("sample (cluster)");
    }
    ZLM_REQUIRE(form != 2, "sample: a row of %d logits is too long for the cluster form", V);
    ZLM_REQUIRE(form >= 0 && form <= 2, "sample: form %d", form);
    const size_t smem = hist;
    static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            zlm_set_error("sample: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        attr_set = true;
    }
    zlm_launch(sample_kernel, R, SAMPLE_THREADS, smem, st, out, logits, V, ld, temperature, top_k, top_p, seed, request,
               position);
    return zlm_check_launch("sample");
}

extern "C" unsigned long long zlm_sample_hash(unsigned long long seed, int request, int position) {
    return splitmix64(seed ^ splitmix64(((unsigned long long)(unsigned)request << 32) | (unsigned)position));
}

ZLM_TRANSLATION_UNIT(sampling)
