// Row functions of the embedding gather and of RMSNorm, as functions of a group of threads
// (the kernels in elementwise.cu run them with the block as the group).
#pragma once
#include "common.cuh"

// out[0..H) = table[id, :] widened to fp32, by `nthreads` threads
template <typename TW>
__device__ __forceinline__ void embed_row(float* o, const TW* table, int id, int H, int V, int tid, int nthreads) {
    // ids are validated on the host; clamp so that a bad id can never read
    // outside the table
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const TW* row = table + (size_t)id * H;
    if (!ZLM_CHK(row, (size_t)H * sizeof(TW))) return;
    if (sizeof(TW) == 2 && H % 8 == 0) {
        // 16-byte loads, two 16-byte stores
        for (int c = tid; c < H / 8; c += nthreads) {
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
    for (int i = tid; i < H; i += nthreads) o[i] = to_f32(row[i]);
}

// four consecutive outputs, i a multiple of 4, as one store
__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
    *(float4*)o = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* o, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *(unsigned*)&lo;
    u.y = *(unsigned*)&hi;
    *(uint2*)o = u;
}

// RMSNorm of one row as a block of `vthreads` threads computes it (the order of the sum
// is that block's), carried out by the gs.threads threads of a group, each of which plays
// up to VPT of the block's threads: thread tid plays tid, tid + gs.threads, ...  A group
// that is the block itself has VPT = 1.  `red` holds 32 floats.
// With H a multiple of 4 every thread keeps its float4s in registers between the
// sum and the scaling, so the row is read once and the latency is one load deep.
#define NORM_MAX_V4 4
template <typename TO, int VPT>
__device__ __forceinline__ void rmsnorm_row(TO* o, const float* xr, VecW w, int H, float eps, float* red,
                                            const int tid, const GroupSync gs, const int vthreads) {
    const int lane = tid & 31, warp = tid >> 5;
    const int rwarps = gs.threads >> 5, nw = (vthreads + 31) >> 5;
    const int nv = H / 4;
    const bool in_regs = H % 4 == 0 && nv <= NORM_MAX_V4 * vthreads;
    if (in_regs) {
        // the weights are wanted only after the sum: start them on their way to L1 now
        const int line = (w.dtype == ZLM_DTYPE_F32 ? 32 : 64);            // elements per 128 bytes
        for (int i = tid * line; i < H; i += gs.threads * line)
            asm volatile("prefetch.global.L1 [%0];\n" ::"l"((const char*)w.p + (size_t)i * (w.dtype == ZLM_DTYPE_F32 ? 4 : 2)));
    }
    float4 v[VPT][NORM_MAX_V4];
    float s[VPT];
#pragma unroll
    for (int p = 0; p < VPT; ++p) {
        const int vt = tid + p * gs.threads;
        s[p] = 0.f;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < NORM_MAX_V4; ++j) {
                const int c = vt + j * vthreads;
                v[p][j] = (vt < vthreads && c < nv) ? *(const float4*)(xr + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                s[p] = fmaf(v[p][j].x, v[p][j].x, s[p]); s[p] = fmaf(v[p][j].y, v[p][j].y, s[p]);
                s[p] = fmaf(v[p][j].z, v[p][j].z, s[p]); s[p] = fmaf(v[p][j].w, v[p][j].w, s[p]);
            }
        } else if (vt < vthreads) {
            for (int i = vt; i < H; i += vthreads) {
                const float a = xr[i];
                s[p] = fmaf(a, a, s[p]);
            }
        }
        s[p] = warp_sum(s[p]);
    }
    gs.sync();
#pragma unroll
    for (int p = 0; p < VPT; ++p)
        if (lane == 0 && warp + p * rwarps < nw) red[warp + p * rwarps] = s[p];
    gs.sync();
    float tot = (lane < nw) ? red[lane] : 0.f;
    tot = warp_sum(tot);
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
#pragma unroll
    for (int p = 0; p < VPT; ++p) {
        const int vt = tid + p * gs.threads;
        if (vt >= vthreads) continue;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < NORM_MAX_V4; ++j) {
                const int c = vt + j * vthreads;
                if (c < nv) {
                    const int i = c * 4;
                    const float4 wv = w.load4(i);
                    store4(o + i, (v[p][j].x * inv) * wv.x, (v[p][j].y * inv) * wv.y, (v[p][j].z * inv) * wv.z,
                           (v[p][j].w * inv) * wv.w);
                }
            }
        } else {
            for (int i = vt; i < H; i += vthreads) o[i] = from_f32<TO>((xr[i] * inv) * w[i]);
        }
    }
}
