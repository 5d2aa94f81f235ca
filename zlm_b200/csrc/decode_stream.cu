// A whole bf16 decode step (up to 8 tokens) as ONE persistent kernel.
//
// A decode step is a chain of a few hundred short operations, each bound by reading its
// weights once.  As separate kernels every one of them pays a launch, the latency of its
// first loads and a drain, during which nothing streams from memory.  Here one block per
// SM stays resident for the whole step and carries out a list of operations (zlm_stream.h)
// in order:
//
//   * warp 0 of every block is a producer.  It walks the list ahead of the others and
//     brings the weight tiles this block will need into a ring of shared-memory slots
//     with TMA (cp.async.bulk.tensor + mbarrier; the tensor maps lie in global memory
//     beside the program).  Weights do not depend on the step's activations, so the
//     producer never waits for a grid-wide barrier: while the other warps wait for the
//     operation before to finish everywhere, the weights of the next product are already
//     landing, and the stream from memory does not stop.
//   * warps 1..8 are consumers.  They carry out the operations: the weight-streaming
//     product (tiles of W from the ring, the step's activations staged once per product
//     in shared memory, tensor-core m16n8k16 with the k of a fragment taken where a
//     16-byte load puts them), and, through the same functions that the stand-alone
//     kernels are made of, embedding, RMSNorm, q/k norm + rotation + cache write,
//     split-KV attention and its combine.  Between operations that depend on each other
//     they pass a barrier over all blocks (a counter in global memory; the launch is
//     cooperative, so all blocks are resident).
//
// A product cuts the rows of W into units of UR <= 16 rows (UR chosen per product so that
// every block gets the same number of rows to within one unit) and deals contiguous runs
// of units to the blocks.  A unit sweeps K in stages of 512 columns: one slot of the
// ring, two TMA boxes of UR x 256.  Stage s of every 8 belongs to consumer warp s, which
// multiplies its 16 blocks of 32 columns in ascending k on four chains of sums; a row's
// partial sums are then added over the warps in ascending order: the same order as
// gemv_bf16.cu, so the step's results are those of the stand-alone kernels bit for bit.
// A thread keeps its fragments of the activations [T, K] in registers for all units of a
// product (every block would otherwise pull them from L2 once per unit, half as many
// bytes again as the weights); a K longer than 8 stages is taken in chunks, the partial
// sums of up to ST_MAXU units kept in shared memory between chunks.
//
// Measured on a B200 at Qwen3-8B sizes, 8 tokens: the products alone stream their
// weights at 4.4 TB/s with the barriers between them (5.4 TB/s without; the stand-alone
// kernels in a CUDA graph reach 4.7 TB/s).  What an operation pays at its start cannot be
// hidden behind the ring: about 1.8 us for the barrier and 2 us until 148 blocks have
// pulled the same 64 KB of activations out of L2, which the 160 KB of weights that landed
// meanwhile only win back if the consumers then run well above the memory's rate; they
// run at about 1.2 times it.  A whole step is slower than the graph of stand-alone
// kernels, so the engine uses this kernel only when asked to.
//
// Every wait (mbarrier, grid barrier) gives up after two seconds, sets an error word
// (zlm_stream_status) and an abort flag that ends all other waits at once; the kernel
// then walks on to its end with whatever it has, so that no thread is left at a barrier.
// (src/runtime/executor.zig:160-420 is the reference's per-token walk over the same
// operations; src/kernels/linear/matvec/form/fused.zig:27-86 its fused products.)
#include "common.cuh"
#include <stdio.h>

#include "attention_decode.cuh"
#include "elementwise.cuh"
#include "rope_kv.cuh"
#include "tc_common.cuh"
#include "zlm_stream.h"

#define ST_CWARPS 8
#define ST_CONSUMERS (ST_CWARPS * 32)
#define ST_THREADS (ST_CONSUMERS + 32)
#define ST_STAGE_K 512
#define ST_SLOT_BYTES (ST_STAGE_K * 32)          // 16 rows of a stage
#define ST_STAGE_BLOCKS (ST_STAGE_K / 32)        // 32-column blocks of a stage
#ifndef ST_SLOTS
#define ST_SLOTS 10
#endif
#define ST_BOX_K 256                            // columns of a TMA box (the most a box takes)
#define ST_BOX_BYTES 8192                       // 16 rows x 512 bytes
#define ST_CHUNK_K (ST_CWARPS * ST_STAGE_K)     // columns of K that the warps sweep at a time, a stage each
#define ST_UNIT 16
#define ST_MAXU 4                               // units whose partial sums are kept between chunks of K
#define ST_GROUP_BYTES 65536                    // shared memory of the non-product operations, and the products' partial sums
#define ST_RED_UNIT (ST_CONSUMERS * 16)          // floats per unit: 16 of its own for every consumer thread
#define ST_RED_FLOATS (ST_MAXU * ST_RED_UNIT)
#define ST_WAIT_NS 2000000000ull                // a wait gives up after two seconds

#define ST_OFF_GROUP (ST_SLOTS * ST_SLOT_BYTES)
#define ST_OFF_RED ST_OFF_GROUP                 // a product uses the area while no other operation does
#define ST_OFF_OPS (ST_OFF_GROUP + ST_GROUP_BYTES)
#define ST_OFF_BARS (ST_OFF_OPS + 2 * 192)
#define ST_OFF_FLAG (ST_OFF_BARS + 2 * ST_SLOTS * 8)
#define ST_SMEM_BYTES (ST_OFF_FLAG + 16)
static_assert(ST_RED_FLOATS * 4 <= ST_GROUP_BYTES, "the partial sums must fit the shared area");
static_assert(ST_SMEM_BYTES <= 232448, "more shared memory than a block can have");

static __device__ int g_stream_error = 0;

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ unsigned st_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void st_bar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(st_smem(bar)), "r"(count));
}
__device__ __forceinline__ void st_bar_expect(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(st_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(st_smem(bar)) : "memory");
}
__device__ __forceinline__ bool st_bar_try(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(st_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long st_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
// bounded by time (a try_wait may itself block for a while, so polls are not counted);
// false if it gave up or somebody else did
__device__ __forceinline__ bool st_bar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, int where) {
    if (st_bar_try(bar, parity)) return true;
    const unsigned long long t0 = st_now_ns();
    for (unsigned it = 1;; ++it) {
        if (st_bar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((it & 63) == 0 && st_now_ns() - t0 > ST_WAIT_NS) break;
    }
    *abort_flag = where;
    atomicCAS(&g_stream_error, 0, where);
    return false;
}
__device__ __forceinline__ void st_bulk_copy(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(st_smem(dst)), "l"(src), "r"(bytes), "r"(st_smem(bar)) : "memory");
}
__device__ __forceinline__ uint4 st_lds16(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(st_smem(p)));
    return v;
}
// activations are written by other blocks during this kernel: read them past L1
__device__ __forceinline__ uint4 st_ldcg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned st_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// How a product is cut for block b of nb: units of UR rows, this block's run of units
// [u_lo, u_hi), chunks of KC columns of K (a thread keeps its activation fragments of one
// chunk in registers), and groups of gsize units that sweep one chunk after the other.
struct StreamCut {
    int UR, u_lo, u_hi, KC, chunks, gsize;
};
__device__ __forceinline__ StreamCut st_cut(const ZlmStreamOp* op, int b, int nb) {
    StreamCut c;
    const int N = op->i[1], K = op->i[2];
    c.UR = op->i[6];
    const long long U = (N + c.UR - 1) / c.UR;
    c.u_lo = (int)(U * b / nb);
    c.u_hi = (int)(U * (b + 1) / nb);
    c.KC = ST_CHUNK_K;
    c.chunks = (K + c.KC - 1) / c.KC;
    c.gsize = c.chunks == 1 ? 1 : ST_MAXU;
    return c;
}

struct StreamCtx {
    unsigned char* smem;
    uint64_t* full;
    uint64_t* empty;
    volatile int* abort_flag;
};

__device__ __forceinline__ void st_tma_2d(void* dst, const void* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(st_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(st_smem(bar)) : "memory");
}

// ---------------------------------------------------------------- the producer warp
// One lane issues; the walk over (group, chunk, unit, stage) is the consumers' walk.
__device__ __forceinline__ void st_producer(const ZlmStreamOp* ops, int n_ops, const StreamCtx& c) {
    if ((threadIdx.x & 31) != 0) return;
    unsigned n = 0;                                   // stages issued so far, over all products
    for (int oi = 0; oi < n_ops; ++oi) {
        const ZlmStreamOp* op = ops + oi;
        if (op->type != ZLM_STREAM_GEMV) continue;
        const int K = op->i[2];
        const void* map = op->p[3];
        const StreamCut cut = st_cut(op, blockIdx.x, gridDim.x);
        if (cut.u_lo >= cut.u_hi) continue;
        // the map was written by the host: make this block's TMA unit see it
        asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;\n" ::"l"(map) : "memory");
        for (int g0 = cut.u_lo; g0 < cut.u_hi; g0 += cut.gsize) {
            const int g1 = min(cut.u_hi, g0 + cut.gsize);
            for (int ch = 0; ch < cut.chunks; ++ch) {
                const int kc1 = min(K, (ch + 1) * cut.KC);
                for (int u = g0; u < g1; ++u) {
                    for (int k0 = ch * cut.KC; k0 < kc1; k0 += ST_STAGE_K, ++n) {
                        const unsigned slot = n % ST_SLOTS, round = n / ST_SLOTS;
                        if (!st_bar_wait(c.empty + slot, (round & 1) ^ 1, c.abort_flag, 1)) return;
                        const int boxes = (min(K - k0, ST_STAGE_K) + ST_BOX_K - 1) / ST_BOX_K;
                        st_bar_expect(c.full + slot, (unsigned)(boxes * cut.UR * ST_BOX_K * 2));
                        unsigned char* dst = c.smem + slot * ST_SLOT_BYTES;
                        for (int bx = 0; bx < boxes; ++bx)
                            st_tma_2d(dst + bx * ST_BOX_BYTES, map, k0 + bx * ST_BOX_K, u * cut.UR, c.full + slot);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------- grid-wide barrier (consumers)
__device__ __forceinline__ void st_consumer_sync() {
    asm volatile("bar.sync 3, %0;\n" ::"n"(ST_CONSUMERS) : "memory");
}
__device__ __forceinline__ void st_grid_barrier(unsigned* counter, unsigned target, const StreamCtx& c, int ctid) {
    st_consumer_sync();
    if (ctid == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        bool ok = false;
        const unsigned long long t0 = st_now_ns();
        for (unsigned it = 1;; ++it) {
            if (st_ld_acquire(counter) >= target) { ok = true; break; }
            if (*c.abort_flag) break;
            if ((it & 63) == 0) {
                if (*(volatile int*)&g_stream_error) *c.abort_flag = 4;      // another block gave up
                else if (st_now_ns() - t0 > ST_WAIT_NS) break;
            }
        }
        if (!ok && !*c.abort_flag) {
            *c.abort_flag = 2;
            atomicCAS(&g_stream_error, 0, 2);
        }
        __threadfence();
    }
    st_consumer_sync();
}

// ---------------------------------------------------------------- the streaming product (consumers)
__device__ __forceinline__ void st_cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(st_smem(smem)), "l"(gmem) : "memory");
}

// One unit's rows are complete: every consumer thread has left its four sums (rows g and
// g + 8, tokens 2q and 2q + 1) in the first four of its 16 floats.  The sum of (row, token)
// over the warps, in ascending order:
__device__ __forceinline__ float st_row_sum(const float* red, int row, int tok) {
    const float* p = red + (((row & 7) * 4 + (tok >> 1)) * 16 + (row >> 3) * 2 + (tok & 1));
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < ST_CWARPS; ++w) s += p[w * 32 * 16];
    return s;
}
// where element e (0..127: row e % 16, token e / 16) of a unit goes, or -1 (a product whose
// epilogue is the fused gate/up has its own mapping and nothing to read first)
__device__ __forceinline__ long long st_unit_offset(int T, int ldy, int mode, int row0, int rows, int e) {
    const int tok = e / ST_UNIT, row = e % ST_UNIT;     // rows fastest: coalesced stores
    return (mode != 3 && tok < T && row < rows) ? (long long)tok * ldy + row0 + row : -1;
}
// `resid`: what the output held before (read early, so that the unit does not end with a
// load and a store that depends on it); used by the accumulating product only
__device__ __forceinline__ void st_unit_epilogue(const float* red, void* Y, int T, int N, int ldy, int mode, int row0,
                                                 int rows, int e, float resid) {
    if (mode == 3) {
        if (e < 64) {
            const int tok = e >> 3, row = e & 7;
            if (tok < T && row0 + row + 8 < N) {
                const float sg = st_row_sum(red, row, tok), su = st_row_sum(red, row + 8, tok);
                ((__nv_bfloat16*)Y)[(size_t)tok * ldy + row0 / 2 + row] = __float2bfloat16_rn((sg / (1.0f + expf(-sg))) * su);
            }
        }
        return;
    }
    const long long o = st_unit_offset(T, ldy, mode, row0, rows, e);
    if (o >= 0) {
        const float s_ = st_row_sum(red, e % ST_UNIT, e / ST_UNIT);
        if (mode == 0) ((__nv_bfloat16*)Y)[o] = __float2bfloat16_rn(s_);
        else if (mode == 1) ((float*)Y)[o] = resid + s_;
        else ((float*)Y)[o] = s_;
    }
}

// n: the ring's stage counter, kept in step with the producer's
__device__ __noinline__ unsigned st_gemv(const ZlmStreamOp* op, unsigned char* const smem, unsigned n, const int ctid) {
    // everything the loop needs is in registers: nothing is read through a pointer to the
    // caller's frame, which every asm statement with a memory clobber would force to be read again
    uint64_t* const full = (uint64_t*)(smem + ST_OFF_BARS);
    uint64_t* const empty = full + ST_SLOTS;
    volatile int* const abort_flag = (volatile int*)(smem + ST_OFF_FLAG);
    const int T = op->i[0], N = op->i[1], K = op->i[2], ldx = op->i[3], ldy = op->i[4], mode = op->i[5];
    void* Y = (void*)op->p[0];
    const __nv_bfloat16* X = (const __nv_bfloat16*)op->p[1];
    const int lane = ctid & 31, warp = ctid >> 5;
    const int g = lane >> 2, q = lane & 3;
    float* red = (float*)(smem + ST_OFF_RED);                // [unit or parity][consumer thread][16]
    const StreamCut cut = st_cut(op, blockIdx.x, gridDim.x);
    if (cut.u_lo >= cut.u_hi) return n;
    const int mine = ctid * 16;                              // this thread's own 16 floats in a unit's red
    // A stage (512 columns of a unit's rows) belongs to ONE warp: stage s of a chunk to warp s.
    // A wait on a slot and its release cost a few hundred cycles; a warp that takes a whole
    // stage pays them once per 16 KB and the eight warps work on eight stages at a time.
    // The stage lies in the slot as two boxes of 256 columns, rows 512 bytes apart (a TMA
    // request costs its issuing thread about a hundred cycles whatever its size, so boxes are as
    // large as they can be; that rules out the swizzled layouts, 128 bytes per row at most, and
    // costs the loads below two-way bank conflicts, which the shared-memory pipe has room for).
    const unsigned woff = g * (ST_BOX_K * 2) + q * 16;       // row g, this thread's 16 bytes of a 32-column block

    // the activation fragments of this warp's stage of one chunk of K: this thread's 8 k of
    // each of the 16 blocks, the same for every unit (zero beyond K and beyond the step's tokens)
    uint4 xr[ST_STAGE_BLOCKS];
    const __nv_bfloat16* xrow = X + (size_t)(g < T ? g : 0) * ldx + warp * ST_STAGE_K + q * 8;
    int parity = 0;
    for (int g0 = cut.u_lo; g0 < cut.u_hi; g0 += cut.gsize) {
        const int g1 = min(cut.u_hi, g0 + cut.gsize);
        for (int ch = 0; ch < cut.chunks; ++ch) {
            const int kc0 = ch * cut.KC, kc1 = min(K, kc0 + cut.KC);
            const int stages = (kc1 - kc0 + ST_STAGE_K - 1) / ST_STAGE_K;     // of this chunk, per unit
            const int k0 = kc0 + warp * ST_STAGE_K;                           // this warp's stage starts here
            if (cut.chunks > 1 || g0 == cut.u_lo) {
#pragma unroll
                for (int i = 0; i < ST_STAGE_BLOCKS; ++i)
                    xr[i] = (g < T && k0 + i * 32 + q * 8 < K) ? st_ldcg16(xrow + kc0 + i * 32) : make_uint4(0, 0, 0, 0);
            }
            for (int u = g0; u < g1; ++u) {
                float* ured = red + (cut.chunks == 1 ? parity : u - g0) * ST_RED_UNIT;
                float resid = 0.f;
                if (cut.chunks == 1 && mode == 1 && ctid < ST_UNIT * 8) {
                    const long long o = st_unit_offset(T, ldy, mode, u * cut.UR, min(cut.UR, N - u * cut.UR), ctid);
                    if (o >= 0) resid = __ldcg((const float*)Y + o);
                }
                // four chains of sums, as in gemv_bf16.cu: chain 2 * (i & 1) + h takes the h-th 16 k of
                // the warp's 32-column block i
                float acc[4][4];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[cc][r] = ch > 0 ? ured[mine + cc * 4 + r] : 0.f;
                if (warp < stages) {
                    const unsigned ns = n + warp;
                    const unsigned slot = ns % ST_SLOTS, round = ns / ST_SLOTS;
                    // one lane polls; the warp barrier passes what it saw on to the others.  After a
                    // wait that gave up the walk goes on (with garbage) so that every thread still
                    // reaches every barrier; all later waits return at once
                    if (lane == 0) st_bar_wait(full + slot, round & 1, abort_flag, 3);
                    __syncwarp();
                    const unsigned char* sb = smem + slot * ST_SLOT_BYTES + woff;
#pragma unroll
                    for (int i0 = 0; i0 < ST_STAGE_BLOCKS; i0 += 4) {
                        // columns beyond K inside a box are zeros (and so are the activations there);
                        // boxes beyond K are not loaded at all: the same for the whole warp
                        if (k0 + i0 * 32 < K) {
                            uint4 a[4], b[4];
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const unsigned char* wp = sb + ((i0 + v) >> 3) * ST_BOX_BYTES + ((i0 + v) & 7) * 64;
                                a[v] = st_lds16(wp);
                                b[v] = st_lds16(wp + 8 * ST_BOX_K * 2);
                            }
                            if (i0 + 4 == ST_STAGE_BLOCKS) {
                                // the last fragments are on their way to registers: the slot goes back
                                __syncwarp();
                                if (lane == 0) st_bar_arrive(empty + slot);
                            }
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const uint4 x = xr[i0 + v];
                                st_mma(acc[2 * (v & 1)], a[v].x, b[v].x, a[v].y, b[v].y, x.x, x.y);
                                st_mma(acc[2 * (v & 1) + 1], a[v].z, b[v].z, a[v].w, b[v].w, x.z, x.w);
                            }
                        } else if (i0 + 4 == ST_STAGE_BLOCKS) {
                            __syncwarp();
                            if (lane == 0) st_bar_arrive(empty + slot);
                        }
                    }
                }
                n += stages;
                if (ch + 1 < cut.chunks) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
#pragma unroll
                        for (int r = 0; r < 4; ++r) ured[mine + cc * 4 + r] = acc[cc][r];
                } else {
#pragma unroll
                    for (int r = 0; r < 4; ++r) ured[mine + r] = (acc[0][r] + acc[1][r]) + (acc[2][r] + acc[3][r]);
                }
                if (cut.chunks == 1) {
                    // the unit is complete.  Two buffers take turns, so one barrier per unit is enough:
                    // a buffer is written again only after the barrier of the unit in between
                    st_consumer_sync();
                    const int row0 = u * cut.UR;
                    if (ctid < ST_UNIT * 8) st_unit_epilogue(ured, Y, T, N, ldy, mode, row0, min(cut.UR, N - row0), ctid, resid);
                    parity ^= 1;
                }
            }
        }
        if (cut.chunks > 1) {
            // (the outputs' old values are few and this happens once per group: they are read here)
            st_consumer_sync();
            for (int e = ctid; e < (g1 - g0) * ST_UNIT * 8; e += ST_CONSUMERS) {
                const int ui = e / (ST_UNIT * 8), row0 = (g0 + ui) * cut.UR, rows = min(cut.UR, N - row0);
                const long long o = mode == 1 ? st_unit_offset(T, ldy, mode, row0, rows, e % (ST_UNIT * 8)) : -1;
                st_unit_epilogue(red + ui * ST_RED_UNIT, Y, T, N, ldy, mode, row0, rows, e % (ST_UNIT * 8),
                                 o >= 0 ? __ldcg((const float*)Y + o) : 0.f);
            }
            st_consumer_sync();                              // red is written again by the next group
        }
    }
    return n;
}

// ---------------------------------------------------------------- the other operations (consumers)
template <int HD>
__device__ __noinline__ void st_attn_items(const ZlmStreamOp* op, unsigned char* area, int gtid, GroupSync gs) {
    const int T = op->i[0], nkv = op->i[5], splits = op->i[8];
    const int items = T * nkv * splits;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int t = it % T, kvh = (it / T) % nkv, split = it / (T * nkv);
        attention_decode_item<HD, false>(
            area, gtid, gs, t, kvh, split, (__nv_bfloat16*)op->p[0], op->i[1], (const __nv_bfloat16*)op->p[1],
            op->i[2], (const __nv_bfloat16*)op->p[2], (const int*)op->p[3], op->i[3], (const int*)op->p[4],
            (const int*)op->p[5], op->i[4], nkv, op->f[0], op->i[7], splits, op->i[9], (float*)op->p[6],
            (float*)op->p[7]);
        gs.sync();                      // the staging memory is reused by the next item
    }
}

template <int NPL, bool VEC>
__device__ __noinline__ void st_rope_items(const ZlmStreamOp* op, float* sm, int gtid, GroupSync gs, int vgroup,
                                              int n_groups) {
    const int T = op->i[0], nq = op->i[5], nkv = op->i[6];
    const int chunks = (nq + 2 * nkv + ROPE_WARPS - 1) / ROPE_WARPS;
    VecW qw{op->p[1], op->i[9]}, kw{op->p[2], op->i[9]};
    for (int it = vgroup; it < T * chunks; it += n_groups) {
        qk_norm_rope_write_item<__nv_bfloat16, NPL, false, VEC>(
            sm, gtid, gs, it % T, it / T, (__nv_bfloat16*)op->p[0], op->i[1], qw, kw, op->i[2], op->f[0],
            (const float*)op->p[3], op->i[3], (const int*)op->p[4], (const int*)op->p[5], (const int*)op->p[6],
            op->i[4], (__nv_bfloat16*)op->p[7], nq, nkv, op->i[7], op->i[8], ROPE_WARPS);
        gs.sync();
    }
}

__device__ __noinline__ void st_rmsnorm_rows(const ZlmStreamOp* op, float* red, int ctid) {
    const GroupSync all{3, ST_CONSUMERS};
    const int R = op->i[0], H = op->i[1], vthreads = op->i[3];
    const int* rows = (const int*)op->p[3];
    VecW w{op->p[2], op->i[2]};
    for (int r = blockIdx.x; r < R; r += gridDim.x) {
        __nv_bfloat16* o = (__nv_bfloat16*)op->p[0] + (size_t)r * H;
        const float* xr = (const float*)op->p[1] + (size_t)(rows ? rows[r] : r) * H;
        if (vthreads <= ST_CONSUMERS) rmsnorm_row<__nv_bfloat16, 1>(o, xr, w, H, op->f[0], red, ctid, all, vthreads);
        else if (vthreads == 2 * ST_CONSUMERS) rmsnorm_row<__nv_bfloat16, 2>(o, xr, w, H, op->f[0], red, ctid, all, vthreads);
        else rmsnorm_row<__nv_bfloat16, 4>(o, xr, w, H, op->f[0], red, ctid, all, vthreads);
        all.sync();
    }
}

__device__ __forceinline__ void st_other(const ZlmStreamOp* op, const StreamCtx& c, int ctid) {
    unsigned char* area = c.smem + ST_OFF_GROUP;
    const int group = ctid >> 7, gtid = ctid & 127;
    const GroupSync gs{1 + group, 128};
    switch (op->type) {
    case ZLM_STREAM_EMBED: {
        const int T = op->i[0], H = op->i[1], V = op->i[2];
        const int* ids = (const int*)op->p[2];
        for (int t = blockIdx.x; t < T; t += gridDim.x)
            embed_row((float*)op->p[0] + (size_t)t * H, (const __nv_bfloat16*)op->p[1], ids[t], H, V, ctid, ST_CONSUMERS);
        break;
    }
    case ZLM_STREAM_RMSNORM:
        st_rmsnorm_rows(op, (float*)area, ctid);
        break;
    case ZLM_STREAM_ROPE: {
        const int hd = op->i[7];
        float* sm = (float*)(area + group * (ST_GROUP_BYTES / 2));
        const int vg = blockIdx.x * 2 + group, ng = gridDim.x * 2;
        // the same form as the stand-alone kernel takes (the recorder asked zlm_rope_vector_form)
        if (op->i[10] && hd == 64) st_rope_items<2, true>(op, sm, gtid, gs, vg, ng);
        else if (op->i[10] && hd == 128) st_rope_items<4, true>(op, sm, gtid, gs, vg, ng);
        else if (hd <= 32) st_rope_items<1, false>(op, sm, gtid, gs, vg, ng);
        else if (hd <= 64) st_rope_items<2, false>(op, sm, gtid, gs, vg, ng);
        else st_rope_items<4, false>(op, sm, gtid, gs, vg, ng);
        break;
    }
    case ZLM_STREAM_ATTN: {
        if (group != 0) break;          // one group's staging memory fits beside the ring
        switch (op->i[6]) {
        case 16: st_attn_items<16>(op, area, gtid, gs); break;
        case 32: st_attn_items<32>(op, area, gtid, gs); break;
        case 48: st_attn_items<48>(op, area, gtid, gs); break;
        case 64: st_attn_items<64>(op, area, gtid, gs); break;
        case 80: st_attn_items<80>(op, area, gtid, gs); break;
        case 96: st_attn_items<96>(op, area, gtid, gs); break;
        case 112: st_attn_items<112>(op, area, gtid, gs); break;
        case 128: st_attn_items<128>(op, area, gtid, gs); break;
        }
        break;
    }
    case ZLM_STREAM_COMBINE: {
        const int T = op->i[0], nq = op->i[2];
        float* fs = (float*)(area + group * (ST_GROUP_BYTES / 2));
        float* red = fs + COMB_MAX_SPLITS;
        for (int it = blockIdx.x * 2 + group; it < T * nq; it += gridDim.x * 2) {
            attention_decode_combine_item(fs, red, gtid, gs, it % T, it / T, (__nv_bfloat16*)op->p[0], op->i[1],
                                          (const float*)op->p[1], (const float*)op->p[2], (const int*)op->p[3], nq,
                                          op->i[3], op->i[4], op->i[5], op->i[6]);
            gs.sync();
        }
        break;
    }
    default: break;
    }
}

// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(ST_THREADS, 1)
decode_stream_kernel(const ZlmStreamOp* ops, int n_ops, unsigned* counter) {
    extern __shared__ __align__(1024) unsigned char smem[];
    StreamCtx c;
    c.smem = smem;
    c.full = (uint64_t*)(smem + ST_OFF_BARS);
    c.empty = c.full + ST_SLOTS;
    c.abort_flag = (volatile int*)(smem + ST_OFF_FLAG);
    if (threadIdx.x == 0) {
        for (int s = 0; s < ST_SLOTS; ++s) {
            st_bar_init(c.full + s, 1);
            st_bar_init(c.empty + s, 1);                 // the one warp that read the stage
        }
        *c.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        st_producer(ops, n_ops, c);
    } else {
        const int ctid = threadIdx.x - 32;
        // the records are fetched one operation ahead into shared memory, so that an operation
        // does not start with a chain of loads from global memory
        unsigned char* opbuf = smem + ST_OFF_OPS;                       // 2 x 192 bytes
        constexpr int OP16 = (int)sizeof(ZlmStreamOp) / 16;
        if (ctid < OP16) st_cp_async16(opbuf + ctid * 16, (const unsigned char*)ops + ctid * 16);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        unsigned n = 0, passed = 0;
        for (int oi = 0; oi < n_ops; ++oi) {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            st_consumer_sync();                                          // record oi is there; oi - 1 is done with
            if (oi + 1 < n_ops && ctid < OP16)
                st_cp_async16(opbuf + ((oi + 1) & 1) * 192 + ctid * 16, (const unsigned char*)(ops + oi + 1) + ctid * 16);
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            const ZlmStreamOp* op = (const ZlmStreamOp*)(opbuf + (oi & 1) * 192);
            if (op->barrier) {
                ++passed;
                st_grid_barrier(counter, passed * gridDim.x, c, ctid);
            }
            if (op->type == ZLM_STREAM_GEMV) {
                n = st_gemv(op, smem, n, ctid);
            } else {
                st_other(op, c, ctid);
            }
        }
    }
    __syncthreads();
    if (*c.abort_flag) {
        // give copies that are still in flight time to land before the block's shared
        // memory is given away (they complete within microseconds)
        for (int i = 0; i < 50; ++i) __nanosleep(10000);
    }
}

// ---------------------------------------------------------------- host side
// checks a program (host copy) before it is ever launched: a size or an alignment that the
// kernel does not take is refused here, with the operation's index
extern "C" int zlm_stream_validate(const ZlmStreamOp* ops, int n_ops) {
    ZLM_REQUIRE(ops && n_ops > 0, "decode stream: empty program");
    for (int oi = 0; oi < n_ops; ++oi) {
        const ZlmStreamOp& op = ops[oi];
        switch (op.type) {
        case ZLM_STREAM_EMBED:
            ZLM_REQUIRE(op.i[0] >= 1 && op.i[1] >= 1 && op.i[2] >= 1, "decode stream: op %d: embed sizes T=%d H=%d V=%d", oi,
                        op.i[0], op.i[1], op.i[2]);
            ZLM_REQUIRE(op.i[1] % 8 || (uintptr_t)op.p[1] % 16 == 0, "decode stream: op %d: table not 16-byte aligned", oi);
            break;
        case ZLM_STREAM_RMSNORM: {
            const int v = op.i[3];
            ZLM_REQUIRE(op.i[0] >= 1 && op.i[1] >= 1, "decode stream: op %d: rmsnorm sizes R=%d H=%d", oi, op.i[0], op.i[1]);
            ZLM_REQUIRE(v == 128 || v == 256 || v == 512 || v == 1024, "decode stream: op %d: rmsnorm block of %d threads", oi, v);
            ZLM_REQUIRE(op.i[1] % 4 != 0 || ((uintptr_t)op.p[0] % 16 == 0 && (uintptr_t)op.p[1] % 16 == 0 && (uintptr_t)op.p[2] % 16 == 0),
                        "decode stream: op %d: rmsnorm input, weight and output must be 16-byte aligned", oi);
            break;
        }
        case ZLM_STREAM_GEMV: {
            const int T = op.i[0], N = op.i[1], K = op.i[2], ldx = op.i[3], mode = op.i[5], UR = op.i[6];
            ZLM_REQUIRE(T >= 1 && T <= ZLM_STREAM_MAX_TOKENS, "decode stream: op %d: product of %d tokens (1 to %d)", oi, T,
                        ZLM_STREAM_MAX_TOKENS);
            ZLM_REQUIRE(N >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0,
                        "decode stream: op %d: product N=%d K=%d (row stride %d): K must be a multiple of 8", oi, N, K, ldx);
            ZLM_REQUIRE(mode >= 0 && mode <= 3 && (mode != 3 || N % 16 == 0), "decode stream: op %d: mode %d with N=%d", oi, mode, N);
            ZLM_REQUIRE(UR >= 1 && UR <= ST_UNIT && (mode != 3 || UR == ST_UNIT), "decode stream: op %d: units of %d rows", oi, UR);
            ZLM_REQUIRE((uintptr_t)op.p[1] % 16 == 0 && (uintptr_t)op.p[2] % 16 == 0,
                        "decode stream: op %d: operands not 16-byte aligned", oi);
            ZLM_REQUIRE(op.p[3] && (uintptr_t)op.p[3] % 64 == 0, "decode stream: op %d: tensor map missing or not 64-byte aligned", oi);
            break;
        }
        case ZLM_STREAM_ROPE: {
            const int hd = op.i[7], n_rot = op.i[3];
            ZLM_REQUIRE(hd >= 2 && hd <= 128 && hd % 2 == 0 && n_rot >= 0 && n_rot <= hd && n_rot % 2 == 0,
                        "decode stream: op %d: rotation of %d of head_dim %d", oi, n_rot, hd);
            break;
        }
        case ZLM_STREAM_ATTN: {
            const int nq = op.i[4], nkv = op.i[5], hd = op.i[6], splits = op.i[8];
            ZLM_REQUIRE(nkv > 0 && nq % nkv == 0 && nq / nkv <= 16 && hd % 16 == 0 && hd >= 16 && hd <= 128,
                        "decode stream: op %d: attention with %d heads over %d kv heads of size %d", oi, nq, nkv, hd);
            ZLM_REQUIRE(splits >= 1 && splits <= COMB_MAX_SPLITS && op.i[9] >= 1, "decode stream: op %d: %d splits of %d pages", oi,
                        splits, op.i[9]);
            ZLM_REQUIRE(splits == 1 || (op.p[6] && op.p[7]), "decode stream: op %d: scratch missing for %d splits", oi, splits);
            ZLM_REQUIRE(op.i[2] % 2 == 0 && (uintptr_t)op.p[1] % 4 == 0, "decode stream: op %d: q not 4-byte aligned", oi);
            break;
        }
        case ZLM_STREAM_COMBINE:
            ZLM_REQUIRE(op.i[4] >= 1 && op.i[4] <= COMB_MAX_SPLITS, "decode stream: op %d: %d splits", oi, op.i[4]);
            break;
        default:
            ZLM_REQUIRE(false, "decode stream: op %d has unknown type %d", oi, op.type);
        }
    }
    return ZLM_OK;
}

// rows per unit of a product of N rows: at most 16, chosen so that the units deal out evenly
// over the blocks (N = 4096 over 148 blocks: 28 rows each, two units of 14)
extern "C" int zlm_stream_unit_rows(int N, int mode, int blocks) {
    if (mode == 3 || blocks < 1) return ST_UNIT;
    const int per_block = (N + blocks - 1) / blocks;
    const int units = (per_block + ST_UNIT - 1) / ST_UNIT;
    const int ur = (per_block + units - 1) / units;
    return ur < 1 ? 1 : (ur > ST_UNIT ? ST_UNIT : ur);
}

// the tensor map of a product's weights W [N, K] (bf16, row-major) for boxes of `unit_rows` rows x 256
// columns, written to 128 bytes of host memory; the caller copies it to 64-byte aligned device memory
extern "C" int zlm_stream_make_map(void* map_host, const void* W, int N, int K, int unit_rows) {
    ZLM_REQUIRE(map_host && W && N >= 1 && K >= 8 && K % 8 == 0 && unit_rows >= 1 && unit_rows <= ST_UNIT,
                "decode stream: tensor map for N=%d K=%d units of %d rows", N, K, unit_rows);
    ZlmEncodeTiledFn enc = zlm_tensor_map_encoder();
    ZLM_REQUIRE(enc, "decode stream: the driver does not provide cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {ST_BOX_K, (cuuint32_t)unit_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc((CUtensorMap*)map_host, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)W, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ZLM_REQUIRE(r == CUDA_SUCCESS, "decode stream: cuTensorMapEncodeTiled failed with %d (N=%d K=%d)", (int)r, N, K);
    return ZLM_OK;
}

// blocks the kernel runs with on the current device (one per SM), or 0 if it cannot run there
extern "C" int zlm_stream_blocks() {
    static int blocks = -1;
    if (blocks >= 0) return blocks;
    int dev = 0, sms = 0, coop = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (cudaFuncSetAttribute(decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return blocks = 0;
    }
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stream_kernel, ST_THREADS, ST_SMEM_BYTES);
    blocks = (coop && per_sm >= 1) ? sms : 0;
    return blocks;
}

// runs a validated program that lives in device memory.  `counter` is one 32-bit word of device
// memory for the grid barrier; it is zeroed here, in stream order, before the launch.
extern "C" int zlm_stream_run(const void* ops_dev, int n_ops, unsigned* counter, cudaStream_t st) {
    const int blocks = zlm_stream_blocks();
    ZLM_REQUIRE(blocks > 0, "decode stream: this device cannot run the persistent decode kernel (no cooperative launch, "
                            "or %d bytes of shared memory per block are not available)", (int)ST_SMEM_BYTES);
    ZLM_REQUIRE(ops_dev && counter && n_ops > 0, "decode stream: missing program or counter");
    cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) {
        zlm_set_error("decode stream: memset: %s", cudaGetErrorString(e));
        return ZLM_ERR_CUDA;
    }
    const ZlmStreamOp* ops = (const ZlmStreamOp*)ops_dev;
    void* args[] = {(void*)&ops, (void*)&n_ops, (void*)&counter};
    e = cudaLaunchCooperativeKernel((void*)decode_stream_kernel, dim3(blocks), dim3(ST_THREADS), args, ST_SMEM_BYTES, st);
    if (e != cudaSuccess) {
        zlm_set_error("decode stream: launch: %s", cudaGetErrorString(e));
        return ZLM_ERR_CUDA;
    }
    return zlm_check_launch("decode_stream");
}

// 0 unless a bounded wait inside the kernel ever gave up: 1 producer (slot never freed),
// 2 grid barrier, 3 consumer (slot never filled).  Synchronises.
extern "C" int zlm_stream_status() {
    int v = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&v, g_stream_error, sizeof(int));
    return v;
}


extern "C" int zlm_stream_op_bytes() { return (int)sizeof(ZlmStreamOp); }
