// Shared helpers of the sm_100a kernel library: dtype codes, loads that widen to
// fp32, warp and block reductions with a fixed order, and the error channel of
// the extern "C" entry points.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define ZLM_DTYPE_F32 0
#define ZLM_DTYPE_BF16 1

// tokens per page of the paged cache; the Python side asserts the same value
#define ZLM_PAGE 64

#define ZLM_OK 0
#define ZLM_ERR_ARG 1
#define ZLM_ERR_CUDA 2
#define ZLM_ERR_UNSUPPORTED 3

void zlm_set_error(const char* fmt, ...);
int zlm_check_launch(const char* what);

// ---------------------------------------------------------------------------
// The library's status block: one small structure in pinned host memory that the GPU
// writes directly.  A bounded wait that gives up, or (in the bounds-check build) an
// access outside every registered range, leaves its mark there, and the host reads it
// without synchronising or copying.  Each translation unit has its own device-side
// pointers to the block and to the bounds table (`g_zlm`), bound once per device by zlm_bind_shared(),
// which the library's set-up calls for every translation unit before anything runs.
// ---------------------------------------------------------------------------
#define ZLM_BC_MAX_RANGES 256
struct ZlmShared {                       // pinned host memory
    int status;                          // first give-up: (kernel family << 8) | where
    int bc_violations;                   // accesses refused by the bounds-check build
    int bc_first_site;                   // (file id << 16) | line of the first one
    int pad;
    unsigned long long bc_first_addr;
};
struct ZlmBoundsTable {                  // device memory; only the bounds-check build reads it
    int n, pad;
    unsigned long long lo[ZLM_BC_MAX_RANGES], hi[ZLM_BC_MAX_RANGES];
};
struct ZlmBinding {
    ZlmShared* shared;
    ZlmBoundsTable* bounds;
};
int zlm_runtime_binding(ZlmBinding* out);        // the current device's block and table (made on first use)
static __device__ ZlmBinding g_zlm = {nullptr, nullptr};

static inline int zlm_bind_shared() {
    static bool bound[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        zlm_set_error("cannot tell the current device");
        return ZLM_ERR_CUDA;
    }
    if (bound[dev]) return ZLM_OK;
    ZlmBinding b;
    int rc = zlm_runtime_binding(&b);
    if (rc != ZLM_OK) return rc;
    cudaError_t e = cudaMemcpyToSymbol(g_zlm, &b, sizeof(b));
    if (e != cudaSuccess) {
        zlm_set_error("cannot bind the status block on device %d: %s", dev, cudaGetErrorString(e));
        return ZLM_ERR_CUDA;
    }
    bound[dev] = true;
    return ZLM_OK;
}
// every .cu file ends with ZLM_TRANSLATION_UNIT(name); status.cu lists the names
#define ZLM_TRANSLATION_UNIT(name) extern "C" int zlm_bind_##name() { return zlm_bind_shared(); }

__device__ __forceinline__ void zlm_report_status(int code) {
    ZlmShared* s = g_zlm.shared;
    if (s && *(volatile int*)&s->status == 0) {
        *(volatile int*)&s->status = code;
        __threadfence_system();
    }
}

// The bounds-check build (-DZLM_BOUNDS_CHECK): every global-memory access of the hand-written
// kernels that is not a TMA copy (those are bounded by their tensor maps) first asks
// ZLM_CHK(pointer, bytes); an access that does not lie inside one of the ranges the caller
// registered (the tensors it passed) is counted, its place recorded, and skipped.  Nothing
// traps.  In the ordinary build the macro is `true` and the compiler drops it.
#ifdef ZLM_BOUNDS_CHECK
#ifndef ZLM_FILE_ID
#define ZLM_FILE_ID 0
#endif
__device__ __noinline__ static bool zlm_bc_ok(const void* p, unsigned long long bytes, int line) {
    ZlmShared* s = g_zlm.shared;
    const ZlmBoundsTable* t = g_zlm.bounds;
    if (!s || !t) return true;
    const unsigned long long a = (unsigned long long)p;
    const int n = t->n;
    for (int i = 0; i < n; ++i)
        if (a >= t->lo[i] && a + bytes <= t->hi[i]) return true;
    if (atomicAdd_system(&s->bc_violations, 1) == 0) {
        s->bc_first_site = (ZLM_FILE_ID << 16) | line;
        s->bc_first_addr = a;
    }
    __threadfence_system();
    return false;
}
#define ZLM_CHK(p, bytes) zlm_bc_ok((const void*)(p), (unsigned long long)(bytes), __LINE__)
#else
#define ZLM_CHK(p, bytes) true
#endif

// the current device, for per-device "done once" flags (function attributes are per device)
static inline int zlm_device_index() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    return dev;
}

#define ZLM_REQUIRE(cond, ...)                 \
    do {                                       \
        if (!(cond)) {                         \
            zlm_set_error(__VA_ARGS__);        \
            return ZLM_ERR_ARG;                \
        }                                      \
    } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// a vector weight (norm weights) may be stored in bf16 or fp32, whatever the
// compute dtype is; read it through this
struct VecW {
    const void* p;
    int dtype;
    __device__ __forceinline__ float operator[](int i) const {
        return dtype == ZLM_DTYPE_F32 ? ((const float*)p)[i]
                                      : __bfloat162float(((const __nv_bfloat16*)p)[i]);
    }
    // elements i .. i + 3, i a multiple of 4 (the vector starts 16-byte aligned)
    __device__ __forceinline__ float4 load4(int i) const {
        if (dtype == ZLM_DTYPE_F32) return *(const float4*)((const float*)p + i);
        const uint2 u = *(const uint2*)((const __nv_bfloat16*)p + i);
        return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                           __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum whose order depends only on blockDim (so a row's result does
// not depend on what else is in the batch).  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// ---------------------------------------------------------------------------
// A group of warps that works like a thread block of its own: the whole block of a
// stand-alone kernel (barrier 0), or some warps of a larger persistent block (a named
// barrier).  Code written against it runs unchanged in both places.
// ---------------------------------------------------------------------------
struct GroupSync {
    int id;         // hardware barrier
    int threads;    // threads that take part, a multiple of 32
    __device__ __forceinline__ void sync() const {
        asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
    }
};

// the sums and maxima above for a group: `tid` counts inside the group
__device__ __forceinline__ float group_sum(float v, float* red, int tid, const GroupSync& gs) {
    const int lane = tid & 31, warp = tid >> 5;
    const int nw = gs.threads >> 5;
    v = warp_sum(v);
    gs.sync();
    if (lane == 0) red[warp] = v;
    gs.sync();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float group_max(float v, float* red, int tid, const GroupSync& gs) {
    const int lane = tid & 31, warp = tid >> 5;
    const int nw = gs.threads >> 5;
    v = warp_max(v);
    gs.sync();
    if (lane == 0) red[warp] = v;
    gs.sync();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A decode step is a chain of short kernels; with
// this launch attribute a kernel's blocks may be scheduled while the kernel before
// it is still draining.  Every kernel of the chain calls pdl_wait() before it
// touches anything an earlier kernel of the step writes (activations, cache,
// scratch); what it reads before the wait must be constant during the step (weights,
// tables, the step's integer arrays, which are uploaded before the step's first
// kernel).  Without the attribute the calls do nothing.
// The trigger that lets the next kernel start is, for the kernels that stream weights or
// the cache, the implicit one at a block's end: an explicit trigger at their start was
// measured slower (the next kernel's blocks then sit on the SMs that this kernel's later
// waves need: 5.32 against 4.46 ms a step at Qwen3-8B sizes), so there
// pdl_launch_dependents() only marks the place.  The small kernels of a decode step (norm,
// rotation and cache write, combine, embedding: a few blocks, all resident at once) trigger
// at their start with pdl_trigger(): the product that follows them is launched, and has its
// first weights on the way, while they run.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() {}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

int zlm_pdl_enabled();
void zlm_count_launch();          // every kernel launch of the library is counted (zlm_launch_count)

template <typename... KArgs, typename... Args>
static inline void zlm_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = zlm_pdl_enabled() ? 1 : 0;
    zlm_count_launch();
    cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);     // errors surface in zlm_check_launch
}
