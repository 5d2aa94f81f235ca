// The status block of the library (see common.cuh): its allocation, the host's view of
// it, the list of translation units whose device-side pointers have to be bound, and the
// bounds-check build's table of registered ranges.
#include "common.cuh"
#include <string.h>

static ZlmShared* g_block = nullptr;                 // pinned host memory, one for all devices
static ZlmBoundsTable* g_tables[64] = {};            // device memory, per device
static ZlmBoundsTable g_table_host;                  // what the tables hold

int zlm_runtime_binding(ZlmBinding* out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        zlm_set_error("cannot tell the current device");
        return ZLM_ERR_CUDA;
    }
    if (!g_block) {
        void* p = nullptr;
        cudaError_t e = cudaHostAlloc(&p, sizeof(ZlmShared), cudaHostAllocMapped | cudaHostAllocPortable);
        if (e != cudaSuccess) {
            zlm_set_error("cannot allocate the status block in pinned host memory: %s", cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        memset(p, 0, sizeof(ZlmShared));
        g_block = (ZlmShared*)p;
    }
    if (!g_tables[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, sizeof(ZlmBoundsTable));
        if (e == cudaSuccess) e = cudaMemcpy(p, &g_table_host, sizeof(ZlmBoundsTable), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            zlm_set_error("cannot allocate the bounds table on device %d: %s", dev, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        g_tables[dev] = (ZlmBoundsTable*)p;
    }
    out->shared = g_block;
    out->bounds = g_tables[dev];
    return ZLM_OK;
}

#define ZLM_UNITS(X) \
    X(attention_decode) X(attention_generic) X(attention_prefill) X(attention_prefill_tc) X(elementwise) \
    X(gemm_bf16_mma) X(gemm_f32) X(gemm_tcgen05) X(gemv_bf16) X(rope_kv) X(sampling)
#define ZLM_DECLARE(name) extern "C" int zlm_bind_##name();
ZLM_UNITS(ZLM_DECLARE)

// Binds the block on the current device for every translation unit.  It copies to device
// symbols, so it must run outside any stream capture: the Python side calls it when the
// kernel object is made.
extern "C" int zlm_runtime_init() {
    int rc;
#define ZLM_BIND(name) if ((rc = zlm_bind_##name()) != ZLM_OK) return rc;
    ZLM_UNITS(ZLM_BIND)
    return ZLM_OK;
}

// 0, or the mark of the first bounded wait that gave up: (kernel family << 8) | place.
// Reads host memory: no synchronisation, so it tells of kernels that have finished.
extern "C" int zlm_status() { return g_block ? *(volatile int*)&g_block->status : 0; }
extern "C" void zlm_status_clear() { if (g_block) *(volatile int*)&g_block->status = 0; }

// ---- the bounds-check build's ranges ----------------------------------------------
extern "C" int zlm_bounds_check_build() {
#ifdef ZLM_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}
static int push_table() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_tables[dev]) return ZLM_OK;
    cudaError_t e = cudaMemcpy(g_tables[dev], &g_table_host, sizeof(ZlmBoundsTable), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        zlm_set_error("bounds check: cannot update the table: %s", cudaGetErrorString(e));
        return ZLM_ERR_CUDA;
    }
    return ZLM_OK;
}
extern "C" int zlm_bounds_clear_ranges() {
    g_table_host.n = 0;
    return push_table();
}
// Registers [base, base + bytes) as memory the kernels may touch (synchronises: the table is
// copied to the device).  A range inside a registered one is not stored again.
extern "C" int zlm_bounds_add_range(const void* base, unsigned long long bytes) {
    const unsigned long long lo = (unsigned long long)base, hi = lo + bytes;
    for (int i = 0; i < g_table_host.n; ++i)
        if (g_table_host.lo[i] <= lo && hi <= g_table_host.hi[i]) return ZLM_OK;
    ZLM_REQUIRE(g_table_host.n < ZLM_BC_MAX_RANGES, "bounds check: more than %d ranges registered", ZLM_BC_MAX_RANGES);
    g_table_host.lo[g_table_host.n] = lo;
    g_table_host.hi[g_table_host.n] = hi;
    g_table_host.n += 1;
    return push_table();
}
extern "C" int zlm_bounds_violations() { return g_block ? *(volatile int*)&g_block->bc_violations : 0; }
extern "C" int zlm_bounds_first_site() { return g_block ? g_block->bc_first_site : 0; }
extern "C" unsigned long long zlm_bounds_first_address() { return g_block ? g_block->bc_first_addr : 0; }
extern "C" void zlm_bounds_reset() {
    if (!g_block) return;
    g_block->bc_violations = 0;
    g_block->bc_first_site = 0;
    g_block->bc_first_addr = 0;
}
