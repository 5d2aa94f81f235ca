// Decode attention without any allocation.
//
// This entry point has no counterpart in the reference (Lucas-Palomo/zlm keeps
// its attention scratch in buffers that its session allocates once).  It exists
// for callers that cannot allocate device memory at the time they call: code
// that runs inside someone else's memory plan (a host application that has
// handed the whole GPU to its own allocator), a plug-in loaded into a process
// whose allocator must not be disturbed, or a latency path where a cudaMalloc,
// which synchronises the device, is not acceptable.  Such callers own their
// inputs and outputs already; what they cannot provide is the scratch memory
// that the split-KV kernel needs for its partial results.
//
// zlm_attention_decode_static computes exactly what zlm_attention_decode
// computes (same kernels, same order of sums), but keeps the split partials in
// a fixed array inside the library:
//
//   * The array holds ZLM_NO_ALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU
//     on which the library is loaded carries it until the process exits.
//   * A call needs T * heads * splits * (head_dim + 2) floats when splits > 1
//     and none when splits == 1.  A larger request is refused with an error
//     that says so (zlm_last_error()); nothing is launched.
//   * No cudaMalloc, cudaFree or allocating library routine is called.
//   * The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and remembers it; make
//     that first call outside any stream capture, and from one host thread at a
//     time (the remembered address and the kernels' per-device set-up are
//     written without a lock).  A call with splits == 1 uses no scratch and
//     looks nothing up.
//   * All calls share the one array, which keeps whatever the last call left
//     there.  Nothing has to start at zero: every partial that the combining
//     kernel reads is written by the same call first.  Two calls whose kernels
//     can overlap on the GPU (different streams) race on the array; run them
//     on one stream or order them with events.
#pragma once
#include <cuda_runtime.h>

#define ZLM_NO_ALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as zlm_attention_decode without the two scratch pointers.  Split s of a
// sequence takes its pages [s * pages_per_split, (s + 1) * pages_per_split); splits *
// pages_per_split pages (of 64 tokens) must cover the longest sequence.
// out [T, nq*hd] bf16 (row stride out_stride), q [T, nq*hd] bf16 (row stride
// q_stride), pool [pages, 2, nkv, 64, hd] bf16, block_table [slots, table_stride]
// int32, token_pos / token_slot [T] int32.  Returns 0, or non-zero with the
// reason in zlm_last_error().
int zlm_attention_decode_static(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                const int* block_table, int table_stride, const int* token_pos,
                                const int* token_slot, int T, int nq, int nkv, int hd, float scale, int window,
                                int splits, int pages_per_split, cudaStream_t stream);

// The existing entry point, for comparison: the caller passes scratch of
// T*nq*splits*hd floats (part_o) and T*nq*splits*2 floats (part_ml).
int zlm_attention_decode(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                         const int* block_table, int table_stride, const int* token_pos, const int* token_slot,
                         int T, int nq, int nkv, int hd, float scale, int window, int splits, int pages_per_split,
                         float* part_o, float* part_ml, cudaStream_t stream);

const char* zlm_last_error(void);

#ifdef __cplusplus
}
#endif
