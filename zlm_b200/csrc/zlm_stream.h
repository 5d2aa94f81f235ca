// The persistent decode kernel's program: a list of operations that one cooperative
// launch carries out in order, with a grid-wide barrier where an operation reads what
// the one before it wrote.  The Python side fills these records (the field order and
// sizes below are mirrored there) and uploads them once per step shape.
#pragma once
#include <stdint.h>

#define ZLM_STREAM_END 0
#define ZLM_STREAM_EMBED 1      // i: T H V                         p: out table ids
#define ZLM_STREAM_RMSNORM 2    // i: R H w_dtype vthreads  f: eps  p: out x w rows
#define ZLM_STREAM_GEMV 3       // i: T N K ldx ldy mode unit_rows  p: Y X W tensor_map(W)
#define ZLM_STREAM_ROPE 4       // i: T row_stride has_norm n_rot table_stride nq nkv hd writes_kv w_dtype vector_form
                                // f: eps    p: qkv q_w k_w inv_freq token_pos token_slot block_table pool
#define ZLM_STREAM_ATTN 5       // i: T out_stride q_stride table_stride nq nkv hd window splits per
                                // f: scale  p: out q pool block_table token_pos token_slot part_o part_ml
#define ZLM_STREAM_COMBINE 6    // i: T out_stride nq hd splits per window      p: out part_o part_ml token_pos

#define ZLM_STREAM_MAX_TOKENS 8

struct ZlmStreamOp {
    int32_t type;
    int32_t barrier;        // 1: every block waits here until all blocks have finished the operation before
    int32_t i[14];
    float f[4];
    const void* p[10];
};                          // 160 bytes
