/* Argument blocks of the kernel libraries' entry points, as plain C structs: what a caller outside the kernel
 * sources (the step executor, a binding) fills in.  Each kernel source keeps its own typed struct and asserts
 * that its layout equals the one here. */
#pragma once

typedef struct LlmeQkvArgs {
    const void* q_in; const void* k_in; const void* v_in;
    long long q_stride, k_stride, v_stride;      /* elements between consecutive tokens */
    const void* q_gain; const void* k_gain;       /* nullable: no norm */
    int gain_dtype;
    float eps;
    const float* cos_sin;                         /* nullable: no rotation; [max_pos, head_dim] = cos | sin */
    const int* positions;
    int max_positions;
    void* q_out; void* k_out;                     /* nullable; [T, nh*hd], [T, nkv*hd] */
    void* cache; const int* slot_mapping;         /* nullable */
    int tokens, nh, nkv, hd, page_size;
} LlmeQkvArgs;

typedef struct LlmeAttnArgs {
    const void* q; const void* cache; void* out;
    const int* positions; const int* token_request; const int* block_tables;
    int max_blocks;
    int tokens, nh, nkv, hd, page_size;
    int window;
    float scale;
} LlmeAttnArgs;

typedef struct LlmeFastAttnArgs {
    const void* q; const void* cache; void* out;
    const int* rows; const int* cu_q_lens; const int* ctx_lens; const int* table_rows; const int* block_tables;
    float* scratch;
    int max_blocks, n_rows, nh, nkv, page_size, window, splits;
    float scale;
} LlmeFastAttnArgs;

typedef struct LlmeFusedQkv {
    const void* qkv; long long stride;
    const void* q_gain; const void* k_gain; int gain_dtype; float eps;
    const float* cos_sin; int max_positions; int write_kv;
} LlmeFusedQkv;

typedef struct LlmeTcAttnArgs {
    void* out; const void* cache;
    const int* rows; const int* cu_q_lens; const int* ctx_lens; const int* table_rows; const int* block_tables;
    int max_blocks, n_rows, nh, nkv, page_size, window;
    float scale;
} LlmeTcAttnArgs;
