/* Split-context decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference project (whose decode attention,
 * paged_attention_decode_batch_kernel in src/runtime/kernels/cuda_kernels.cu:697-754, needs
 * no scratch memory because one block walks a whole context).  It exists for users of this
 * library whose device memory is not theirs to hand out at call time:
 *
 *   - a host application that divides the whole device among its tenants or arenas up front
 *     and forbids the libraries it loads from calling cudaMalloc behind its back;
 *   - a serving loop that must not stall: cudaMalloc and cudaFree may synchronise the device,
 *     and an allocation can fail long after start-up, in the middle of a request.
 *
 * The regular entry point, llme_attention_decode, leaves the scratch buffer for the partial
 * results of the context splits to its caller.  llme_attention_decode_static instead keeps
 * that buffer inside the library, as a device array of fixed size, so a caller passes only
 * inputs and outputs.  It allocates nothing: no cudaMalloc, no cudaFree, no library routine
 * that allocates.
 *
 * Limits and rules
 *   - The array holds LLME_STATIC_SCRATCH_FLOATS 32-bit values (4 MiB).  Every GPU on which the
 *     library is loaded holds that much until the process exits.  A call needs
 *     65536 + n_rows * nh * splits * (HEAD_DIM + 2) values when splits > 1 (none when splits == 1); a
 *     call that needs more is refused with an error message and launches nothing.
 *   - The first call on each device looks up the array's device address (once per device, with
 *     that device current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Two calls whose kernels may overlap on the GPU
 *     (different streams, no ordering between them) race on it: keep calls of this entry point
 *     ordered on one stream, or order them with events.
 *   - The array keeps whatever the previous call left there.  Only its first 65536 words (ticket
 *     counters) have to be zero when a call starts: they are zero when the library is loaded, and every
 *     call puts back to zero the counters it used.  Every other value that a call reads it has written
 *     itself before.
 *
 * The argument block is the one llme_attention_decode takes; its `scratch` member is ignored.
 * The library is compiled for one head size (-DHEAD_DIM=...).
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLME_STATIC_SCRATCH_FLOATS (1 << 20)

/* Same layout as the argument block of llme_attention_decode (csrc/attention_fast.cu). */
typedef struct LlmeDecodeArgs {
    const void* q;             /* bfloat16 [T, nh, HEAD_DIM] */
    const void* cache;         /* bfloat16 [pages][K|V][nkv][page_size][HEAD_DIM] */
    void* out;                 /* bfloat16 [T, nh, HEAD_DIM] */
    const int* rows;           /* [n_rows] batch rows served by this call */
    const int* cu_q_lens;      /* [R+1] */
    const int* ctx_lens;       /* [R] cached length of each request, the new token included */
    const int* table_rows;     /* [R] row of block_tables of each request */
    const int* block_tables;   /* [*, max_blocks] */
    float* scratch;            /* ignored by llme_attention_decode_static */
    int max_blocks, n_rows, nh, nkv, page_size, window, splits;
    float scale;
} LlmeDecodeArgs;

/* Returns 0 on success, a cudaError_t value for a CUDA failure, -1 for refused arguments
 * (llme_last_error() then holds the reason). */
int llme_attention_decode_static(const LlmeDecodeArgs* args, cudaStream_t stream);

/* Capacity of the built-in scratch array, in 32-bit values. */
long long llme_attention_decode_static_capacity(void);

#ifdef __cplusplus
}
#endif
