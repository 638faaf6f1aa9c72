// Plain paged attention: one warp per (token, query head), keys visited one at a time
// straight from the cache pages, online softmax in 32-bit.  It serves every case with
// one code path (a prompt portion of any length at any start position, a single decoded
// token, any mix of them in one launch) and is the whole attention of the 32-bit path.
// A token's result depends only on its own query and the keys of its request, never on
// what else is in the launch.
//
// Reference counterparts: paged_attention_decode_batch_kernel
// (src/runtime/kernels/cuda_kernels.cu:697-754) for one query per request, and the
// chunked causal loop of the CPU adapter (src/runtime/kernels/cpu_kernel_adapter.cpp:528-566)
// for portions: query at absolute position p sees keys 0..p.
#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

struct AttnArgs {
    const void* q;              // [T, nh, hd]
    const void* cache;          // [pages][K|V][nkv][page_size][hd]
    void* out;                  // [T, nh, hd]
    const int* positions;       // [T] absolute position of each token
    const int* token_request;   // [T] row of block_tables for each token
    const int* block_tables;    // [R, max_blocks]
    int max_blocks;
    int tokens, nh, nkv, hd, page_size;
    int window;                 // 0 = all keys up to the query; W > 0 = the last W of them
    float scale;
};
#include "kernel_args.h"
static_assert(sizeof(AttnArgs) == sizeof(LlmeAttnArgs), "the argument block must match kernel_args.h");

template <typename T, int REGS>
__global__ void attention_plain_kernel(AttnArgs a) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int h = blockIdx.y;
    if (t >= a.tokens) return;
    const int hd = a.hd, ps = a.page_size;
    const int kvh = h / (a.nh / a.nkv);
    const int p = a.positions[t];
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int* bt = a.block_tables + (size_t)a.token_request[t] * a.max_blocks;

    float q[REGS], acc[REGS];
    const T* qp = (const T*)a.q + ((size_t)t * a.nh + h) * hd;
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int d = lane + 32 * i;
        q[i] = d < hd ? to_f32(qp[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int j = lo; j <= p; ++j) {
        const int page = bt[j / ps];
        const int off = j - (j / ps) * ps;
        const T* kp = (const T*)a.cache + ((((size_t)page * 2 + 0) * a.nkv + kvh) * ps + off) * hd;
        const T* vp = kp + (size_t)a.nkv * ps * hd;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) s += q[i] * to_f32(kp[d]);
        }
        s = warp_sum(s) * a.scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);       // exp(-inf) = 0 on the first key
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) acc[i] = acc[i] * corr + e * to_f32(vp[d]);
        }
        m = m_new;
    }
    T* op = (T*)a.out + ((size_t)t * a.nh + h) * hd;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) op[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
static int launch_plain(const AttnArgs& a, cudaStream_t s) {
    const int wpb = 4;
    dim3 grid((a.tokens + wpb - 1) / wpb, a.nh);
    const int regs = (a.hd + 31) / 32;
    if (regs <= 1) llme_launch(attention_plain_kernel<T, 1>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 2) llme_launch(attention_plain_kernel<T, 2>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 4) llme_launch(attention_plain_kernel<T, 4>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 8) llme_launch(attention_plain_kernel<T, 8>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 16) llme_launch(attention_plain_kernel<T, 16>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else LLME_REFUSE("attention: head_dim %d is larger than 512", a.hd);
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_attention_plain(const AttnArgs* args, int dtype, cudaStream_t stream) {
    const AttnArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.q || !a.cache || !a.out || !a.positions || !a.token_request || !a.block_tables)
        LLME_REFUSE("attention: null pointer");
    if (a.nh <= 0 || a.nkv <= 0 || a.nh % a.nkv) LLME_REFUSE("attention: %d query heads are not a multiple of %d key/value heads", a.nh, a.nkv);
    if (a.hd <= 0 || a.page_size <= 0 || a.max_blocks <= 0) LLME_REFUSE("attention: non-positive size");
    if (a.nh > 65535) LLME_REFUSE("attention: more than 65535 query heads");
    if (dtype == LLME_F32) return launch_plain<float>(a, stream);
    if (dtype == LLME_BF16) return launch_plain<__nv_bfloat16>(a, stream);
    LLME_REFUSE("attention: unsupported dtype %d", dtype);
}
