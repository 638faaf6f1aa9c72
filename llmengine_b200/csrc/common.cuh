// Shared helpers of the sm_100a kernels: element types, warp/block reductions and
// the launch-status convention.
//
// Every launcher is an `extern "C"` function that takes raw device pointers, plain
// integers and a stream, validates what it can on the host, launches, and returns a
// cudaError_t-compatible int (0 = success, negative = an argument this build
// refuses; the message is kept for llme_last_error()).  Launch errors are read with
// cudaGetLastError() and never by synchronising the device, as the reference does in
// src/runtime/kernels/cuda_kernels.cu:49-51.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLME_API extern "C" __attribute__((visibility("default")))

enum LlmeDType : int { LLME_F32 = 0, LLME_BF16 = 1 };

// Error text of the last refused call in this thread.
inline char* llme_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

#include <stdio.h>
#define LLME_REFUSE(...)                                              \
    do {                                                              \
        snprintf(llme_error_buffer(), 512, __VA_ARGS__);              \
        return -1;                                                    \
    } while (0)

#define LLME_LAUNCH_STATUS()                                          \
    do {                                                              \
        cudaError_t e__ = cudaGetLastError();                         \
        if (e__ != cudaSuccess) {                                     \
            snprintf(llme_error_buffer(), 512, "%s", cudaGetErrorString(e__)); \
        }                                                             \
        return (int)e__;                                              \
    } while (0)

// Programmatic dependent launch.  A kernel launched through llme_launch may begin while the kernel
// before it in the stream is still running (its blocks become resident once every block of the earlier
// kernel has started); what it reads from or writes to memory that the earlier kernel touches must come
// after pdl_wait(), which returns when the earlier kernel has completed.  Work that does not depend on
// it (reading weights) may come first.  pdl_launch_dependents() lets the next kernel be scheduled early.
// Both are no-ops for kernels launched the ordinary way.  It is on unless LLME_PDL=0 is set in the environment.
// Measured inside CUDA graphs on B200 (Qwen3-8B shape, batch 8), a layer's operations pair by pair: every transition
// between products and norms gains 0.1 to 0.9 us.  The decode attention may begin early (its block table and first
// key/value loads come before its pdl_wait(): 1.1 us), but must not let its successor in before it has finished: with
// pdl_launch_dependents() before its merge, the transitions before and after it lose 10 and 7 us (a layer then needs
// 132 us against 95 us without any of this, a step 5.1 ms against 3.85 ms; 6.7 ms when every kernel let its successor
// in at its very start).  The products and norms do let their successors in at their start (their blocks fill an SM's
// registers, so the successor's blocks move in only as theirs leave): a layer takes 88.2 us so, 89.8 us with the
// products' successors let in only before their short epilogue.  As it is now a decode step at batch 8 takes 3.41 ms
// against 3.55 ms without any of this, a step of 121 prompt tokens beside 7 decoded ones 5.7 ms against 6.1 ms; the GPU
// tests pass either way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
#include <string.h>
#include <utility>
inline bool llme_pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("LLME_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t llme_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = llme_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// silu(g) * u where g and u have been through bfloat16: the hardware's exp2-based exponential and reciprocal
// (a few units in the last place of 32-bit, far below a bfloat16 digit) instead of expf and a division, which
// cost some forty instructions per value and, in a product's epilogue, take issue slots from the thread that
// issues the matrix instructions.  The 32-bit path keeps expf and the division.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) { return (g * __frcp_rn(1.0f + __expf(-g))) * u; }

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum over the 32 lanes; every lane gets the same value, and the order of additions
// is fixed, so a result never depends on what else runs in the launch.
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

// Block-wide sum for blocks of up to 1024 threads (a multiple of 32); `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? scratch[lane] : 0.0f;
    return warp_sum(t);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? scratch[lane] : -INFINITY;
    return warp_max(t);
}
