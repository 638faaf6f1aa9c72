// Two helpers beside the model's kernels: the random-weights generator on the device, and a read-only
// stream over a buffer that measures what the memory delivers to a kernel that only loads.
//
// The generator restates weights/loader.py:counter_normal exactly, in the same integer arithmetic: element i of
// the stream of `key` is the centred sum of twelve 16-bit fields of three splitmix64 hashes of its counter.
// Nothing of it depends on the launch shape, so a tensor made here equals the one made by the host code bit
// for bit.  The reference has no random-weights mode (it loads GGUF files: src/io/gguf_weight_loader.cpp).
#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, unsigned long long key, long long start, long long count,
                                   float scale, float offset, int round_bf16_first) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long base = (unsigned long long)(start + i) * 0x9E3779B97F4A7C15ull + key;
        int total = 0;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const unsigned long long h = mix64(base + 0xD1B54A32D192ED03ull * (unsigned long long)(j + 1));
            total += (int)(h & 0xFFFF) + (int)((h >> 16) & 0xFFFF) + (int)((h >> 32) & 0xFFFF) + (int)(h >> 48);
        }
        const float z = __fmul_rn((float)(total - 393210), 1.0f / 65536.0f);
        float v = __fadd_rn(offset, __fmul_rn(scale, z));          // two roundings, as the host code has them
        if (round_bf16_first) v = __bfloat162float(__float2bfloat16_rn(v));
        out[i] = from_f32<T>(v);
    }
}

__global__ void read_stream_kernel(const uint4* __restrict__ data, long long n16, unsigned* __restrict__ sink) {
    unsigned acc = 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    // eight independent 16-byte loads in flight per thread
    for (; i + 7 * stride < n16; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = __ldcs(data + i + k * stride);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc ^= v[k].x ^ v[k].y ^ v[k].z ^ v[k].w;
    }
    for (; i < n16; i += stride) {
        const uint4 v = __ldcs(data + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9E3779B9u) *sink = acc;       // practically never: keeps the loads alive without a store per thread
}

}  // namespace

// out[0..count) = offset + scale * z(key, start + i), stored as `dtype` (rounded through bfloat16 first when
// round_bf16_first, as a value read from a bfloat16 file would be).
LLME_API int llme_random_fill(void* out, int dtype, unsigned long long key, long long start, long long count, float scale,
                              float offset, int round_bf16_first, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (!out) LLME_REFUSE("random_fill: null pointer");
    const int threads = 256;
    const long long blocks = (count + threads - 1) / threads;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    if (dtype == LLME_F32)
        random_fill_kernel<float><<<grid, threads, 0, stream>>>((float*)out, key, start, count, scale, offset, round_bf16_first);
    else if (dtype == LLME_BF16)
        random_fill_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)out, key, start, count, scale, offset, round_bf16_first);
    else
        LLME_REFUSE("random_fill: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

// Reads `bytes` bytes (a multiple of 16, 16-byte aligned) once and stores nothing.
LLME_API int llme_read_stream(const void* data, long long bytes, unsigned* sink, int blocks_per_sm, cudaStream_t stream) {
    if (!data || !sink || bytes <= 0 || bytes % 16 || ((uintptr_t)data) % 16) LLME_REFUSE("read_stream: needs a 16-byte aligned buffer of a multiple of 16 bytes");
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (blocks_per_sm <= 0) blocks_per_sm = 4;
    read_stream_kernel<<<sms * blocks_per_sm, 512, 0, stream>>>((const uint4*)data, bytes / 16, sink);
    LLME_LAUNCH_STATUS();
}
