// Memory-bound kernels of the layer body: embedding gather, RMS norm fused with the
// residual add, per-head QK norm + rotary encoding + write into the paged cache, and
// the SwiGLU gate.  All arithmetic is 32-bit; only storage may be bfloat16.
//
// Reference counterparts (src/runtime/kernels/cuda_kernels.cu): embedding_kernel
// :380-397, rmsnorm_kernel :360-378 (also used as QK norm), add_kernel :224-227,
// rope_kernel :430-450, swiglu_kernel :245-248, and the per-token cudaMemcpy cache
// writes of src/runtime/cache/paged_kv_cache.cpp:189-207, which the fused write replaces.
#include <type_traits>

#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

// ----------------------------------------------------------------------------- embedding
// out[t, :] = float(table[ids[t], :]).  An id outside the table gives a row of zeros here;
// the engine refuses such ids on the host before it launches anything.
template <typename W>
__global__ void embedding_kernel(const int* __restrict__ ids, const W* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = 0.0f;
        return;
    }
    const W* row = table + (size_t)id * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = to_f32(row[j]);
}

// The same for bfloat16 tables whose rows are a multiple of 8 wide: 16 bytes in, 32 bytes out per thread.
__global__ void embedding_bf16x8_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * hidden);
    float4* o = reinterpret_cast<float4*>(out + (size_t)t * hidden);
    for (int j = threadIdx.x; j < hidden / 8; j += blockDim.x) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (ok) {
            const uint4 v = row[j];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
            const float2 f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
            a = make_float4(f0.x, f0.y, f1.x, f1.y);
            b = make_float4(f2.x, f2.y, f3.x, f3.y);
        }
        o[2 * j] = a;
        o[2 * j + 1] = b;
    }
}

LLME_API int llme_embedding(const int* ids, const void* table, int table_dtype, float* out,
                            int tokens, int hidden, int vocab, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (!ids || !table || !out || hidden <= 0 || vocab <= 0) LLME_REFUSE("embedding: null pointer or non-positive size");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == LLME_BF16 && hidden % 8 == 0 && ((uintptr_t)table % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        llme_launch(embedding_bf16x8_kernel, dim3(tokens), dim3(hidden >= 2048 ? 256 : 64), 0, stream, ids, (const __nv_bfloat16*)table, out, hidden, vocab);
        LLME_LAUNCH_STATUS();
    }
    if (table_dtype == LLME_F32)
        llme_launch(embedding_kernel<float>, dim3(tokens), dim3(threads), 0, stream, ids, (const float*)table, out, hidden, vocab);
    else if (table_dtype == LLME_BF16)
        llme_launch(embedding_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, ids, (const __nv_bfloat16*)table, out, hidden, vocab);
    else
        LLME_REFUSE("embedding: unsupported table dtype %d", table_dtype);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- RMS norm (+ residual add)
// For output row i (source row r = rows ? rows[i] : i):
//   v = x[r] (+ delta[r], stored back into x[r]);  y[i] = (v * 1/sqrt(mean(v^2) + eps)) * gain.
// One block per row; the sum of squares is reduced in a fixed order.
template <typename D, typename G, typename O, bool HAS_DELTA>
__global__ void rmsnorm_kernel(float* __restrict__ x, const D* __restrict__ delta, const G* __restrict__ gain,
                               O* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* xr = x + (size_t)r * hidden;
    const D* dr = HAS_DELTA ? delta + (size_t)r * hidden : nullptr;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = xr[j];
        if (HAS_DELTA) {
            v += to_f32(dr[j]);
            xr[j] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
    O* o = out + (size_t)i * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        // same thread wrote xr[j] above, so the re-read sees the sum
        o[j] = from_f32<O>((xr[j] * rinv) * to_f32(gain[j]));
    }
}

// Vector form for rows that are a multiple of 4 wide: each thread keeps up to V groups of 4 values of the
// row in registers, so the row is read once, and all its loads are in flight together.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        uint2 raw;
        *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename D, typename G, typename O, bool HAS_DELTA, int V>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const D* __restrict__ delta, const G* __restrict__ gain,
                                   O* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* xr = x + (size_t)r * hidden;
    const int groups = hidden >> 2;
    float4 v[V], g[V];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < V; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < groups) {
            v[k] = Vec4<float>::load(xr + 4 * j);
            g[k] = Vec4<G>::load(gain + 4 * j);
            if (HAS_DELTA) {
                const float4 d = Vec4<D>::load(delta + (size_t)r * hidden + 4 * j);
                v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < groups) {
            if (HAS_DELTA) Vec4<float>::store(xr + 4 * j, v[k]);
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
    O* o = out + (size_t)i * hidden;
#pragma unroll
    for (int k = 0; k < V; ++k) {
        const int j = threadIdx.x + k * blockDim.x;
        if (j < groups)
            Vec4<O>::store(o + 4 * j, make_float4((v[k].x * rinv) * g[k].x, (v[k].y * rinv) * g[k].y,
                                                  (v[k].z * rinv) * g[k].z, (v[k].w * rinv) * g[k].w));
    }
}

template <typename D, typename G, typename O, bool HAS_DELTA>
static bool launch_rmsnorm_vec(float* x, const void* delta, const void* gain, void* out, const int* rows,
                               int n_out, int hidden, float eps, cudaStream_t s) {
    if (hidden % 4 || hidden > 16384) return false;
    if (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)out) % 16) return false;
    const int groups = hidden / 4;
    // few rows: short dependency chains matter more than occupancy, so spread the row over many threads
    if (groups <= 256)
        llme_launch(rmsnorm_vec_kernel<D, G, O, HAS_DELTA, 1>, dim3(n_out), dim3(((groups + 31) / 32) * 32), 0, s, x, (const D*)delta, (const G*)gain, (O*)out, rows, hidden, eps);
    else if (groups <= 1024)
        llme_launch(rmsnorm_vec_kernel<D, G, O, HAS_DELTA, 2>, dim3(n_out), dim3((((groups + 1) / 2 + 31) / 32) * 32), 0, s, x, (const D*)delta, (const G*)gain, (O*)out, rows, hidden, eps);
    else
        llme_launch(rmsnorm_vec_kernel<D, G, O, HAS_DELTA, 4>, dim3(n_out), dim3((((groups + 3) / 4 + 31) / 32) * 32), 0, s, x, (const D*)delta, (const G*)gain, (O*)out, rows, hidden, eps);
    return true;
}

template <typename D, typename G, typename O, bool HAS_DELTA>
static void launch_rmsnorm(float* x, const void* delta, const void* gain, void* out, const int* rows,
                           int n_out, int hidden, float eps, cudaStream_t s) {
    if (launch_rmsnorm_vec<D, G, O, HAS_DELTA>(x, delta, gain, out, rows, n_out, hidden, eps, s)) return;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    llme_launch(rmsnorm_kernel<D, G, O, HAS_DELTA>, dim3(n_out), dim3(threads), 0, s, x, (const D*)delta, (const G*)gain, (O*)out, rows, hidden, eps);
}

template <typename D, bool HAS_DELTA>
static int dispatch_rmsnorm(float* x, const void* delta, const void* gain, int gain_dtype, void* out, int out_dtype,
                            const int* rows, int n_out, int hidden, float eps, cudaStream_t s) {
    if (gain_dtype == LLME_F32 && out_dtype == LLME_F32) launch_rmsnorm<D, float, float, HAS_DELTA>(x, delta, gain, out, rows, n_out, hidden, eps, s);
    else if (gain_dtype == LLME_F32 && out_dtype == LLME_BF16) launch_rmsnorm<D, float, __nv_bfloat16, HAS_DELTA>(x, delta, gain, out, rows, n_out, hidden, eps, s);
    else if (gain_dtype == LLME_BF16 && out_dtype == LLME_F32) launch_rmsnorm<D, __nv_bfloat16, float, HAS_DELTA>(x, delta, gain, out, rows, n_out, hidden, eps, s);
    else if (gain_dtype == LLME_BF16 && out_dtype == LLME_BF16) launch_rmsnorm<D, __nv_bfloat16, __nv_bfloat16, HAS_DELTA>(x, delta, gain, out, rows, n_out, hidden, eps, s);
    else LLME_REFUSE("rmsnorm: unsupported gain/out dtype %d/%d", gain_dtype, out_dtype);
    LLME_LAUNCH_STATUS();
}

// x [*, hidden] 32-bit (updated in place when delta is given); delta nullable; rows nullable
// (n_out source-row indices); out [n_out, hidden].
LLME_API int llme_rmsnorm(float* x, const void* delta, int delta_dtype, const void* gain, int gain_dtype,
                          void* out, int out_dtype, const int* rows, int n_out, int hidden, float eps,
                          cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (!x || !gain || !out || hidden <= 0) LLME_REFUSE("rmsnorm: null pointer or non-positive size");
    if (!(eps > 0.0f)) LLME_REFUSE("rmsnorm: eps must be positive");
    if (!delta) return dispatch_rmsnorm<float, false>(x, nullptr, gain, gain_dtype, out, out_dtype, rows, n_out, hidden, eps, stream);
    if (delta_dtype == LLME_F32) return dispatch_rmsnorm<float, true>(x, delta, gain, gain_dtype, out, out_dtype, rows, n_out, hidden, eps, stream);
    if (delta_dtype == LLME_BF16) return dispatch_rmsnorm<__nv_bfloat16, true>(x, delta, gain, gain_dtype, out, out_dtype, rows, n_out, hidden, eps, stream);
    LLME_REFUSE("rmsnorm: unsupported delta dtype %d", delta_dtype);
}

// ----------------------------------------------------------------------------- QK norm + rotary + cache write
// One warp per (token, head).  Heads 0..nh-1 are query heads, then nkv key heads, then nkv
// value heads.  Query and key heads: optional RMS norm over head_dim (gain shared by all
// heads), optional rotation of the pairs (d, d + head_dim/2) with cos/sin read from a table
// row chosen by the token's position.  Queries go to q_out, keys to k_out and/or the cache,
// values to the cache.  Cache layout: [page][K|V][kv head][slot in page][head_dim]; a token's
// place is slot_mapping[t] = page * page_size + slot, negative = not stored.
struct QkvArgs {
    const void* q_in; const void* k_in; const void* v_in;
    long long q_stride, k_stride, v_stride;      // elements between consecutive tokens
    const void* q_gain; const void* k_gain;       // nullable: no norm
    int gain_dtype;
    float eps;
    const float* cos_sin;                         // nullable: no rotation; [max_pos, head_dim] = cos | sin
    const int* positions;
    int max_positions;
    void* q_out; void* k_out;                     // nullable; [T, nh*hd], [T, nkv*hd]
    void* cache; const int* slot_mapping;         // nullable
    int tokens, nh, nkv, hd, page_size;
};
#include "kernel_args.h"
static_assert(sizeof(QkvArgs) == sizeof(LlmeQkvArgs), "the argument block must match kernel_args.h");

template <typename I, typename O, typename G>
__global__ void qkv_post_kernel(QkvArgs a) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int heads = a.nh + 2 * a.nkv;
    if (wid >= (long long)a.tokens * heads) return;
    const int t = (int)(wid / heads);
    const int h = (int)(wid % heads);
    const int hd = a.hd, half = hd >> 1;

    if (h >= a.nh + a.nkv) {                       // value head: copy into the cache
        if (!a.cache || !a.v_in) return;
        const int slot = a.slot_mapping[t];
        if (slot < 0) return;
        const int kvh = h - a.nh - a.nkv;
        const I* src = (const I*)a.v_in + (size_t)t * a.v_stride + (size_t)kvh * hd;
        const int page = slot / a.page_size, off = slot % a.page_size;
        O* dst = (O*)a.cache + ((((size_t)page * 2 + 1) * a.nkv + kvh) * a.page_size + off) * hd;
        for (int d = lane; d < hd; d += 32) dst[d] = from_f32<O>(to_f32(src[d]));
        return;
    }

    const bool is_q = h < a.nh;
    const int head = is_q ? h : h - a.nh;
    const I* src;
    if (is_q) {
        if (!a.q_in) return;
        src = (const I*)a.q_in + (size_t)t * a.q_stride + (size_t)head * hd;
    } else {
        if (!a.k_in) return;
        src = (const I*)a.k_in + (size_t)t * a.k_stride + (size_t)head * hd;
    }
    const G* gain = (const G*)(is_q ? a.q_gain : a.k_gain);

    float rinv = 1.0f;
    if (gain) {
        float ss = 0.0f;
        for (int d = lane; d < hd; d += 32) {
            const float v = to_f32(src[d]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        rinv = 1.0f / sqrtf(ss / (float)hd + a.eps);
    }

    O* q_dst = (is_q && a.q_out) ? (O*)a.q_out + ((size_t)t * a.nh + head) * hd : nullptr;
    O* k_dst = (!is_q && a.k_out) ? (O*)a.k_out + ((size_t)t * a.nkv + head) * hd : nullptr;
    O* c_dst = nullptr;
    if (!is_q && a.cache) {
        const int slot = a.slot_mapping[t];
        if (slot >= 0) {
            const int page = slot / a.page_size, off = slot % a.page_size;
            c_dst = (O*)a.cache + ((((size_t)page * 2 + 0) * a.nkv + head) * a.page_size + off) * hd;
        }
    }
    const float* cs = nullptr;
    if (a.cos_sin) {
        int pos = a.positions[t];
        pos = pos < 0 ? 0 : (pos >= a.max_positions ? a.max_positions - 1 : pos);   // the host refuses such positions
        cs = a.cos_sin + (size_t)pos * hd;
    }
    for (int d = lane; d < half; d += 32) {
        float x0 = to_f32(src[d]), x1 = to_f32(src[d + half]);
        if (gain) {
            x0 = (x0 * rinv) * to_f32(gain[d]);
            x1 = (x1 * rinv) * to_f32(gain[d + half]);
        }
        float y0 = x0, y1 = x1;
        if (cs) {
            const float c = cs[d], s = cs[half + d];
            y0 = x0 * c - x1 * s;
            y1 = x0 * s + x1 * c;
        }
        const O o0 = from_f32<O>(y0), o1 = from_f32<O>(y1);
        if (q_dst) { q_dst[d] = o0; q_dst[d + half] = o1; }
        if (k_dst) { k_dst[d] = o0; k_dst[d + half] = o1; }
        if (c_dst) { c_dst[d] = o0; c_dst[d + half] = o1; }
    }
}

// Vector form for head sizes that are a multiple of 4: a lane holds two neighbouring values of the
// first half of the head and the two values they are paired with in the second half, for up to NP such
// groups; the head is read once (4- or 8-byte loads) and stays in registers through norm and rotation.
template <typename T> struct Vec2;
template <> struct Vec2<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct Vec2<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }
};

// TPW: tokens per warp.  With many tokens a warp takes the same head of TPW consecutive tokens and issues all
// their loads (head, gains, cos/sin rows) before the first reduction, so that four times as many bytes are in
// flight per warp; with few tokens (a decode step) every (token, head) pair gets a warp of its own.
template <typename I, typename O, typename G, int NP, int TPW>
__global__ void qkv_post_vec_kernel(QkvArgs a) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    // grid: x = group of TPW tokens, y = group of heads (one per warp of the block); no division per warp
    const int lane = threadIdx.x & 31;
    const int heads = a.nh + 2 * a.nkv;
    const int t0 = (int)blockIdx.x * TPW;
    const int h = (int)blockIdx.y * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5);
    if (h >= heads) return;
    const int hd = a.hd, half = hd >> 1;
    const int page_shift = (a.page_size & (a.page_size - 1)) == 0 ? __ffs(a.page_size) - 1 : -1;

    if (h >= a.nh + a.nkv) {                       // value head: copy into the cache
        if (!a.cache || !a.v_in) return;
        const int kvh = h - a.nh - a.nkv;
        float2 v[TPW][2 * NP];
        int slot[TPW];
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            const int t = t0 + u;
            slot[u] = t < a.tokens ? a.slot_mapping[t] : -1;
            const I* src = (const I*)a.v_in + (size_t)(t < a.tokens ? t : t0) * a.v_stride + (size_t)kvh * hd;
#pragma unroll
            for (int i = 0; i < 2 * NP; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < hd) v[u][i] = Vec2<I>::load(src + d);
            }
        }
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            if (slot[u] < 0) continue;
            const int page = page_shift >= 0 ? slot[u] >> page_shift : slot[u] / a.page_size;
            const int off = slot[u] - page * a.page_size;
            O* dst = (O*)a.cache + ((((size_t)page * 2 + 1) * a.nkv + kvh) * a.page_size + off) * hd;
#pragma unroll
            for (int i = 0; i < 2 * NP; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < hd) Vec2<O>::store(dst + d, v[u][i]);
            }
        }
        return;
    }

    const bool is_q = h < a.nh;
    const int head = is_q ? h : h - a.nh;
    const I* base = (const I*)(is_q ? a.q_in : a.k_in);
    if (!base) return;
    const long long stride = is_q ? a.q_stride : a.k_stride;
    const G* gain = (const G*)(is_q ? a.q_gain : a.k_gain);

    // every load first: the heads, the gains, the rows of the cos/sin table and the cache slots
    float2 lo[TPW][NP], hi[TPW][NP], co[TPW][NP], si[TPW][NP], g0[NP], g1[NP];
    int slot[TPW];
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
        const int t = t0 + u < a.tokens ? t0 + u : t0;
        const I* src = base + (size_t)t * stride + (size_t)head * hd;
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < half) {
                lo[u][i] = Vec2<I>::load(src + d);
                hi[u][i] = Vec2<I>::load(src + d + half);
            }
        }
        slot[u] = (!is_q && a.cache && t0 + u < a.tokens) ? a.slot_mapping[t] : -1;
        if (a.cos_sin) {
            int pos = a.positions[t];
            pos = pos < 0 ? 0 : (pos >= a.max_positions ? a.max_positions - 1 : pos);   // the host refuses such positions
            const float* cs = a.cos_sin + (size_t)pos * hd;
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < half) {
                    co[u][i] = *reinterpret_cast<const float2*>(cs + d);
                    si[u][i] = *reinterpret_cast<const float2*>(cs + half + d);
                }
            }
        }
    }
    if (gain) {
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < half) {
                g0[i] = Vec2<G>::load(gain + d);
                g1[i] = Vec2<G>::load(gain + d + half);
            }
        }
    }

#pragma unroll
    for (int u = 0; u < TPW; ++u) {
        if (t0 + u >= a.tokens) break;
        const int t = t0 + u;
        if (gain) {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < half) ss += lo[u][i].x * lo[u][i].x + lo[u][i].y * lo[u][i].y + hi[u][i].x * hi[u][i].x + hi[u][i].y * hi[u][i].y;
            }
            ss = warp_sum(ss);
            const float rinv = 1.0f / sqrtf(ss / (float)hd + a.eps);
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < half) {
                    lo[u][i].x = (lo[u][i].x * rinv) * g0[i].x; lo[u][i].y = (lo[u][i].y * rinv) * g0[i].y;
                    hi[u][i].x = (hi[u][i].x * rinv) * g1[i].x; hi[u][i].y = (hi[u][i].y * rinv) * g1[i].y;
                }
            }
        }
        if (a.cos_sin) {
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < half) {
                    const float2 c = co[u][i], sn = si[u][i];
                    const float2 x0 = lo[u][i], x1 = hi[u][i];
                    lo[u][i] = make_float2(x0.x * c.x - x1.x * sn.x, x0.y * c.y - x1.y * sn.y);
                    hi[u][i] = make_float2(x0.x * sn.x + x1.x * c.x, x0.y * sn.y + x1.y * c.y);
                }
            }
        }
        O* q_dst = (is_q && a.q_out) ? (O*)a.q_out + ((size_t)t * a.nh + head) * hd : nullptr;
        O* k_dst = (!is_q && a.k_out) ? (O*)a.k_out + ((size_t)t * a.nkv + head) * hd : nullptr;
        O* c_dst = nullptr;
        if (slot[u] >= 0) {
            const int page = page_shift >= 0 ? slot[u] >> page_shift : slot[u] / a.page_size;
            const int off = slot[u] - page * a.page_size;
            c_dst = (O*)a.cache + ((((size_t)page * 2 + 0) * a.nkv + head) * a.page_size + off) * hd;
        }
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < half) {
                if (q_dst) { Vec2<O>::store(q_dst + d, lo[u][i]); Vec2<O>::store(q_dst + d + half, hi[u][i]); }
                if (k_dst) { Vec2<O>::store(k_dst + d, lo[u][i]); Vec2<O>::store(k_dst + d + half, hi[u][i]); }
                if (c_dst) { Vec2<O>::store(c_dst + d, lo[u][i]); Vec2<O>::store(c_dst + d + half, hi[u][i]); }
            }
        }
    }
}

// Many tokens, bfloat16 in and out, a head size of 32, 64, 128 or 256: a warp takes one token and a run of
// heads.  What belongs to the token (its position's cos/sin values, its cache slot, the gains) is loaded once
// per warp instead of once per head, a lane holds 4 + 4 values of a head (8-byte loads and stores), and the
// 32 lanes cover 32 / LPH heads at a time, so that a head costs about half the instructions of the kernel above.
constexpr int QKV_WIDE_ITERS = 2;      // head groups per warp
constexpr int QKV_WIDE_WARPS = 8;      // = tokens per block

__device__ __forceinline__ void bf16x4_to_f32(uint2 v, float (&f)[4]) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 f32_to_bf16x4(const float (&f)[4]) {
    uint2 v;
    *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(f[0], f[1]);
    *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(f[2], f[3]);
    return v;
}
template <typename G> __device__ __forceinline__ void load_gain4(const G* p, float (&g)[4]);
template <> __device__ __forceinline__ void load_gain4<float>(const float* p, float (&g)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    g[0] = v.x; g[1] = v.y; g[2] = v.z; g[3] = v.w;
}
template <> __device__ __forceinline__ void load_gain4<__nv_bfloat16>(const __nv_bfloat16* p, float (&g)[4]) {
    bf16x4_to_f32(*reinterpret_cast<const uint2*>(p), g);
}

template <typename G, int LPH>
__global__ void __launch_bounds__(QKV_WIDE_WARPS * 32, 4) qkv_post_wide_kernel(QkvArgs a) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    typedef __nv_bfloat16 bf16;
    constexpr int HPW = 32 / LPH;                  // heads the warp's lanes cover at a time
    constexpr int HD = LPH * 8, HALF = HD / 2;
    const int lane = threadIdx.x & 31;
    const int t = (int)blockIdx.x * QKV_WIDE_WARPS + (int)(threadIdx.x >> 5);
    if (t >= a.tokens) return;
    const int heads = a.nh + 2 * a.nkv;
    const int d = 4 * (lane % LPH);                // this lane's values: d .. d+3 and HALF+d .. HALF+d+3
    const int h0 = (int)blockIdx.y * (HPW * QKV_WIDE_ITERS) + lane / LPH;

    // the heads first (the loads that take longest), then what belongs to the token
    uint2 lo[QKV_WIDE_ITERS], hi[QKV_WIDE_ITERS];
#pragma unroll
    for (int it = 0; it < QKV_WIDE_ITERS; ++it) {
        const int h = h0 + it * HPW;
        const bf16* src = nullptr;
        if (h < a.nh) { if (a.q_in) src = (const bf16*)a.q_in + (size_t)t * a.q_stride + (size_t)h * HD; }
        else if (h < a.nh + a.nkv) { if (a.k_in) src = (const bf16*)a.k_in + (size_t)t * a.k_stride + (size_t)(h - a.nh) * HD; }
        else if (h < heads) { if (a.v_in) src = (const bf16*)a.v_in + (size_t)t * a.v_stride + (size_t)(h - a.nh - a.nkv) * HD; }
        lo[it] = make_uint2(0u, 0u); hi[it] = make_uint2(0u, 0u);
        if (src) {
            lo[it] = *reinterpret_cast<const uint2*>(src + d);
            hi[it] = *reinterpret_cast<const uint2*>(src + HALF + d);
        }
    }
    float co[4] = {1.0f, 1.0f, 1.0f, 1.0f}, si[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (a.cos_sin) {
        int pos = a.positions[t];
        pos = pos < 0 ? 0 : (pos >= a.max_positions ? a.max_positions - 1 : pos);   // the host refuses such positions
        const float* cs = a.cos_sin + (size_t)pos * HD;
        load_gain4<float>(cs + d, co);
        load_gain4<float>(cs + HALF + d, si);
    }
    float qg0[4], qg1[4], kg0[4], kg1[4];
    if (a.q_gain) { load_gain4<G>((const G*)a.q_gain + d, qg0); load_gain4<G>((const G*)a.q_gain + HALF + d, qg1); }
    if (a.k_gain) { load_gain4<G>((const G*)a.k_gain + d, kg0); load_gain4<G>((const G*)a.k_gain + HALF + d, kg1); }
    bf16* cache_row = nullptr;                     // the token's place in the cache: key of head 0
    size_t kv_step = 0, head_step = 0;
    if (a.cache) {
        const int slot = a.slot_mapping[t];
        if (slot >= 0) {
            const int page = slot / a.page_size, off = slot - page * a.page_size;
            head_step = (size_t)a.page_size * HD;
            kv_step = (size_t)a.nkv * head_step;
            cache_row = (bf16*)a.cache + (size_t)page * 2 * kv_step + (size_t)off * HD;
        }
    }

#pragma unroll
    for (int it = 0; it < QKV_WIDE_ITERS; ++it) {
        const int h = h0 + it * HPW;
        const bool is_q = h < a.nh, is_k = !is_q && h < a.nh + a.nkv, is_v = !is_q && !is_k && h < heads;
        float x0[4], x1[4];
        bf16x4_to_f32(lo[it], x0);
        bf16x4_to_f32(hi[it], x1);
        // every lane takes part in the sums, whatever its head is
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += x0[i] * x0[i] + x1[i] * x1[i];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (is_v) {
            if (cache_row && a.v_in) {
                bf16* dst = cache_row + kv_step + (size_t)(h - a.nh - a.nkv) * head_step;
                *reinterpret_cast<uint2*>(dst + d) = lo[it];
                *reinterpret_cast<uint2*>(dst + HALF + d) = hi[it];
            }
            continue;
        }
        if (!(is_q || is_k) || !(is_q ? a.q_in : a.k_in)) continue;
        if (is_q ? a.q_gain != nullptr : a.k_gain != nullptr) {
            const float rinv = 1.0f / sqrtf(ss / (float)HD + a.eps);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x0[i] = (x0[i] * rinv) * (is_q ? qg0[i] : kg0[i]);
                x1[i] = (x1[i] * rinv) * (is_q ? qg1[i] : kg1[i]);
            }
        }
        if (a.cos_sin) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float u = x0[i], v = x1[i];
                x0[i] = u * co[i] - v * si[i];
                x1[i] = u * si[i] + v * co[i];
            }
        }
        const uint2 o0 = f32_to_bf16x4(x0), o1 = f32_to_bf16x4(x1);
        if (is_q) {
            if (a.q_out) {
                bf16* dst = (bf16*)a.q_out + ((size_t)t * a.nh + h) * HD;
                *reinterpret_cast<uint2*>(dst + d) = o0;
                *reinterpret_cast<uint2*>(dst + HALF + d) = o1;
            }
        } else {
            const int head = h - a.nh;
            if (a.k_out) {
                bf16* dst = (bf16*)a.k_out + ((size_t)t * a.nkv + head) * HD;
                *reinterpret_cast<uint2*>(dst + d) = o0;
                *reinterpret_cast<uint2*>(dst + HALF + d) = o1;
            }
            if (cache_row) {
                bf16* dst = cache_row + (size_t)head * head_step;
                *reinterpret_cast<uint2*>(dst + d) = o0;
                *reinterpret_cast<uint2*>(dst + HALF + d) = o1;
            }
        }
    }
}

template <typename G, int LPH>
static void launch_qkv_wide_lph(const QkvArgs& a, cudaStream_t s) {
    const int heads = a.nh + 2 * a.nkv;
    const int per_warp = (32 / LPH) * QKV_WIDE_ITERS;
    llme_launch(qkv_post_wide_kernel<G, LPH>, dim3((unsigned)((a.tokens + QKV_WIDE_WARPS - 1) / QKV_WIDE_WARPS), (unsigned)((heads + per_warp - 1) / per_warp)),
                dim3(QKV_WIDE_WARPS * 32), 0, s, a);
}

// Whether the wide kernel takes this call (and then launches it): bfloat16 in and out is the caller's business.
template <typename G>
static bool launch_qkv_wide(const QkvArgs& a, cudaStream_t s) {
    const int heads = a.nh + 2 * a.nkv;
    if (a.hd != 32 && a.hd != 64 && a.hd != 128 && a.hd != 256) return false;
    const int groups = (heads + (256 / a.hd) * QKV_WIDE_ITERS - 1) / ((256 / a.hd) * QKV_WIDE_ITERS);
    if (groups > 65535) return false;
    if ((long long)a.tokens * groups < 148LL * 16) return false;                // few tokens: a warp per (token, head)
    if ((a.q_stride | a.k_stride | a.v_stride) & 3) return false;
    const uintptr_t ptrs = (uintptr_t)a.q_in | (uintptr_t)a.k_in | (uintptr_t)a.v_in | (uintptr_t)a.q_gain |
                           (uintptr_t)a.k_gain | (uintptr_t)a.cos_sin | (uintptr_t)a.q_out | (uintptr_t)a.k_out |
                           (uintptr_t)a.cache;
    if (ptrs % 16) return false;
    switch (a.hd) {
        case 32: launch_qkv_wide_lph<G, 4>(a, s); break;
        case 64: launch_qkv_wide_lph<G, 8>(a, s); break;
        case 128: launch_qkv_wide_lph<G, 16>(a, s); break;
        default: launch_qkv_wide_lph<G, 32>(a, s); break;
    }
    return true;
}

constexpr int QKV_WARPS_PER_BLOCK = 8;
constexpr int QKV_TOKENS_PER_WARP = 4;

template <typename I, typename O, typename G, int NP>
static bool launch_qkv_vec_np(const QkvArgs& a, cudaStream_t s) {
    const int heads = a.nh + 2 * a.nkv;
    const unsigned head_groups = (unsigned)((heads + QKV_WARPS_PER_BLOCK - 1) / QKV_WARPS_PER_BLOCK);
    if (head_groups > 65535u) return false;
    // enough (token, head) pairs to fill the GPU several times over: a warp takes four tokens
    if ((long long)a.tokens * heads >= 148LL * 64 * QKV_TOKENS_PER_WARP) {
        const unsigned token_groups = (unsigned)((a.tokens + QKV_TOKENS_PER_WARP - 1) / QKV_TOKENS_PER_WARP);
        llme_launch(qkv_post_vec_kernel<I, O, G, NP, QKV_TOKENS_PER_WARP>, dim3(token_groups, head_groups), dim3(QKV_WARPS_PER_BLOCK * 32), 0, s, a);
    } else {
        llme_launch(qkv_post_vec_kernel<I, O, G, NP, 1>, dim3((unsigned)a.tokens, head_groups), dim3(QKV_WARPS_PER_BLOCK * 32), 0, s, a);
    }
    return true;
}

template <typename I, typename O, typename G>
static bool launch_qkv_vec(const QkvArgs& a, cudaStream_t s) {
    if (a.hd % 4 || a.hd > 512) return false;
    if ((a.q_stride | a.k_stride | a.v_stride) & 1) return false;
    const uintptr_t ptrs = (uintptr_t)a.q_in | (uintptr_t)a.k_in | (uintptr_t)a.v_in | (uintptr_t)a.q_gain |
                           (uintptr_t)a.k_gain | (uintptr_t)a.cos_sin | (uintptr_t)a.q_out | (uintptr_t)a.k_out |
                           (uintptr_t)a.cache;
    if (ptrs % 8) return false;
    const int half = a.hd / 2;
    if (half <= 64) return launch_qkv_vec_np<I, O, G, 1>(a, s);
    if (half <= 128) return launch_qkv_vec_np<I, O, G, 2>(a, s);
    return launch_qkv_vec_np<I, O, G, 4>(a, s);
}

template <typename I, typename O>
static int dispatch_qkv_gain(const QkvArgs& a, cudaStream_t s) {
    const long long warps = (long long)a.tokens * (a.nh + 2 * a.nkv);
    const int wpb = 8;
    const long long blocks = (warps + wpb - 1) / wpb;
    if (blocks > 2147483647LL) LLME_REFUSE("qkv_post: too many (token, head) pairs for one launch");
    constexpr bool BF16_IO = std::is_same<I, __nv_bfloat16>::value && std::is_same<O, __nv_bfloat16>::value;
    if (a.gain_dtype == LLME_F32 || !(a.q_gain || a.k_gain)) {
        if (BF16_IO && launch_qkv_wide<float>(a, s)) LLME_LAUNCH_STATUS();
        if (launch_qkv_vec<I, O, float>(a, s)) LLME_LAUNCH_STATUS();
    } else if (a.gain_dtype == LLME_BF16) {
        if (BF16_IO && launch_qkv_wide<__nv_bfloat16>(a, s)) LLME_LAUNCH_STATUS();
        if (launch_qkv_vec<I, O, __nv_bfloat16>(a, s)) LLME_LAUNCH_STATUS();
    }
    if (a.gain_dtype == LLME_F32) llme_launch(qkv_post_kernel<I, O, float>, dim3((unsigned)blocks), dim3(wpb * 32), 0, s, a);
    else if (a.gain_dtype == LLME_BF16) llme_launch(qkv_post_kernel<I, O, __nv_bfloat16>, dim3((unsigned)blocks), dim3(wpb * 32), 0, s, a);
    else LLME_REFUSE("qkv_post: unsupported gain dtype %d", a.gain_dtype);
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_qkv_post(const QkvArgs* args, int in_dtype, int out_dtype, cudaStream_t stream) {
    const QkvArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (a.nh < 0 || a.nkv < 0 || a.hd <= 0 || (a.hd & 1)) LLME_REFUSE("qkv_post: head_dim must be positive and even, got %d", a.hd);
    if (a.cache && (!a.slot_mapping || a.page_size <= 0)) LLME_REFUSE("qkv_post: a cache needs slot_mapping and page_size");
    if (a.cos_sin && (!a.positions || a.max_positions <= 0)) LLME_REFUSE("qkv_post: rotation needs positions");
    if ((a.q_gain || a.k_gain) && !(a.eps > 0.0f)) LLME_REFUSE("qkv_post: eps must be positive");
    if (in_dtype == LLME_F32 && out_dtype == LLME_F32) return dispatch_qkv_gain<float, float>(a, stream);
    if (in_dtype == LLME_BF16 && out_dtype == LLME_BF16) return dispatch_qkv_gain<__nv_bfloat16, __nv_bfloat16>(a, stream);
    if (in_dtype == LLME_F32 && out_dtype == LLME_BF16) return dispatch_qkv_gain<float, __nv_bfloat16>(a, stream);
    if (in_dtype == LLME_BF16 && out_dtype == LLME_F32) return dispatch_qkv_gain<__nv_bfloat16, float>(a, stream);
    LLME_REFUSE("qkv_post: unsupported in/out dtype %d/%d", in_dtype, out_dtype);
}

// ----------------------------------------------------------------------------- SwiGLU
// in [T, 2*inter] = gate | up;  out[t, i] = gate / (1 + exp(-gate)) * up.
template <typename I, typename O>
__global__ void swiglu_kernel(const I* __restrict__ in, O* __restrict__ out, long long total, int inter) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const long long t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = to_f32(in[t * 2 * inter + i]);
        const float u = to_f32(in[t * 2 * inter + inter + i]);
        if (sizeof(I) == 2) out[idx] = from_f32<O>(silu_mul_bf16(g, u));
        else out[idx] = from_f32<O>((g / (1.0f + expf(-g))) * u);
    }
}

// Vector form: 8 values per thread (two 16-byte loads, one 16-byte store for bfloat16), grid (column chunks, tokens).
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int inter) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= inter) return;
    const size_t t = blockIdx.y;
    const uint4 gv = *reinterpret_cast<const uint4*>(in + t * 2 * inter + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(in + t * 2 * inter + inter + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(silu_mul_bf16(g.x, u.x), silu_mul_bf16(g.y, u.y));
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = ov;
}

LLME_API int llme_swiglu(const void* in, int in_dtype, void* out, int out_dtype, int tokens, int inter,
                         cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (!in || !out || inter <= 0) LLME_REFUSE("swiglu: null pointer or non-positive size");
    if (in_dtype == LLME_BF16 && out_dtype == LLME_BF16 && inter % 8 == 0 && tokens <= 65535 &&
        ((uintptr_t)in | (uintptr_t)out) % 16 == 0) {
        const int threads = inter >= 2048 ? 256 : 64;
        dim3 grid((inter / 8 + threads - 1) / threads, tokens);
        llme_launch(swiglu_bf16x8_kernel, dim3(grid), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, inter);
        LLME_LAUNCH_STATUS();
    }
    const long long total = (long long)tokens * inter;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (in_dtype == LLME_F32 && out_dtype == LLME_F32)
        llme_launch(swiglu_kernel<float, float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)in, (float*)out, total, inter);
    else if (in_dtype == LLME_BF16 && out_dtype == LLME_BF16)
        llme_launch(swiglu_kernel<__nv_bfloat16, __nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, inter);
    else if (in_dtype == LLME_F32 && out_dtype == LLME_BF16)
        llme_launch(swiglu_kernel<float, __nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)in, (__nv_bfloat16*)out, total, inter);
    else
        LLME_REFUSE("swiglu: unsupported in/out dtype %d/%d", in_dtype, out_dtype);
    LLME_LAUNCH_STATUS();
}
