// Token sampling on the device, one block per row of logits, in the order of the
// reference's Sampler::sample (src/runtime/sampler.cpp:11-141): repetition penalty,
// temperature, softmax with the maximum subtracted, top-k, top-p, then either the
// argmax (greedy, first maximum wins) or a draw: the first candidate, in vocabulary
// order, at which the running sum of renormalised probabilities reaches the caller's
// uniform number u in (0,1).  (The reference walks the candidates in sorted order with a
// Mersenne-twister draw; the walk order and the source of u are this engine's own.)
// Top-k and top-p are found without sorting, by bisection on the bit pattern of
// exp(z - max): values that tie with the last kept candidate are all kept.
#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

// logit[row[i], token[i]] is divided (if positive) or multiplied (otherwise) by `penalty[row]`
// `count[i]` times: once per occurrence of the token in the request's history
// (src/runtime/sampler.cpp:22-32).  The (row, token) pairs must be distinct.
__global__ void repetition_penalty_kernel(float* logits, long long ld, const int* row, const int* token,
                                          const int* count, const float* penalty, int pairs, int vocab) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int tok = token[i];
    if (tok < 0 || tok >= vocab) return;
    const float p = penalty[row[i]];
    if (p == 1.0f) return;
    float* z = logits + (size_t)row[i] * ld + tok;
    float v = *z;
    for (int c = 0; c < count[i]; ++c) v = v > 0.0f ? v / p : v * p;
    *z = v;
}

LLME_API int llme_repetition_penalty(float* logits, long long ld, const int* row, const int* token, const int* count,
                                     const float* penalty, int pairs, int vocab, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (!logits || !row || !token || !count || !penalty) LLME_REFUSE("repetition_penalty: null pointer");
    llme_launch(repetition_penalty_kernel, dim3((pairs + 255) / 256), dim3(256), 0, stream, logits, ld, row, token, count, penalty, pairs, vocab);
    LLME_LAUNCH_STATUS();
}

struct SampleArgs {
    const float* logits; long long ld;
    int rows, vocab;
    const int* greedy;            // [rows] non-zero = argmax
    const float* temperature;     // [rows]; 1 or <= 0 = no scaling
    const int* top_k;             // [rows]; <= 0 or >= vocab = off
    const float* top_p;           // [rows]; outside (0,1) = off
    const float* u;               // [rows] in (0,1)
    int* out;                     // [rows]
};

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int t = (lane < (int)(blockDim.x >> 5)) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(SampleArgs a) {
    pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ float prefix[SAMPLE_THREADS + 1];
    __shared__ int found;
    const int r = blockIdx.x, tid = threadIdx.x, V = a.vocab;
    const float* z = a.logits + (size_t)r * a.ld;
    const float temp = a.temperature ? a.temperature[r] : 1.0f;
    const float inv_t = (temp != 1.0f && temp > 0.0f) ? 1.0f / temp : 1.0f;

    // maximum and its first index (NaN entries never win)
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = z[i] * inv_t;
        if (v > best) { best = v; best_i = i; }
    }
    const float m = block_max(best, fs);
    int cand = (best == m && best_i != 0x7fffffff) ? best_i : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((tid & 31) == 0) is[tid >> 5] = cand;
    __syncthreads();
    int arg = (tid & 31) < (SAMPLE_THREADS >> 5) ? is[tid & 31] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) arg = min(arg, __shfl_xor_sync(0xffffffffu, arg, o));
    if (arg == 0x7fffffff) arg = 0;            // every logit is -inf or NaN: the reference returns token 0

    const bool greedy = !a.greedy || a.greedy[r] != 0;
    if (greedy || !isfinite(m)) {
        // A non-finite maximum makes the reference fall back to a uniform distribution; for the
        // draw this engine then also returns the argmax slot (token 0 when all are -inf).
        if (tid == 0) a.out[r] = arg;
        return;
    }

    // e_i = exp(z_i - m) in [0, 1]; sum over the row
    float part = 0.0f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) part += expf(z[i] * inv_t - m);
    const float sum_all = block_sum(part, fs);

    unsigned thr = 0u;                          // keep e_i whose bit pattern is >= thr
    const int k = a.top_k ? a.top_k[r] : 0;
    if (k > 0 && k < V) {
        unsigned lo = 0u, hi = 0x3f800001u;     // count(e >= lo) >= k holds at lo, fails at hi
        while (hi - lo > 1u) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            int c = 0;
            for (int i = tid; i < V; i += SAMPLE_THREADS) c += (__float_as_uint(expf(z[i] * inv_t - m)) >= mid) ? 1 : 0;
            c = block_sum_int(c, is);
            if (c >= k) lo = mid; else hi = mid;
        }
        thr = lo;
    }
    const float tp = a.top_p ? a.top_p[r] : 0.0f;
    if (tp > 0.0f && tp < 1.0f) {
        const float need = tp * sum_all;
        unsigned lo = thr, hi = 0x3f800001u;
        // mass(e >= lo, kept) >= need ?  If even the whole kept set falls short, all of it stays.
        float s0 = 0.0f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float e = expf(z[i] * inv_t - m);
            s0 += (__float_as_uint(e) >= lo) ? e : 0.0f;
        }
        s0 = block_sum(s0, fs);
        if (s0 >= need) {
            while (hi - lo > 1u) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                float s = 0.0f;
                for (int i = tid; i < V; i += SAMPLE_THREADS) {
                    const float e = expf(z[i] * inv_t - m);
                    s += (__float_as_uint(e) >= mid) ? e : 0.0f;
                }
                s = block_sum(s, fs);
                if (s >= need) lo = mid; else hi = mid;
            }
            thr = lo;
        }
    }

    // Draw: thread t owns the contiguous indices [t*C, (t+1)*C); exclusive prefix of the chunk sums,
    // then the owner of the crossing walks its chunk.
    const int C = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int b = tid * C, e_end = min(V, b + C);
    float mine = 0.0f;
    for (int i = b; i < e_end; ++i) {
        const float e = expf(z[i] * inv_t - m);
        mine += (__float_as_uint(e) >= thr) ? e : 0.0f;
    }
    prefix[tid] = mine;
    if (tid == 0) found = 0x7fffffff;
    __syncthreads();
    if (tid < 32) {                              // serial-in-warp scan of 1024 chunk sums: fixed order
        const int per = SAMPLE_THREADS / 32;
        float run = 0.0f;
        for (int j = 0; j < per; ++j) run += prefix[tid * per + j];
        float incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, incl, o);
            if (tid >= o) incl += n;
        }
        float base = incl - run;
        for (int j = 0; j < per; ++j) {
            const float v = prefix[tid * per + j];
            prefix[tid * per + j] = base;        // exclusive prefix
            base += v;
        }
        if (tid == 31) prefix[SAMPLE_THREADS] = base;   // total of the kept mass
    }
    __syncthreads();
    // Thread t owns the interval (prefix[t], prefix[t+1]]: the intervals cover (0, total] without a gap.
    const float total = prefix[SAMPLE_THREADS];
    const float target = a.u[r] * total;
    const float before = prefix[tid];
    if (before < target && target <= prefix[tid + 1]) {
        float run = before;
        int pick = -1, last = -1;
        for (int i = b; i < e_end; ++i) {
            const float e = expf(z[i] * inv_t - m);
            if (__float_as_uint(e) >= thr && e > 0.0f) {
                run += e;
                last = i;
                if (run >= target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last;
        if (pick >= 0) atomicMin(&found, pick);
    }
    __syncthreads();
    if (tid == 0) a.out[r] = (found == 0x7fffffff) ? arg : found;
}

LLME_API int llme_sample(const SampleArgs* args, cudaStream_t stream) {
    const SampleArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (!a.logits || !a.out || a.vocab <= 0 || a.ld < a.vocab) LLME_REFUSE("sample: null pointer or bad sizes");
    if (!a.u) LLME_REFUSE("sample: the uniform numbers are missing");
    llme_launch(sample_kernel, dim3(a.rows), dim3(SAMPLE_THREADS), 0, stream, a);
    LLME_LAUNCH_STATUS();
}
