// out[M,N] = x[M,K] * W[N,K]^T for a handful of tokens (M <= 16), bfloat16 operands, 32-bit
// accumulation: the matrix product of a decode step, which is bound by reading W once from HBM.
//
// The roles are swapped with respect to a large product: 16 rows of W are the M side of a
// mma.sync.m16n8k16 tile and the tokens are its N side, so no tensor-core row is wasted on padding.
// A block owns RT*16 rows of W and all of K.  Its four warps take the 64-wide chunks of K in turn
// (warp w: chunks w, w+4, ...) and each streams its chunks of W, with the matching chunk of x, through a
// pipeline of its own (cp.async, STAGES chunks per warp, no block-wide barrier in the loop), so that
// enough bytes are in flight per SM to cover the memory latency.  At the end the four partial sums of
// every output are added in a fixed order.  A token's result does not depend on how many other tokens
// are in the call.
//
// Reference counterpart: sgemm_nt_kernel / cublasSgemm for Linear (src/runtime/kernels/cuda_kernels.cu:282-294,
// :892-908), where a decode step runs the same kernels as a prompt.
#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int KC = 64;            // k values per chunk
constexpr int LDK = KC + 8;       // padded row length in shared memory (elements)
constexpr int STAGES = 4;
constexpr int THREADS = 128;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct SkinnyArgs {
    const bf16* x; long long ldx;
    const bf16* w; long long ldw;
    void* out; long long ldo;
    int M, N, K;
};

// RT: 16-row tiles of W per block.  MT: 8-token tiles (1: M <= 8, 2: M <= 16).
template <int RT, int MT, typename O>
__global__ void __launch_bounds__(THREADS) gemm_skinny_kernel(SkinnyArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int ROWS = RT * 16, TOK = MT * 8;
    constexpr int STAGE = (ROWS + TOK) * LDK;            // elements: W rows, then x rows
    bf16* base = reinterpret_cast<bf16*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bf16* mine = base + (size_t)warp * STAGES * STAGE;
    const int n0 = blockIdx.x * ROWS;
    const int chunks = (a.K + KC - 1) / KC;

    auto load_w = [&](int stage, int chunk) {
        bf16* ws = mine + (size_t)stage * STAGE;
        const int k0 = chunk * KC;
#pragma unroll
        for (int c = lane; c < ROWS * 8; c += 32) {      // 8 pieces of 16 bytes per row
            const int row = c >> 3, piece = c & 7;
            const int n = n0 + row, k = k0 + piece * 8;
            const bool valid = n < a.N && k < a.K;       // K is a multiple of 8: a piece is inside or outside
            cp_async_16(ws + row * LDK + piece * 8, valid ? a.w + (size_t)n * a.ldw + k : a.w, valid);
        }
    };
    auto load_x = [&](int stage, int chunk) {
        bf16* xs = mine + (size_t)stage * STAGE + ROWS * LDK;
        const int k0 = chunk * KC;
#pragma unroll
        for (int c = lane; c < TOK * 8; c += 32) {
            const int row = c >> 3, piece = c & 7;
            const int k = k0 + piece * 8;
            const bool valid = row < a.M && k < a.K;
            cp_async_16(xs + row * LDK + piece * 8, valid ? a.x + (size_t)row * a.ldx + k : a.x, valid);
        }
    };

    float acc[RT][MT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m][0] = acc[r][m][1] = acc[r][m][2] = acc[r][m][3] = 0.0f;

    // The weights do not depend on the kernel before this one: their first chunks are requested before
    // waiting for it; x, which it produced, only after.  (All these weight copies fall into the first
    // group, which the first wait below then covers.)
    pdl_launch_dependents();
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        const int chunk = warp + 4 * st;
        if (chunk < chunks) load_w(st, chunk);
    }
    pdl_wait();
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        const int chunk = warp + 4 * st;
        if (chunk < chunks) load_x(st, chunk);
        cp_async_commit();
    }
    int n = 0;
    for (int chunk = warp; chunk < chunks; chunk += 4, ++n) {
        const int ahead = chunk + 4 * (STAGES - 1);
        if (ahead < chunks) {
            load_w((n + STAGES - 1) % STAGES, ahead);
            load_x((n + STAGES - 1) % STAGES, ahead);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const bf16* ws = mine + (size_t)(n % STAGES) * STAGE;
        const bf16* xs = ws + ROWS * LDK;
#pragma unroll
        for (int kp = 0; kp < KC / 32; ++kp) {           // two k-steps of 16 at a time
            unsigned bx[2][MT][2];
            if (MT == 1) {
                // tokens 0-7: one load brings the operands of both k-steps
                unsigned t4[4];
                ldmatrix_x4(t4, xs + (lane & 7) * LDK + kp * 32 + (lane >> 3) * 8);
                bx[0][0][0] = t4[0]; bx[0][0][1] = t4[1];
                bx[1][0][0] = t4[2]; bx[1][0][1] = t4[3];
            } else {
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    unsigned t4[4];
                    const int mi = lane >> 3;
                    ldmatrix_x4(t4, xs + ((lane & 7) + (mi >> 1) * 8) * LDK + (kp * 2 + ks) * 16 + (mi & 1) * 8);
                    bx[ks][0][0] = t4[0]; bx[ks][0][1] = t4[1];
                    bx[ks][MT - 1][0] = t4[2]; bx[ks][MT - 1][1] = t4[3];
                }
            }
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    unsigned af[4];
                    ldmatrix_x4(af, ws + (r * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (kp * 2 + ks) * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int m = 0; m < MT; ++m) mma_bf16(acc[r][m], af, bx[ks][m][0], bx[ks][m][1]);
                }
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();

    // sum the four warps' partial results in a fixed order and write out[token][n0 + row]
    float* red = reinterpret_cast<float*>(smem_raw);       // [4 warps][TOK][ROWS]
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int row = r * 16 + (lane >> 2) + (c >> 1) * 8;
                const int tok = m * 8 + (lane & 3) * 2 + (c & 1);
                red[((size_t)warp * TOK + tok) * ROWS + row] = acc[r][m][c];
            }
    __syncthreads();
    for (int i = threadIdx.x; i < TOK * ROWS; i += THREADS) {
        const int tok = i / ROWS, row = i - tok * ROWS;
        if (tok < a.M && n0 + row < a.N) {
            const float v = ((red[i] + red[TOK * ROWS + i]) + red[2 * TOK * ROWS + i]) + red[3 * TOK * ROWS + i];
            reinterpret_cast<O*>(a.out)[(size_t)tok * a.ldo + n0 + row] = from_f32<O>(v);
        }
    }
}

template <int RT, int MT, typename O>
int launch(const SkinnyArgs& a, cudaStream_t s) {
    constexpr size_t smem = (size_t)4 * STAGES * (RT * 16 + MT * 8) * LDK * sizeof(bf16);
    static_assert((size_t)4 * MT * 8 * RT * 16 * sizeof(float) <= smem, "the reduction buffer must fit the stages");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<RT, MT, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLME_REFUSE("gemm_skinny: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int blocks = (a.N + RT * 16 - 1) / (RT * 16);
    llme_launch(gemm_skinny_kernel<RT, MT, O>, dim3(blocks), dim3(THREADS), smem, s, a);
    LLME_LAUNCH_STATUS();
}

template <typename O>
int dispatch(const SkinnyArgs& a, cudaStream_t s) {
    // two 16-row tiles per block halve the re-reading of x, but need enough rows to fill the GPU
    const bool wide = (a.N + 31) / 32 >= 2 * 148;
    if (a.M <= 8) return wide ? launch<2, 1, O>(a, s) : launch<1, 1, O>(a, s);
    return wide ? launch<2, 2, O>(a, s) : launch<1, 2, O>(a, s);
}

}  // namespace

// 1 if llme_gemm_skinny_bf16 takes this problem, 0 if the caller should use the general product.
LLME_API int llme_gemm_skinny_supports(int M, int N, int K, long long ldx, long long ldw) {
    return M >= 1 && M <= 16 && N >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

// x [M,K] and W [N,K] bfloat16 with row strides ldx, ldw (elements); out [M,N] float (out_dtype 0) or
// bfloat16 (1) with row stride ldo.
LLME_API int llme_gemm_skinny_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                                   long long ldo, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out) LLME_REFUSE("gemm_skinny: null pointer");
    if (!llme_gemm_skinny_supports(M, N, K, ldx, ldw)) LLME_REFUSE("gemm_skinny: M=%d N=%d K=%d ldx=%lld ldw=%lld is not supported (M <= 16, K and strides multiples of 8)", M, N, K, ldx, ldw);
    if (((uintptr_t)x | (uintptr_t)w) % 16) LLME_REFUSE("gemm_skinny: operands must be 16-byte aligned");
    if (ldo < N) LLME_REFUSE("gemm_skinny: output row stride shorter than the row");
    SkinnyArgs a{(const bf16*)x, ldx, (const bf16*)w, ldw, out, ldo, M, N, K};
    if (out_dtype == LLME_F32) return dispatch<float>(a, stream);
    if (out_dtype == LLME_BF16) return dispatch<bf16>(a, stream);
    LLME_REFUSE("gemm_skinny: unsupported output dtype %d", out_dtype);
}
