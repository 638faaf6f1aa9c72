// True 32-bit matrix product C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores (FMA, no
// tensor cores, no reduced-precision mode).  Every output element is one accumulator
// that adds its K products in the order k = 0..K-1, so a row's result does not depend
// on how many other rows are in the launch.  It is the matrix product of the whole
// 32-bit path and the plain twin that the tensor-core kernels are checked against.
//
// Reference counterparts: sgemm_nt_kernel (src/runtime/kernels/cuda_kernels.cu:282-294,
// one thread per output, no tiling) and the cublasSgemm call of sgemm_nt_cublas (:892-908).
#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename WT>
__global__ void __launch_bounds__(256) gemm_nt_f32_kernel(const float* __restrict__ A, const WT* __restrict__ W,
                                                          float* __restrict__ C, int M, int N, int K,
                                                          long long lda, long long ldw, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, each TM x TN outputs
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements per operand, 4 per thread; consecutive threads read consecutive k
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e >> 4, kk = e & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.0f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

// A [M,K] row stride lda; W [N,K] row stride ldw (float or bfloat16); C [M,N] row stride ldc.
LLME_API int llme_gemm_nt_f32(const float* A, const void* W, int w_dtype, float* C, int M, int N, int K,
                              long long lda, long long ldw, long long ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!A || !W || !C || K <= 0) LLME_REFUSE("gemm_f32: null pointer or non-positive K");
    if (lda < K || ldw < K || ldc < N) LLME_REFUSE("gemm_f32: a row stride is shorter than the row");
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) LLME_REFUSE("gemm_f32: M = %d needs more than 65535 row tiles", M);
    if (w_dtype == LLME_F32) gemm_nt_f32_kernel<float><<<grid, 256, 0, stream>>>(A, (const float*)W, C, M, N, K, lda, ldw, ldc);
    else if (w_dtype == LLME_BF16) gemm_nt_f32_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(A, (const __nv_bfloat16*)W, C, M, N, K, lda, ldw, ldc);
    else LLME_REFUSE("gemm_f32: unsupported weight dtype %d", w_dtype);
    LLME_LAUNCH_STATUS();
}
