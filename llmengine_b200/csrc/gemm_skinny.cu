// out[M,N] = x[M,K] * W[N,K]^T for a handful of tokens (M <= 16), bfloat16 operands, 32-bit
// accumulation: the matrix product of a decode step, which is bound by reading W once from HBM.
//
// The roles are swapped with respect to a large product: 16 rows of W are the M side of a
// mma.sync.m16n8k16 tile and the tokens are its N side, so no tensor-core row is wasted on padding.
// Nothing goes through shared memory on the way in: the order in which the k values of a dot product
// are added is free, so within every block of 32 k values the four lanes of a quad take 8 consecutive
// values each, for W and for x alike.  A lane's operands for two tensor-core steps are then exactly one
// 16-byte load of a W row (two rows per lane) and one 16-byte load of an x row, straight into the
// registers the instruction reads.  How many bytes are in flight is then a matter of registers and
// resident warps, not of shared-memory stages.
//
// A block owns one group of 16 rows of W.  Its eight warps take the 64-wide chunks of K in turn (warp w:
// chunks w, w+8, ...); at the end the eight partial sums of every output are added in a fixed order.  A
// token's result does not depend on how many other tokens are in the call.  (A grid of as many blocks as
// the GPU keeps resident, each with an equal share of (row group, chunk) units and shared row groups
// finished by the block that comes second, was measured and was slower: 14.7 against 12.4 us for
// 6144 x 4096, 37.6 against 33.6 us for 24576 x 4096; short shares keep too few loads in flight.)
//
// A second entry point fuses the SwiGLU activation of a feed-forward: W = [gate | up] with `inter` rows
// each; a row group is then 8 gate rows and the 8 up rows of the same outputs, and the block stores
// silu(gate) * up directly.
//
// Reference counterpart: sgemm_nt_kernel / cublasSgemm for Linear (src/runtime/kernels/cuda_kernels.cu:282-294,
// :892-908), where a decode step runs the same kernels as a prompt; swiglu_kernel (:360-372).
#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int KC = 64;            // k values per chunk (two blocks of 32)
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
int g_dense = 0;                  // llme_gemm_skinny_dense()
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// weights are read once: do not keep them in L1
__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct SkinnyArgs {
    const bf16* x; long long ldx;
    const bf16* w; long long ldw;
    void* out; long long ldo;
    int M, N, K;
    int inter;      // 0: plain product; > 0: W = [gate | up] of `inter` rows each and out = silu(gate) * up
};

// MT: 8-token tiles (1: M <= 8, 2: M <= 16).  Every block of a token's row re-reads the tokens' operands from L2, so
// beyond 16 tokens that traffic outgrows the weights' and the library product is faster (measured at 17 to 32 tokens:
// 2.1 to 3.6 TB/s against 4.1 to 5.2 TB/s).
// UNROLL: chunks of K whose loads a warp issues together; BLOCKS: blocks that must fit an SM (2 with 4 chunks in flight,
// 3 with 2: fewer bytes in flight per SM, but 444 places instead of 296 for the row groups of a product).
template <int MT, typename O, int UNROLL, int BLOCKS>
__global__ void __launch_bounds__(THREADS, BLOCKS) gemm_skinny_kernel(SkinnyArgs a) {
    __shared__ float red[WARPS][MT * 8][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane & 3, r = lane >> 2;
    const bool act = a.inter > 0;
    const int rg = blockIdx.x;                                      // this block's row group
    // rows of W this lane reads (clamped: a row past the end is read but never stored)
    int row0, row1;
    if (act) {
        row0 = min(rg * 8 + r, a.inter - 1);
        row1 = a.inter + row0;
    } else {
        row0 = min(rg * 16 + r, a.N - 1);
        row1 = min(rg * 16 + r + 8, a.N - 1);
    }
    const bf16* w0 = a.w + (size_t)row0 * a.ldw + quad * 8;
    const bf16* w1 = a.w + (size_t)row1 * a.ldw + quad * 8;
    // the token rows of x this lane reads (token = lane / 4 of each 8-token tile)
    const bf16* xr[MT];
    bool xok[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        xok[m] = m * 8 + r < a.M;
        xr[m] = a.x + (size_t)(xok[m] ? m * 8 + r : 0) * a.ldx + quad * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;

    // A warp takes the chunks warp, warp + 8, ... of K, four at a time with all their loads issued together; a chunk
    // past the end of K (the last round of a K that is no multiple of 4 x 8 x 64, or the open end of the last chunk)
    // contributes zeros.  Whatever K is, the loads of a round are in flight together: a round of single chunks at the
    // end left a K of 5,120 or 17,408 at two thirds of the rate of a K of 4,096.
    const int chunks_all = (a.K + KC - 1) / KC;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    bool first = true;
    for (int c = warp; c < chunks_all; c += UNROLL * WARPS) {
        uint4 wa[UNROLL][2], wb[UNROLL][2], xv[UNROLL][MT][2];
        bool ok[UNROLL][2];
        // the weights do not depend on the kernel before this one: the first group of them is requested
        // before waiting for it; x, which that kernel produced, only after
#pragma unroll
        for (int q = 0; q < UNROLL; ++q) {
            const int k = (c + q * WARPS) * KC;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                ok[q][b] = k + b * 32 + quad * 8 < a.K;       // K is a multiple of 8: a piece is inside or outside
                wa[q][b] = ok[q][b] ? load_stream(w0 + k + b * 32) : zero;
                wb[q][b] = ok[q][b] ? load_stream(w1 + k + b * 32) : zero;
            }
        }
        if (first) {
            // The next kernel may be scheduled from here on: its blocks move in as this kernel's leave (this kernel's
            // blocks fill the SMs' registers, so nothing of it is displaced), and its own first loads, or its tables,
            // are under way when this kernel ends.  (A layer's operations at batch 8 take 88.2 us so, 89.8 us with
            // the successor let in only before this kernel's short epilogue.)
            pdl_launch_dependents();
            pdl_wait();
            first = false;
        }
#pragma unroll
        for (int q = 0; q < UNROLL; ++q) {
            const int k = (c + q * WARPS) * KC;
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    xv[q][m][b] = (ok[q][b] && xok[m]) ? *reinterpret_cast<const uint4*>(xr[m] + k + b * 32) : zero;
        }
#pragma unroll
        for (int q = 0; q < UNROLL; ++q)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma_bf16(acc[m], wa[q][b].x, wb[q][b].x, wa[q][b].y, wb[q][b].y, xv[q][m][b].x, xv[q][m][b].y);
                    mma_bf16(acc[m], wa[q][b].z, wb[q][b].z, wa[q][b].w, wb[q][b].w, xv[q][m][b].z, xv[q][m][b].w);
                }
    }
    if (first) pdl_wait();

    // the warps' partial sums, added in a fixed order: value (token, row) at index token * 16 + row
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][m * 8 + quad * 2 + (i & 1)][r + (i >> 1) * 8] = acc[m][i];
    __syncthreads();
    auto total = [&](int i) -> float {
        float v = red[0][i >> 4][i & 15];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) v += red[w][i >> 4][i & 15];
        return v;
    };
    if (!act) {
        for (int i = threadIdx.x; i < MT * 8 * 16; i += THREADS) {
            const int tok = i >> 4, row = rg * 16 + (i & 15);
            if (tok < a.M && row < a.N) reinterpret_cast<O*>(a.out)[(size_t)tok * a.ldo + row] = from_f32<O>(total(i));
        }
    } else {
        // rows 0..7 of the group are gate rows, rows 8..15 the up rows of the same outputs; both go through
        // bfloat16 first, as they do when the activation is a kernel of its own
        for (int i = threadIdx.x; i < MT * 8 * 8; i += THREADS) {
            const int tok = i >> 3, j = i & 7, col = rg * 8 + j;
            if (tok < a.M && col < a.inter) {
                const float g = __bfloat162float(__float2bfloat16_rn(total(tok * 16 + j)));
                const float up = __bfloat162float(__float2bfloat16_rn(total(tok * 16 + j + 8)));
                reinterpret_cast<O*>(a.out)[(size_t)tok * a.ldo + col] = from_f32<O>(silu_mul_bf16(g, up));
            }
        }
    }
}

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 148;
        return v;
    }();
    return n;
}

template <int MT, typename O>
int launch(const SkinnyArgs& a, cudaStream_t s) {
    const int groups = a.inter > 0 ? (a.inter + 7) / 8 : (a.N + 15) / 16;
    // Two blocks per SM (296 places) keep the most bytes in flight.  Row groups that fill their rounds of 296 badly
    // but rounds of 444 well (6,144 rows: 384 groups; 5,120 rows: 320; 10,240 rows: 640) go to three lighter blocks
    // per SM: measured at 8 tokens, 5120 x 25600 takes 42.9 us against 56.9 us (cuBLAS 44.6), 6144 x 4096 10.6
    // against 11.0 (cuBLAS 11.1); with 256 groups, which fit one round either way, the lighter blocks lose (9.0
    // against 8.2 us).  The executor's choice between this kernel and the library uses the same two figures.
    const long long p2 = 2LL * sm_count(), p3 = 3LL * sm_count();
    const long long w2 = (groups + p2 - 1) / p2 * p2, w3 = (groups + p3 - 1) / p3 * p3;          // places of the rounds taken
    const bool fills2 = 10LL * groups >= 8 * w2, fills3 = 10LL * groups >= 7 * w3;
    const bool dense = MT == 1 && (g_dense == 2 || (g_dense == 0 && !fills2 && fills3 && 4LL * groups > p2));
    if (dense) llme_launch(gemm_skinny_kernel<MT, O, 2, 3>, dim3(groups), dim3(THREADS), 0, s, a);
    else llme_launch(gemm_skinny_kernel<MT, O, 4, 2>, dim3(groups), dim3(THREADS), 0, s, a);
    LLME_LAUNCH_STATUS();
}

template <typename O>
int dispatch(const SkinnyArgs& a, cudaStream_t s) {
    return a.M <= 8 ? launch<1, O>(a, s) : launch<2, O>(a, s);
}

}  // namespace

// 0 (the default): three lighter blocks per SM where the row groups then fit one round; 1: never; 2: always (up to 8 tokens).
LLME_API int llme_gemm_skinny_dense(int how) {
    if (how >= 0 && how <= 2) g_dense = how;
    return g_dense;
}

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
    SkinnyArgs a{(const bf16*)x, ldx, (const bf16*)w, ldw, out, ldo, M, N, K, 0};
    if (out_dtype == LLME_F32) return dispatch<float>(a, stream);
    if (out_dtype == LLME_BF16) return dispatch<bf16>(a, stream);
    LLME_REFUSE("gemm_skinny: unsupported output dtype %d", out_dtype);
}

// out[M, inter] = silu(x * Wg^T) * (x * Wu^T) with W = [Wg | Wu] stacked by rows ([2 * inter, K]); out bfloat16 or float.
LLME_API int llme_gemm_skinny_swiglu_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out,
                                          int out_dtype, long long ldo, int M, int inter, int K, cudaStream_t stream) {
    if (M <= 0 || inter <= 0) return 0;
    if (!x || !w || !out) LLME_REFUSE("gemm_skinny: null pointer");
    if (inter > (1 << 29) || !llme_gemm_skinny_supports(M, 2 * inter, K, ldx, ldw)) LLME_REFUSE("gemm_skinny: M=%d inter=%d K=%d ldx=%lld ldw=%lld is not supported (M <= 16, K and strides multiples of 8)", M, inter, K, ldx, ldw);
    if (((uintptr_t)x | (uintptr_t)w) % 16) LLME_REFUSE("gemm_skinny: operands must be 16-byte aligned");
    if (ldo < inter) LLME_REFUSE("gemm_skinny: output row stride shorter than the row");
    SkinnyArgs a{(const bf16*)x, ldx, (const bf16*)w, ldw, out, ldo, M, 2 * inter, K, inter};
    if (out_dtype == LLME_F32) return dispatch<float>(a, stream);
    if (out_dtype == LLME_BF16) return dispatch<bf16>(a, stream);
    LLME_REFUSE("gemm_skinny: unsupported output dtype %d", out_dtype);
}
