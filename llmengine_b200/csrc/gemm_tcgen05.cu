// out[M,N] = x[M,K] * W[N,K]^T for many tokens (prompt portions), bfloat16 operands, 32-bit
// accumulation, on the fifth-generation tensor cores of sm_100a:
//
//   TMA (cp.async.bulk.tensor) brings 128 x 64 tiles of x and BN x 64 tiles of W into shared memory
//   with the 128-byte swizzle, STAGES deep, completion counted on mbarriers;
//   one thread issues tcgen05.mma (kind::f16, 128 x BN x 16 per instruction) with both operands read
//   from shared memory through matrix descriptors and the accumulator living in tensor memory (TMEM);
//   tcgen05.commit releases a shared-memory stage to the producer as soon as the instructions that
//   read it have finished, and at the end tells the epilogue that the accumulator is complete;
//   four epilogue warps read the accumulator back with tcgen05.ld (32 lanes x 32 columns each),
//   convert and store it.
//
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner and MMA issuer, warps 2..5 = epilogue.
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel sets an error flag, stops
// issuing work, waits (again bounded) for its copies in flight, frees its tensor memory and returns;
// llme_gemm_tc_status() reports the flag.
//
// Reference counterpart: the Linear op of the reference runs cublasSgemm or a one-thread-per-output
// kernel (src/runtime/kernels/cuda_kernels.cu:282-294, :892-908); it has no tensor-core code of its own.
#include <cuda.h>

#include "common.cuh"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr unsigned WAIT_LIMIT = 1u << 20;   // polls (each may suspend for a while): far beyond any legitimate wait

__device__ int g_status = 0;           // 0 = fine; otherwise where a wait gave up

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `where`) when the limit is reached or another role gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int where) {
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = where;
    atomicCAS(&g_status, 0, where);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major tile written by TMA with the 128-byte swizzle; rows are 128
// bytes, eight rows form a 1024-byte group (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFFu) >> 4);          // start address, bits [0,14)
    d |= (unsigned long long)1 << 16;                                      // leading byte offset (unused here)
    d |= (unsigned long long)(1024 >> 4) << 32;                            // stride byte offset, bits [32,46)
    d |= (unsigned long long)1 << 46;                                      // version
    d |= (unsigned long long)2 << 61;                                      // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16: D = F32, A = B = BF16, both K-major, shape M x N.
__host__ __device__ constexpr unsigned umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(unsigned addr, unsigned (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(addr));
}

struct TcArgs {
    void* out; long long ldo;
    int M, N, K;
};

template <int BN, int STAGES, typename O>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, TcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + STAGES * A_BYTES;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(b_tiles + STAGES * B_BYTES);
    unsigned long long* empty = full + STAGES;
    unsigned long long* acc_full = empty + STAGES;
    unsigned* tmem_holder = reinterpret_cast<unsigned*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int k_blocks = (a.K + BK - 1) / BK;
    constexpr unsigned TMEM_COLS = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                      // one warp allocates the accumulator's tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(empty + s, ((kb / STAGES) - 1) & 1, abort_flag, 1)) break;
                if (*abort_flag) break;
                mbar_expect_tx(full + s, A_BYTES + B_BYTES);
                tma_load_2d(a_tiles + s * A_BYTES, &map_x, kb * BK, m0, full + s);
                tma_load_2d(b_tiles + s * B_BYTES, &map_w, kb * BK, n0, full + s);
                issued = kb + 1;
            }
            if (*abort_flag) {
                // gave up somewhere: let the copies that are still in flight land before the block exits
                for (int kb = max(0, issued - STAGES); kb < issued; ++kb) {
                    const int s = kb % STAGES;
                    for (unsigned i = 0; i < WAIT_LIMIT && !mbar_try_wait(full + s, (kb / STAGES) & 1); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc = umma_idesc(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % STAGES;
                ok = mbar_wait(full + s, (kb / STAGES) & 1, abort_flag, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long da = umma_desc(a_tiles + s * A_BYTES);
                const unsigned long long db = umma_desc(b_tiles + s * B_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // the next 16 k values lie 32 bytes further inside the swizzled rows: +2 in the address field
                    umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty + s);           // the stage is free once these instructions have read it
            }
            umma_commit(acc_full);                // all instructions done: the accumulator is complete
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;             // the TMEM lanes this warp may read: 32 * (warp % 4) ...
        const bool ok = mbar_wait(acc_full, 0, abort_flag, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                unsigned v[32];
                tmem_ld_32x32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(c * 32), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col = n0 + c * 32;
                if (row < a.M && col < a.N) {
                    O* dst = reinterpret_cast<O*>(a.out) + (size_t)row * a.ldo + col;
                    if (col + 32 <= a.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        if (sizeof(O) == 4) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 pk;
                                unsigned* pw = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                                    pw[e] = *reinterpret_cast<unsigned*>(&h);
                                }
                                reinterpret_cast<uint4*>(dst)[j] = pk;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < a.N) dst[j] = from_f32<O>(__uint_as_float(v[j]));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld (elements), cut into boxes of box_rows x 64, 128-byte swizzle;
// parts of a box outside the matrix read as zeros.
int make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) LLME_REFUSE("gemm_tc: cuTensorMapEncodeTiled is not available in this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) LLME_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int BN, int STAGES, typename O>
int launch(const void* x, long long ldx, const void* w, long long ldw, const TcArgs& a, cudaStream_t s) {
    alignas(64) CUtensorMap mx, mw;
    if (int rc = make_map(&mx, x, a.M, a.K, ldx, BM)) return rc;
    if (int rc = make_map(&mw, w, a.N, a.K, ldw, BN)) return rc;
    constexpr size_t smem = 1024 + (size_t)STAGES * (BM + BN) * BK * 2 + (2 * STAGES + 1) * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLME_REFUSE("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
    if (grid.y > 65535) LLME_REFUSE("gemm_tc: M = %d needs more than 65535 row tiles", a.M);
    gemm_tc_kernel<BN, STAGES, O><<<grid, THREADS, smem, s>>>(mx, mw, a);
    LLME_LAUNCH_STATUS();
}

}  // namespace

// 1 if llme_gemm_tc_bf16 takes this problem.
LLME_API int llme_gemm_tc_supports(int M, int N, int K, long long ldx, long long ldw, long long ldo) {
    return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldo >= N;
}

// x [M,K], W [N,K] bfloat16 (row strides ldx, ldw in elements, base addresses 16-byte aligned);
// out [M,N] float (out_dtype 0) or bfloat16 (1), row stride ldo.
LLME_API int llme_gemm_tc_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                               long long ldo, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!x || !w || !out) LLME_REFUSE("gemm_tc: null pointer");
    if (!llme_gemm_tc_supports(M, N, K, ldx, ldw, ldo)) LLME_REFUSE("gemm_tc: M=%d N=%d K=%d ldx=%lld ldw=%lld ldo=%lld is not supported (K and operand strides must be multiples of 8)", M, N, K, ldx, ldw, ldo);
    if (((uintptr_t)x | (uintptr_t)w) % 16) LLME_REFUSE("gemm_tc: operands must be 16-byte aligned");
    TcArgs a{out, ldo, M, N, K};
    if (out_dtype == LLME_F32) return N > 128 ? launch<256, 4, float>(x, ldx, w, ldw, a, stream) : launch<128, 6, float>(x, ldx, w, ldw, a, stream);
    if (out_dtype == LLME_BF16) return N > 128 ? launch<256, 4, bf16>(x, ldx, w, ldw, a, stream) : launch<128, 6, bf16>(x, ldx, w, ldw, a, stream);
    LLME_REFUSE("gemm_tc: unsupported output dtype %d", out_dtype);
}

// Reads and clears the error flag of the kernels (synchronises the device).  0 = no wait ever gave up.
LLME_API int llme_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
