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
// From 129 tokens on, two blocks on neighbouring SMs share a 256 x 256 tile (tcgen05.mma.cta_group::2, see PAIR
// below): measured on the 8B shape at 2,048 tokens, 75 / 53 / 153 us for the q|k|v, output and down products against
// 81 / 57 / 161 us with one block per tile (cuBLAS: 72 / 51 / 157), 284 against 303 us for gate|up with the SwiGLU; at
// 8,192 tokens 289 / 194 / 704 us against 320 / 228 / 709 (cuBLAS: 301 / 259 / 806).
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

#include "umma.cuh"

int g_pairing = 0;      // llme_gemm_tc_pairing()

struct TcArgs {
    void* out; long long ldo;
    int M, N, K;
    int m_tiles, n_tiles;
    int inter;      // ACT kernels: W = [gate | up] with `inter` rows each, out[M, inter] = silu(gate) * up
};

// Persistent kernel: one block per SM walks over the output tiles (m fastest, so blocks that run together
// share a tile of W).  The accumulator is double-buffered in tensor memory (2 x BN columns): while the
// epilogue warps read tile i out of one buffer, the MMA warp already fills the other with tile i+1.
// TMA_STORE: the epilogue stages 32-row x 128-byte pieces in (swizzled) shared memory and writes them with
// cp.async.bulk.tensor stores; otherwise it stores from registers (any alignment of the output).
// ACT: the SwiGLU of a feed-forward in the epilogue.  W = [gate | up]; a tile's BN accumulator columns are
// BN/2 gate rows and the BN/2 up rows of the same outputs (two TMA boxes per stage), and the epilogue
// stores silu(gate) * up, BN/2 columns per tile, both factors rounded to bfloat16 first as they are when
// the activation is a kernel of its own.
//
// PAIR: two blocks on neighbouring SMs (a cluster of two) work on one 256 x BN tile with tcgen05.mma.cta_group::2.
// Each block loads its own 128 rows of x and HALF of the tile's rows of W; the instruction, issued by the first
// block of the pair alone, reads both halves from the two blocks' shared memory and adds into both blocks' tensor
// memory (128 lanes each).  A block then brings 32 KB per 64 k values from L2 instead of 48 KB for the same 128 x BN
// outputs, and one instruction does twice the work.  Both blocks' loads count on the first block's barrier (TMA with
// .cta_group::2, which lets a load signal the partner's barrier); tcgen05.commit with a two-block mask frees the stage
// in both blocks and tells both epilogues that the accumulator is complete; the second block's epilogue warps hand
// an accumulator buffer back with an arrive on the first block's barrier.  With ACT the first block's half of W is
// the gate rows and the second block's the up rows.
template <int BN, int STAGES, typename O, bool TMA_STORE, bool ACT, bool PAIR>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& map_x, const CUtensorMap& map_w, const CUtensorMap& map_o, const TcArgs& a) {
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;     // what THIS block holds of a stage
    constexpr int TILE_M = PAIR ? 2 * BM : BM;
    constexpr int STAGING = TMA_STORE ? 4 * 2 * 4096 : 0;          // 4 warps x 2 buffers x (32 rows x 128 bytes)
    unsigned char* a_tiles = smem;
    unsigned char* b_tiles = smem + STAGES * A_BYTES;
    unsigned char* staging = b_tiles + STAGES * B_BYTES;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(staging + STAGING);
    unsigned long long* empty = full + STAGES;
    unsigned long long* acc_full = empty + STAGES;                 // [2]
    unsigned long long* acc_empty = acc_full + 2;                  // [2]
    unsigned* tmem_holder = reinterpret_cast<unsigned*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (a.K + BK - 1) / BK;
    const int tiles = a.m_tiles * a.n_tiles;
    const unsigned rank = PAIR ? cluster_rank() : 0u;                  // 0: the block that issues the pair's instructions
    const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr unsigned TMEM_COLS = 2 * BN <= 32 ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + b, 1);
            mbar_init(acc_empty + b, PAIR ? 8 : 4);   // one arrival per epilogue warp (of both blocks of a pair)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                      // one warp allocates the accumulators' tensor memory (of a pair: the same warp of both blocks)
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync();             // the partner's barriers are initialised before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            unsigned it = 0, first_in_flight = 0;
            bool ok = true;
            for (int t = walker; t < tiles && ok; t += walkers) {
                const int m0 = (t % a.m_tiles) * TILE_M + (int)rank * BM, n0 = (t / a.m_tiles) * (ACT ? BN / 2 : BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const unsigned s = it % STAGES;
                    ok = mbar_wait(empty + s, ((it / STAGES) & 1) ^ 1, abort_flag, 1) && !*abort_flag;
                    if (!ok) break;
                    if (PAIR) {
                        // both blocks' bytes are counted on the first block's barrier, which that block arms
                        const unsigned bar = map_to_cta(smem_u32(full + s), 0);
                        if (rank == 0) mbar_expect_tx(full + s, 2 * (A_BYTES + B_BYTES));
                        tma_load_2d_pair(a_tiles + s * A_BYTES, &map_x, kb * BK, m0, bar);
                        // this block's half of the tile's rows of W (a box of map_w has BN/2 rows); with ACT the first
                        // block's half is the gate rows n0.., the second's the up rows of the same outputs
                        tma_load_2d_pair(b_tiles + s * B_BYTES, &map_w, kb * BK, ACT ? (int)rank * a.inter + n0 : n0 + (int)rank * (BN / 2), bar);
                        continue;
                    }
                    mbar_expect_tx(full + s, A_BYTES + B_BYTES);
                    tma_load_2d(a_tiles + s * A_BYTES, &map_x, kb * BK, m0, full + s);
                    if (ACT) {
                        // gate rows n0.., then the up rows of the same outputs (a box of map_w has BN/2 rows)
                        tma_load_2d(b_tiles + s * B_BYTES, &map_w, kb * BK, n0, full + s);
                        tma_load_2d(b_tiles + s * B_BYTES + B_BYTES / 2, &map_w, kb * BK, a.inter + n0, full + s);
                    } else {
                        tma_load_2d(b_tiles + s * B_BYTES, &map_w, kb * BK, n0, full + s);
                    }
                }
            }
            if (!ok) {
                // gave up somewhere: let the copies that may still be in flight land before the block exits (the
                // second block of a pair has no barrier of its own to watch: it sleeps for far longer than a copy takes)
                first_in_flight = it > STAGES ? it - STAGES : 0;
                if (PAIR && rank != 0) {
                    for (int i = 0; i < 200; ++i) __nanosleep(5000);
                } else {
                    for (unsigned j = first_in_flight; j < it; ++j)
                        for (unsigned i = 0; i < WAIT_LIMIT && !mbar_try_wait(full + j % STAGES, (j / STAGES) & 1); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            constexpr unsigned idesc = umma_idesc(TILE_M, BN);
            unsigned it = 0;
            bool ok = true;
            int i = 0;
            for (int t = walker; t < tiles && ok; t += walkers, ++i) {
                const int b = i & 1;
                ok = mbar_wait(acc_empty + b, ((i >> 1) & 1) ^ 1, abort_flag, 4);   // the epilogue has drained this buffer
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)(b * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const unsigned s = it % STAGES;
                    ok = mbar_wait(full + s, (it / STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long da = umma_desc(a_tiles + s * A_BYTES);
                    const unsigned long long db = umma_desc(b_tiles + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // the next 16 k values lie 32 bytes further inside the swizzled rows: +2 in the address field
                        if (PAIR) umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    // the stage is free (in both blocks of a pair) once these instructions have read it
                    if (PAIR) umma_commit_pair(empty + s); else umma_commit(empty + s);
                }
                // all of the tile's instructions done: the accumulator is complete (in both blocks of a pair)
                if (PAIR) umma_commit_pair(acc_full + b); else umma_commit(acc_full + b);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;             // the TMEM lanes this warp may read: 32 * (warp % 4) ...
        constexpr int COLS = 128 / (int)sizeof(O);    // output columns per 128-byte staging row
        unsigned char* my_staging = staging + quarter * 2 * 4096;
        int i = 0, piece = 0;
        bool ok = true;
        const unsigned acc_empty_first = PAIR ? map_to_cta(smem_u32(acc_empty), 0) : 0u;     // the first block's barriers
        for (int t = walker; t < tiles && ok; t += walkers, ++i) {
            constexpr int OUT_COLS = ACT ? BN / 2 : BN;        // output columns of a tile
            const int m0 = (t % a.m_tiles) * TILE_M + (int)rank * BM, n0 = (t / a.m_tiles) * OUT_COLS;
            const int n_limit = ACT ? a.inter : a.N;
            const int b = i & 1;
            ok = mbar_wait(acc_full + b, (i >> 1) & 1, abort_flag, 3);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            const unsigned tmem_row = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(b * BN);
#pragma unroll 1
            for (int c = 0; c < OUT_COLS; c += COLS) {
                unsigned char* buf = my_staging + (piece & 1) * 4096;
                if (TMA_STORE) {
                    // the store that last used this buffer (two pieces ago) must have read it
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                }
#pragma unroll
                for (int half = 0; half < COLS / 32; ++half) {
                    unsigned v[32];
                    tmem_ld_32x32(tmem_row + (unsigned)(c + half * 32), v);
                    if (ACT) {
                        unsigned up[32];
                        tmem_ld_32x32(tmem_row + (unsigned)(BN / 2 + c + half * 32), up);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j])));
                            const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(up[j])));
                            v[j] = __float_as_uint(silu_mul_bf16(g, u));
                        }
                    } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    }
                    if (c + COLS >= OUT_COLS && half == COLS / 32 - 1) {
                        // the tile has left tensor memory: hand the buffer back to the MMA warp
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            if (PAIR) mbar_arrive_cluster(acc_empty_first + (unsigned)(b * 8));
                            else mbar_arrive(acc_empty + b);
                        }
                    }
                    if (TMA_STORE) {
                        // row `lane` of the piece; its 16-byte chunk q goes to position q ^ (lane % 8): the 128-byte swizzle
                        if (sizeof(O) == 4) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                *reinterpret_cast<uint4*>(buf + lane * 128 + ((q ^ (lane & 7)) << 4)) =
                                    make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint4 pk;
                                unsigned* pw = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * e]), __uint_as_float(v[8 * q + 2 * e + 1]));
                                    pw[e] = *reinterpret_cast<unsigned*>(&h);
                                }
                                *reinterpret_cast<uint4*>(buf + lane * 128 + (((half * 4 + q) ^ (lane & 7)) << 4)) = pk;
                            }
                        }
                    } else {
                        const int col = n0 + c + half * 32;
                        if (row < a.M && col < n_limit) {
                            O* dst = reinterpret_cast<O*>(a.out) + (size_t)row * a.ldo + col;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < n_limit) dst[j] = from_f32<O>(__uint_as_float(v[j]));
                        }
                    }
                }
                if (TMA_STORE) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the generic-proxy writes above, seen by the TMA
                    __syncwarp();
                    if (lane == 0) {
                        // rows or columns of the piece that lie outside the matrix are clipped by the TMA
                        if (m0 + quarter * 32 < a.M && n0 + c < n_limit) tma_store_2d(&map_o, buf, n0 + c, m0 + quarter * 32);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    ++piece;
                }
            }
        }
        if (TMA_STORE && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // a pair leaves together: no instruction of the first block still reads the second's shared memory or writes its
    // tensor memory, and no arrive is on its way to a block that has gone
    if (PAIR) cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

template <int BN, int STAGES, typename O, bool TMA_STORE, bool ACT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_o, TcArgs a) {
    gemm_tc_body<BN, STAGES, O, TMA_STORE, ACT, false>(map_x, map_w, map_o, a);
}

template <int BN, int STAGES, typename O, bool TMA_STORE, bool ACT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_o, TcArgs a) {
    gemm_tc_body<BN, STAGES, O, TMA_STORE, ACT, true>(map_x, map_w, map_o, a);
}

template <int BN, int STAGES, typename O, bool TMA_STORE, bool ACT, bool PAIR>
int launch_kernel(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const TcArgs& a, cudaStream_t s) {
    constexpr size_t smem = 1024 + (size_t)STAGES * (BM + (PAIR ? BN / 2 : BN)) * BK * 2 + (TMA_STORE ? 4 * 2 * 4096 : 0) + (2 * STAGES + 4) * 8 + 16;
    static_assert(smem <= 232448, "the block's shared memory must fit an SM");
    auto kernel = PAIR ? gemm_tc_pair_kernel<BN, STAGES, O, TMA_STORE, ACT> : gemm_tc_kernel<BN, STAGES, O, TMA_STORE, ACT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLME_REFUSE("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int tiles = a.m_tiles * a.n_tiles;
    int walkers = PAIR ? sm_count() / 2 : sm_count();                     // blocks, or pairs of blocks
    if (PAIR) {
        // The two blocks of a pair need two free SMs of one GPC: a GPU may hold fewer pairs than half its SMs.  A pair
        // that had to wait for another to finish would double the kernel's time, so there are never more than fit.
        static int held = 0;
        if (!held) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * 1024, 1, 1);
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = smem;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = walkers; }
            held = n;
        }
        if (held < walkers) walkers = held;
    }
    const int grid = (tiles < walkers ? tiles : walkers) * (PAIR ? 2 : 1);
    kernel<<<grid, THREADS, smem, s>>>(mx, mw, mo, a);
    LLME_LAUNCH_STATUS();
}

// PAIR: tiles of 256 rows, a box of W has BN/2 rows (one block's half)
template <int BN, int STAGES, typename O, bool PAIR>
int launch(const void* x, long long ldx, const void* w, long long ldw, TcArgs a, cudaStream_t s) {
    alignas(64) CUtensorMap mx, mw, mo;
    if (int rc = make_map(&mx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.M, a.K, ldx, BM, BK)) return rc;
    if (int rc = make_map(&mw, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.N, a.K, ldw, PAIR ? BN / 2 : BN, BK)) return rc;
    a.m_tiles = (a.M + (PAIR ? 2 : 1) * BM - 1) / ((PAIR ? 2 : 1) * BM);
    a.n_tiles = (a.N + BN - 1) / BN;
    // a TMA store needs a 16-byte aligned base and row stride
    const bool tma_store = ((uintptr_t)a.out % 16 == 0) && ((a.ldo * (long long)sizeof(O)) % 16 == 0);
    if (tma_store) {
        const CUtensorMapDataType t = sizeof(O) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        if (int rc = make_map(&mo, a.out, t, (int)sizeof(O), a.M, a.N, a.ldo, 32, 128 / (int)sizeof(O))) return rc;
        return launch_kernel<BN, STAGES, O, true, false, PAIR>(mx, mw, mo, a, s);
    }
    mo = mx;
    return launch_kernel<BN, STAGES, O, false, false, PAIR>(mx, mw, mo, a, s);
}

// out[M, inter] = silu(x Wg^T) * (x Wu^T), W = [Wg | Wu]: tiles of BN/2 outputs, boxes of BN/2 rows of W.
template <int BN, int STAGES, typename O, bool PAIR>
int launch_act(const void* x, long long ldx, const void* w, long long ldw, TcArgs a, cudaStream_t s) {
    alignas(64) CUtensorMap mx, mw, mo;
    if (int rc = make_map(&mx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.M, a.K, ldx, BM, BK)) return rc;
    if (int rc = make_map(&mw, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.N, a.K, ldw, BN / 2, BK)) return rc;
    a.m_tiles = (a.M + (PAIR ? 2 : 1) * BM - 1) / ((PAIR ? 2 : 1) * BM);
    a.n_tiles = (a.inter + BN / 2 - 1) / (BN / 2);
    const CUtensorMapDataType t = sizeof(O) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (int rc = make_map(&mo, a.out, t, (int)sizeof(O), a.M, a.inter, a.ldo, 32, 128 / (int)sizeof(O))) return rc;
    return launch_kernel<BN, STAGES, O, true, true, PAIR>(mx, mw, mo, a, s);
}

// Pairs of blocks pay from two 128-row tiles of tokens on, and need a W wide enough for 256-column tiles.
bool use_pairs(int M, int N, int how) { return how == 2 || (how == 0 && M > BM && N > 128); }

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
    TcArgs a{out, ldo, M, N, K, 0, 0, 0};
    const bool pairs = use_pairs(M, N, g_pairing);
    if (out_dtype == LLME_F32) {
        if (pairs) return launch<256, 6, float, true>(x, ldx, w, ldw, a, stream);
        return N > 128 ? launch<256, 4, float, false>(x, ldx, w, ldw, a, stream) : launch<128, 6, float, false>(x, ldx, w, ldw, a, stream);
    }
    if (out_dtype == LLME_BF16) {
        if (pairs) return launch<256, 6, bf16, true>(x, ldx, w, ldw, a, stream);
        return N > 128 ? launch<256, 4, bf16, false>(x, ldx, w, ldw, a, stream) : launch<128, 6, bf16, false>(x, ldx, w, ldw, a, stream);
    }
    LLME_REFUSE("gemm_tc: unsupported output dtype %d", out_dtype);
}

// 0: pairs of blocks (tcgen05 with .cta_group::2) where they pay; 1: never; 2: always.  For tests and measurements.
LLME_API int llme_gemm_tc_pairing(int how) {
    if (how >= 0 && how <= 2) g_pairing = how;
    return g_pairing;
}

// 1 if llme_gemm_tc_swiglu_bf16 takes this problem (the output is written with TMA stores: 16-byte aligned rows).
LLME_API int llme_gemm_tc_swiglu_supports(int M, int inter, int K, long long ldx, long long ldw, long long ldo) {
    return M >= 1 && inter >= 8 && inter <= (1 << 29) && K >= 8 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldo >= inter && ldo % 8 == 0;
}

// out[M, inter] (bfloat16) = silu(x Wg^T) * (x Wu^T) with W = [Wg | Wu] stacked by rows ([2 * inter, K]).
LLME_API int llme_gemm_tc_swiglu_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
                                      int M, int inter, int K, cudaStream_t stream) {
    if (M <= 0 || inter <= 0) return 0;
    if (!x || !w || !out) LLME_REFUSE("gemm_tc: null pointer");
    if (!llme_gemm_tc_swiglu_supports(M, inter, K, ldx, ldw, ldo)) LLME_REFUSE("gemm_tc: M=%d inter=%d K=%d ldx=%lld ldw=%lld ldo=%lld is not supported (K and strides must be multiples of 8)", M, inter, K, ldx, ldw, ldo);
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) % 16) LLME_REFUSE("gemm_tc: operands and output must be 16-byte aligned");
    TcArgs a{out, ldo, M, 2 * inter, K, 0, 0, inter};
    if (use_pairs(M, 2 * inter, g_pairing)) return launch_act<256, 6, bf16, true>(x, ldx, w, ldw, a, stream);
    return launch_act<256, 4, bf16, false>(x, ldx, w, ldw, a, stream);
}

// Reads and clears the error flag of the kernels (synchronises the device).  0 = no wait ever gave up.
LLME_API int llme_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
