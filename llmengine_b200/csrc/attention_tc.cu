// Paged causal attention for prompt portions on the tcgen05 tensor cores of sm_100a (bfloat16, head size
// HEAD_DIM = 64 or 128, compiled per head size like attention_fast.cu).
//
// A block serves one request, one key/value head and 256 rows, a row being a (token, query head of the
// group) pair: two Q tiles of 128 rows that share every key/value tile the block loads.  Keys and values
// stream through shared memory 128 at a time:
//
//   warp 0      producer: TMA loads of the Q tiles (3-D boxes: tokens x heads of the group x 64 columns) and,
//               page by page through the block table, of the K and V tiles (128-byte swizzle, two stages
//               each, one load per lane, the keys one tile ahead of the values).  A page that holds keys
//               beyond what the block may see is copied by hand instead, with those rows zeroed, so that
//               stale memory (NaN included) never reaches the tensor cores.
//   warp 1      issues the matrix instructions, alternating between the two Q tiles so that the tensor pipe
//               works for one while the softmax of the other runs: S_t = Q_t K^T (128 x 128 x HEAD_DIM) into
//               the tile's score columns of tensor memory, and O_t += P_t V (128 x HEAD_DIM x 128) into its
//               output accumulator, also in tensor memory.  P_t is read from tensor memory (it replaces
//               the scores it was made from); V is read as an MN-major operand, exactly as it lies in the cache.
//               One round is: wait for V(i) | K(i+1) (one barrier) and for P_t(i), sixteen instructions
//               (O_t(i), then S_t(i+1)), commits.  The pipe holds very few instructions in advance, and an
//               access of this thread to a barrier in shared memory takes 100 to 160 cycles while the pipe
//               reads its operands from there: what the thread does between two instructions is time the pipe
//               stands idle, so waits and commits are few and lie where products are in flight.
//   warps 2..17 softmax, eight warps per Q tile: two threads per row, 64 keys of the tile each (a warp may
//               only touch the 32 lanes of tensor memory given by its index modulo 4).  Each reads its
//               scores once, takes the probabilities relative to the row's reference maximum of the tile
//               before and tells its partner its half's maximum (shared memory, a 64-thread named
//               barrier); only if the row's maximum has grown by more than 2^8 does the reference move,
//               the accumulator get rescaled and the scores get read again.  Sums are 32-bit; the
//               probabilities go back into tensor memory as bfloat16 pairs (tcgen05.st) over the thread's
//               own scores.
//
// Every mbarrier wait is bounded; a wait that gives up sets an error flag (read with
// llme_attention_tc_status()), and the block drains its copies, frees its tensor memory and returns.  A warp
// that has given up still attends every named barrier of its pair.
//
// Measured (2,048-token prompt, 32 query and 8 key/value heads of 128, B200): 53 us with pages of 64 tokens, 57 us
// with pages of 16 (the SM clock is about 1.62 GHz while it runs; a round of sixteen instructions then needs 0.71 us
// of the pipe, the thread's bookkeeping 0.2 to 0.3 us more, and a tile's softmax about 1 us, of which 0.6 us are its
// 8,192 exponentials on the two warps a scheduler has of it).  Storing the output straight from the threads that
// hold it (16 bytes a lane, every lane another row) cost 1.4 us a block, 3 to 4 us of the launch; through shared
// memory it is whole rows.  With O_t(i) and S_t(i+1) as separate rounds of eight, each with waits and commits of its
// own: 62.7 us.  One Q tile per block with P in shared memory took 71 us.  A second issuing warp (one per Q tile)
// made it slower (66.8 us).  One softmax thread a row (four warps a Q tile, nothing exchanged between threads, the
// next 32 scores on their way from tensor memory while 32 are worked on): 56.3 us; a thread's 128 exponentials
// in a row leave the two warps a scheduler then has too little to overlap.  Every fourth exponential as a cubic on the
// FMA units (range reduction through the exponent bits, relative error 1e-4) instead of the special-function unit:
// 56.6 us; the softmax warps are short of issue slots, not of exponentials.
//
// Also tried and dropped, each correct and each slower (62 to 65 us): one block per SM that walks a list of
// 128-row items (queries and probabilities in tensor memory, four threads a row, the scores one or two key tiles
// ahead of the outputs, separate loader warps for keys and values, the items of a block decoded at once during
// set-up).  It removes the 5 us a block spends before its first and after its last tile, but a key tile of
// 128 x 128 took it 1.40 to 1.45 us whatever ran ahead: the thread that issues the matrix instructions and the
// softmax warps were each busy for that long.  Sixteen instructions keep the issuing thread for 0.8 to 0.9 us (the
// pipe takes few in advance, so their issue runs at the pipe's pace), its waits and commits for 0.5 us more, during
// which the pipe drains; a tile's softmax took 0.85 us of exponentials plus 0.4 us to hand the probabilities over.
// Two Q tiles that share every key tile, as here, pay those once for 256 rows.
//
// Reference counterpart: flash_sdpa_tiled_kernel (src/runtime/kernels/cuda_kernels.cu:558-645): one block per
// query row, scalar FMA, keys of the same launch only.
#include <cuda.h>

#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or -DHEAD_DIM=128"
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "HEAD_DIM must be 64 or 128");

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int HD = HEAD_DIM;
constexpr int HALVES = HD / 64;        // 64-column (128-byte) halves of a row
constexpr int BM = 128;                // rows per Q tile
constexpr int QT = 2;                  // Q tiles per block: they share every key/value tile the block loads
constexpr int BN = 128;                // keys per tile
constexpr int BOX_ROWS = 32;           // most keys one TMA load brings; a tile's loads are started by as many lanes
constexpr int THREADS = 32 * (2 + 8 * QT);   // producer, matrix warp, eight softmax warps per Q tile
constexpr int HALF_BYTES = 128 * 128;  // a [128 rows x 64 columns] bfloat16 tile with 128-byte rows
constexpr int TILE_BYTES = HALVES * HALF_BYTES;
constexpr unsigned WAIT_LIMIT = 1u << 20;
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_status = 0;

struct TcAttnArgs {
    bf16* out;                   // [T, nh, HD]
    const bf16* cache;           // [pages][K|V][nkv][page_size][HD]
    const int* rows;             // [n_rows] batch rows (requests) this launch serves
    const int* cu_q_lens;        // [R+1]
    const int* ctx_lens;         // [R] cached length after this step
    const int* table_rows;       // [R] row of block_tables of each request
    const int* block_tables;     // [*, max_blocks]
    int max_blocks, n_rows, nh, nkv, page_size, window;
    float scale;
};
#include "kernel_args.h"
static_assert(sizeof(TcAttnArgs) == sizeof(LlmeTcAttnArgs), "the argument block must match kernel_args.h");

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = where;
    atomicCAS(&g_status, 0, where);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

// K-major operand with 128-byte rows and the 128-byte swizzle (Q, K, P): eight rows form a 1024-byte group.
__device__ __forceinline__ unsigned long long desc_k_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFFu) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// MN-major operand (V as it lies in the cache: one key per 128-byte row, 64 columns of the head per row):
// the 64-column chunks of the N side lie HALF_BYTES apart (leading byte offset), groups of eight keys
// 1024 bytes apart (stride byte offset).
__device__ __forceinline__ unsigned long long desc_mn_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFFu) >> 4);
    d |= (unsigned long long)(HALF_BYTES >> 4) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: D = F32, A = B = BF16, A K-major, B K-major (b_mn = 0) or MN-major (1).
__host__ __device__ constexpr unsigned idesc(int M, int N, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_mn << 16) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}
// The matrix instructions of one group, in one piece of assembly: between two of them nothing but the two
// additions that move the descriptors on by 16 k values (the issuing thread is alone on its path: every extra
// instruction of its dependent chain holds both Q tiles up).
// S = Q K^T over 64 columns of the head (four steps of 16): descriptors + 2 per step (32 bytes inside the swizzled rows).
template <bool FIRST_NEW>
__device__ __forceinline__ void umma_qk_half(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned id) {
    asm volatile(
        "{\n\t.reg .pred pn, pa;\n\t.reg .b64 a, b;\n\t"
        "setp.eq.u32 pn, 1, %4;\n\t"
        "setp.eq.u32 pa, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pn;\n\t"
        "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pa;\n\t"
        "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pa;\n\t"
        "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pa;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "n"(FIRST_NEW ? 0 : 1) : "memory");
}
// O (+)= P V over 64 keys (four steps of 16): P in tensor memory, 8 columns per step; V MN-major, two 1024-byte
// groups (+ 128 in the descriptor) per step.  `acc_first`: whether the first step adds to what O holds.
__device__ __forceinline__ void umma_pv_half(unsigned tmem_d, unsigned tmem_p, unsigned long long dv, unsigned id, unsigned acc_first) {
    asm volatile(
        "{\n\t.reg .pred pf, pa;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
        "setp.ne.b32 pf, %4, 0;\n\t"
        "setp.eq.u32 pa, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
        "add.u32 a, %1, 8;\n\tadd.u64 b, %2, 128;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pa;\n\t"
        "add.u32 a, %1, 16;\n\tadd.u64 b, %2, 256;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pa;\n\t"
        "add.u32 a, %1, 24;\n\tadd.u64 b, %2, 384;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pa;\n\t}"
        ::"r"(tmem_d), "r"(tmem_p), "l"(dv), "r"(id), "r"(acc_first) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned addr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(unsigned addr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr),
          "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32u(unsigned addr, const unsigned (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr),
          "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Barriers {
    // kv_full / kv_empty [i % 2]: the values of key tile i together with the keys of tile i + 1, which the
    // matrix warp takes in one go; the keys of the first tile have a barrier pair of their own
    unsigned long long q_full, k0_full, k0_empty, kv_full[2], kv_empty[2];
    unsigned long long s_full[QT], p_full[QT], o_full;
    unsigned tmem_base;
    int abort_flag;
    float row_sum[QT][2][BM];     // the two halves' sums of a row, at the end
    float row_max[QT][2][2][BM];  // [Q tile][tile parity][half][row]: the halves' maxima of a key tile
};

__global__ void __launch_bounds__(THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, TcAttnArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tiles = smem;                             // QT x HALVES x [128 rows x 128 B]
    unsigned char* k_tiles = q_tiles + QT * TILE_BYTES;        // 2 stages
    unsigned char* v_tiles = k_tiles + 2 * TILE_BYTES;         // 2 stages
    Barriers* bar = reinterpret_cast<Barriers*>(v_tiles + 2 * TILE_BYTES);
    volatile int* abort_flag = &bar->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = a.rows[blockIdx.z];
    // blockIdx.x = pair * nkv + head: the blocks with the most keys, of all heads, start first
    const int kvh = (int)(blockIdx.x % (unsigned)a.nkv), pair_index = (int)(blockIdx.x / (unsigned)a.nkv);
    const int G = a.nh / a.nkv;
    const int q0 = a.cu_q_lens[r];
    const int q_len = a.cu_q_lens[r + 1] - q0;
    const int M = q_len * G;
    const int m0 = ((M + QT * BM - 1) / (QT * BM) - 1 - pair_index) * (QT * BM);    // first row of the block's first Q tile
    if (m0 < 0) return;
    const int n_q = m0 + BM < M ? QT : 1;                             // Q tiles of this block that hold rows
    const int start = a.ctx_lens[r] - q_len;
    const int* bt = a.block_tables + (size_t)a.table_rows[r] * a.max_blocks;
    const int ps = a.page_size;
    const int t_lo = m0 / G, t_hi = min(q_len - 1, (m0 + n_q * BM - 1) / G);
    const int hi_max = start + t_hi;                                  // last key any row of the block sees
    const int lo_min = a.window > 0 ? max(0, start + t_lo - a.window + 1) : 0;
    const int tile_first = lo_min / BN, tile_last = hi_max / BN;
    const int n_tiles = tile_last - tile_first + 1;

    if (threadIdx.x == 0) {
        mbar_init(&bar->q_full, 1);
        mbar_init(&bar->k0_full, 1);
        mbar_init(&bar->k0_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bar->kv_full[s], 2);         // the load of the values and the load of the keys
            mbar_init(&bar->kv_empty[s], 1);
        }
        for (int t = 0; t < QT; ++t) {
            mbar_init(&bar->s_full[t], 1);
            mbar_init(&bar->p_full[t], 8);          // the eight softmax warps of a Q tile
        }
        mbar_init(&bar->o_full, 1);
        bar->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the value tiles start as zeros: rows that are never loaded (before a window, past the last key) must not be NaN
    for (int i = threadIdx.x; i < 2 * TILE_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(v_tiles)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = bar->tmem_base;
    // columns: S of Q tile 0, S of Q tile 1, O of Q tile 0, O of Q tile 1
    const unsigned tmem_s[QT] = {tmem, tmem + 128};
    const unsigned tmem_o[QT] = {tmem + 256, tmem + 384};

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            mbar_expect_tx(&bar->q_full, (unsigned)(n_q * TILE_BYTES));
            for (int t = 0; t < n_q; ++t)
                for (int h = 0; h < HALVES; ++h)
                    tma_load_3d(q_tiles + t * TILE_BYTES + h * HALF_BYTES, &map_q, h * 64, kvh * G, q0 + (m0 + t * BM) / G, &bar->q_full);
        }
        // Rows one TMA load of the cache brings: a power of two (pages of 8..32 tokens, or 32 rows of a larger
        // page).  A lane looks after one TMA load of a tile (box lane / HALVES, 64-column half lane % HALVES): it
        // looks up the box's page (two tiles ahead of its use, so that the look-up's latency is not in front of
        // the copies), and decides whether the box is needed whole (a TMA load), in part (copied by hand), or
        // not at all.  No division in the loop: the producer's instructions are a dependent chain, and nothing
        // hides their latency.
        const int rows_per_box = ps < BOX_ROWS ? ps : BOX_ROWS;
        const int box_shift = __ffs(rows_per_box) - 1;
        const int n_boxes = BN >> box_shift;
        const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
        constexpr int H_SHIFT = HALVES == 2 ? 1 : 0;
        const unsigned load_bytes = (unsigned)(rows_per_box * 128);     // one TMA load: a box of one 64-column half
        const int my_box = lane >> H_SHIFT, my_half = lane & (HALVES - 1);
        const long long head_rows = (long long)kvh * ps;                 // row of this head within a page's K (or V) block
        const long long page_rows = (long long)2 * a.nkv * ps, v_rows = (long long)a.nkv * ps;
        bool ok = true;
        auto first_row = [&](int i) -> long long {                       // cache row of this lane's box in tile i (its K rows), or -1
            const int ja = (tile_first + i) * BN + (my_box << box_shift);
            if (i >= n_tiles || my_box >= n_boxes || ja + rows_per_box - 1 < lo_min || ja > hi_max) return -1;
            const int blk = ps_shift >= 0 ? ja >> ps_shift : ja / ps;
            return (long long)bt[blk] * page_rows + head_rows + (ja - blk * ps);
        };
        // One load of a tile: its keys (which = 0) or its values (1), into the stage i % 2; `full` counts its bytes,
        // `empty` (if any) with `empty_parity` says when the stage may be overwritten.
        auto load_tile = [&](int i, int which, long long my_row, unsigned long long* full, unsigned long long* empty, unsigned empty_parity) {
            const int j0 = (tile_first + i) * BN;
            const int ja = j0 + (my_box << box_shift), jb = ja + rows_per_box - 1;
            const bool whole = my_row >= 0 && ja >= lo_min && jb <= hi_max;
            const unsigned whole_mask = __ballot_sync(0xffffffffu, whole);                 // one bit per TMA load
            const unsigned part_mask = __ballot_sync(0xffffffffu, my_row >= 0 && !whole && my_half == 0);
            const unsigned tx = (unsigned)__popc(whole_mask) * load_bytes;
            unsigned char* tile = (which ? v_tiles : k_tiles) + (i & 1) * TILE_BYTES;
            if (empty) ok = mbar_wait(empty, empty_parity, abort_flag, 10 + which);
            ok = ok && !*abort_flag;
            if (!ok) return;
            // First the boxes that straddle an edge of the visible range: they are copied by hand, visible
            // rows only, the rest zeroed.  Then, after those writes are published, one lane arms the barrier
            // and the lanes start the TMA loads of the boxes that are needed whole.
            if (part_mask) {
                for (unsigned rest = part_mask; rest; rest &= rest - 1) {
                    const int src_lane = __ffs(rest) - 1, b = (src_lane >> H_SHIFT) << box_shift;
                    const long long row0 = __shfl_sync(0xffffffffu, my_row, src_lane) + (which ? v_rows : 0);
                    for (int c = lane; c < rows_per_box * (HD / 8); c += 32) {
                        const int rr = c / (HD / 8), ch = c % (HD / 8);
                        const int j = j0 + b + rr;
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (j >= lo_min && j <= hi_max) v = *reinterpret_cast<const uint4*>(a.cache + (row0 + rr) * HD + ch * 8);
                        const int h = ch >> 3, q = ch & 7, row = b + rr;
                        *reinterpret_cast<uint4*>(tile + h * HALF_BYTES + row * 128 + ((q ^ (row & 7)) << 4)) = v;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) mbar_expect_tx(full, tx);
            __syncwarp();
            // every lane starts the load of its own box: issued from one thread, the many small boxes of
            // small pages went out one after the other and took longer than the arithmetic on them
            if (whole)
                tma_load_2d(tile + my_half * HALF_BYTES + (my_box << box_shift) * 128, &map_kv, my_half * 64,
                            (int)(my_row + (which ? v_rows : 0)), full);
            __syncwarp();
        };
        // The keys run one tile ahead of the values: the matrix warp takes V(i) and K(i+1) together (O += P V(i),
        // then S = Q K(i+1)^T), and gives both stages back together when tile i is done.
        long long row_cur = first_row(0), row_next = first_row(1);
        load_tile(0, 0, row_cur, &bar->k0_full, nullptr, 0u);
        for (int i = 0; i < n_tiles && ok; ++i) {
            const long long row_after = first_row(i + 2);
            unsigned long long* full = &bar->kv_full[i & 1];
            unsigned long long* empty = &bar->kv_empty[i & 1];
            const unsigned parity = ((unsigned)(i >> 1) & 1u) ^ 1u;          // passes at once while the stages are fresh
            // K(2) goes where K(0) lay, which no kv_empty speaks for
            if (i == 1) ok = mbar_wait(&bar->k0_empty, 0, abort_flag, 12);
            if (i + 1 < n_tiles) {
                if (ok) load_tile(i + 1, 0, row_next, full, empty, parity);
            } else if (lane == 0) {
                mbar_arrive(full);                                           // no keys behind the last tile
            }
            if (ok) load_tile(i, 1, row_cur, full, empty, parity);
            row_cur = row_next;
            row_next = row_after;
        }
        if (*abort_flag) {
            // gave up somewhere: give the copies that are still in flight time to land before the block exits
            for (int i = 0; i < 200; ++i) __nanosleep(5000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ matrix instructions
        // Per key tile i and Q tile t: S_t = Q_t K(i)^T, then, when the softmax warps of t have turned S_t into
        // P_t, O_t += P_t V(i).  The two Q tiles alternate, so that the tensor pipe works for one while the
        // softmax of the other runs: S_0(0) S_1(0) | O_0(0) S_0(1) O_1(0) S_1(1) | O_0(1) S_0(2) ...
        if (lane == 0) {
            constexpr unsigned id_s = idesc(BM, BN, 0);
            constexpr unsigned id_o = idesc(BM, HD, 1);
            bool ok = mbar_wait(&bar->q_full, 0, abort_flag, 20);
            // The one thread that issues the matrix instructions runs a dependent chain of its own: every
            // instruction it spends between two products delays both Q tiles (measured: 0.7 us per group of
            // eight products when the descriptors were built inside the loop, against 0.27 us that the tensor
            // pipe needs for them).  So the descriptors are built once, and a group is waits, eight
            // instructions and commits.
            unsigned long long dq[QT][HALVES], dk[2][HALVES], dv[2];
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
#pragma unroll
                for (int t = 0; t < QT; ++t) dq[t][h] = desc_k_major(q_tiles + t * TILE_BYTES + h * HALF_BYTES);
#pragma unroll
                for (int s = 0; s < 2; ++s) dk[s][h] = desc_k_major(k_tiles + s * TILE_BYTES + h * HALF_BYTES);
            }
#pragma unroll
            for (int s = 0; s < 2; ++s) dv[s] = desc_mn_major(v_tiles + s * TILE_BYTES);
            auto issue_first = [&](int t) {                           // S_t(0) = Q_t K(0)^T
                ok = ok && mbar_wait(&bar->k0_full, 0, abort_flag, 21);
                if (!ok) return;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned d = t == 0 ? tmem_s[0] : tmem_s[1];
                umma_qk_half<true>(d, t == 0 ? dq[0][0] : dq[QT - 1][0], dk[0][0], id_s);
                if (HALVES == 2) umma_qk_half<false>(d, t == 0 ? dq[0][HALVES - 1] : dq[QT - 1][HALVES - 1], dk[0][HALVES - 1], id_s);
                if (t == n_q - 1) umma_commit(&bar->k0_empty);        // both Q tiles have read K(0)
                umma_commit(&bar->s_full[t]);
            };
            // O_t(i) += P_t(i) V(i) and, straight behind it, S_t(i+1) = Q_t K(i+1)^T: every wait comes before the
            // sixteen instructions and every commit after them, so that the thread's own bookkeeping (which the
            // tensor pipe would otherwise stand idle for: it holds very few instructions in advance) overlaps
            // with the products it has just issued.
            auto issue_pair = [&](int t, int i) {
                const int s = i & 1, round = i >> 1;
                const bool more = i + 1 < n_tiles;
                const int s1 = s ^ 1;
                ok = ok && mbar_wait(&bar->kv_full[s], round & 1, abort_flag, 24);
                ok = ok && mbar_wait(&bar->p_full[t], i & 1, abort_flag, 23);
                if (!ok) return;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned d = t == 0 ? tmem_o[0] : tmem_o[1];
                const unsigned pa = t == 0 ? tmem_s[0] : tmem_s[1];
                const unsigned long long b0 = s == 0 ? dv[0] : dv[1];
                // P lies in tensor memory, over the scores it was made from: the probabilities of keys 0..63 in
                // columns 0..31 of S_t, those of keys 64..127 in columns 64..95
                umma_pv_half(d, pa, b0, id_o, i > 0 ? 1u : 0u);
                umma_pv_half(d, pa + 64u, b0 + 4ull * (2048 >> 4), id_o, 1u);
                if (more) {
                    // S_t is free again once the products above have read P_t(i); the pipe runs them in order
                    umma_qk_half<true>(pa, t == 0 ? dq[0][0] : dq[QT - 1][0], s1 == 0 ? dk[0][0] : dk[1][0], id_s);
                    if (HALVES == 2)
                        umma_qk_half<false>(pa, t == 0 ? dq[0][HALVES - 1] : dq[QT - 1][HALVES - 1], s1 == 0 ? dk[0][HALVES - 1] : dk[1][HALVES - 1], id_s);
                    umma_commit(&bar->s_full[t]);
                }
                if (t == n_q - 1) {
                    umma_commit(&bar->kv_empty[s]);                   // both Q tiles have read V(i) and K(i+1)
                    if (!more) umma_commit(&bar->o_full);             // the output accumulators are complete
                }
            };
            for (int t = 0; t < n_q && ok; ++t) issue_first(t);
            for (int i = 0; i < n_tiles && ok; ++i)
                for (int t = 0; t < n_q && ok; ++t) issue_pair(t, i);
        }
    } else {
        // ------------------------------------------------------------------ softmax and output
        // Warp w may touch the 32 lanes of tensor memory given by w % 4 (a quarter of a Q tile's rows); the four
        // warps with the same quarter serve (Q tile 0 | 1) x (first | second half of the columns).  The output
        // accumulator stays in tensor memory and is added to by the matrix warp tile after tile.  A row's
        // probabilities are taken relative to a reference maximum that is only moved when the true maximum has
        // grown by more than RESCALE (in base-2 units): the final division by the sum, taken relative to the
        // same reference, makes the result exact, and moving the reference means a round trip of the accumulator
        // through registers and a second reading of the scores, which then happens only in the first few tiles.
        constexpr float RESCALE = 8.0f;
        constexpr int BH = BN / 2;                           // keys of a tile per thread
        constexpr int OC = HD / 2;                           // columns of the output accumulator per thread
        const int quarter = warp & 3;
        const int role = (warp - 2) >> 2;                    // 0..3
        const int t = role >> 1, ch = role & 1;              // Q tile, half of the columns
        if (t < n_q) {
            const int row = quarter * 32 + lane;             // this thread's row of its Q tile
            const int mt0 = m0 + t * BM;
            const int m = mt0 + row;
            const bool row_ok = m < M;
            const int p = start + min(m, M - 1) / G;         // its position
            const int phi = row_ok ? p : -1;
            const int plo = a.window > 0 ? max(0, p - a.window + 1) : 0;
            const unsigned lane_off = (unsigned)(quarter * 32) << 16;
            const float sc = a.scale * LOG2E;
            // what every row of this warp sees entirely, without a mask
            const int warp_p_lo = start + min(q_len - 1, (mt0 + quarter * 32) / G);
            const int warp_p_hi = start + min(q_len - 1, (mt0 + quarter * 32 + 31) / G);
            const int warp_lo_last = a.window > 0 ? max(0, warp_p_hi - a.window + 1) : 0;
            const bool warp_full = mt0 + quarter * 32 + 31 < M;
            // the two warps of a (Q tile, quarter) meet at a named barrier of their own (64 threads)
            auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + t * 4 + quarter) : "memory"); };
            float m_ref = -INFINITY, l_run = 0.0f;
            bool ok = true;
            for (int i = 0; i < n_tiles; ++i) {
                const int j0 = (tile_first + i) * BN;
                unsigned pk[32];
                const int s2 = i & 1;
                ok = ok && mbar_wait(&bar->s_full[t], i & 1, abort_flag, 30);
                bool unmasked = false;
                float own_max = -INFINITY;
                const float ref_old = m_ref == -INFINITY ? 0.0f : m_ref;
                float sum = 0.0f;
                // This thread's 64 scores -> probabilities, their sum and their maximum.  The probabilities are taken
                // relative to the reference maximum of the tile before: it almost never has to move (only when the
                // row's maximum has grown by more than RESCALE), and then the scores are read a second time below.
                auto half_pass = [&](float ref, bool with_max) {
                    float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};          // four partial sums, added in a fixed order
                    float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int c0 = 0; c0 < BH; c0 += 32) {
                        float v[32];
                        tmem_ld32(tmem_s[t] + lane_off + (unsigned)(ch * BH + c0), v);
                        if (!unmasked) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) {
                                const int j = j0 + ch * BH + c0 + e;
                                if (j < plo || j > phi) v[e] = -INFINITY;
                            }
                        }
                        if (with_max) {
#pragma unroll
                            for (int e = 0; e < 32; e += 4) {
                                mq[0] = fmaxf(mq[0], v[e]); mq[1] = fmaxf(mq[1], v[e + 1]);
                                mq[2] = fmaxf(mq[2], v[e + 2]); mq[3] = fmaxf(mq[3], v[e + 3]);
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            const float e0 = fast_exp2(fmaf(v[e], sc, -ref));            // a masked score is -inf: exactly 0
                            const float e1 = fast_exp2(fmaf(v[e + 1], sc, -ref));
                            sq[(e >> 1) & 3] += e0 + e1;
                            __nv_bfloat162 hh = __floats2bfloat162_rn(e0, e1);
                            pk[(c0 + e) >> 1] = *reinterpret_cast<unsigned*>(&hh);
                        }
                    }
                    sum = (sq[0] + sq[1]) + (sq[2] + sq[3]);
                    if (with_max) own_max = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
                };
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unmasked = warp_full && j0 + BN - 1 <= warp_p_lo && j0 >= warp_lo_last;
                    half_pass(ref_old, true);
                }
                // the two threads of a row tell each other their half's maximum (every iteration comes to the pair's
                // named barrier exactly once, also after a wait has given up: the partner must never be left there)
                bar->row_max[t][s2][ch][row] = own_max;
                pair_sync();
                if (ok) {
                    const float m_true = fmaxf(own_max, bar->row_max[t][s2][ch ^ 1][row]) * sc;
                    const bool move = m_true > m_ref + RESCALE || (m_ref == -INFINITY && m_true > -INFINITY);
                    if (__any_sync(0xffffffffu, move)) {
                        // The reference maximum of some row of this warp moves.  Both threads of a row take the same
                        // decision; each rescales its half of the accumulator's columns (at rest once P V of the tile
                        // before has finished) and takes its probabilities again, relative to the new reference.
                        const float m_new = move ? m_true : m_ref;
                        const float ref = m_new == -INFINITY ? 0.0f : m_new;
                        if (i > 0) {
                            // The accumulator is at rest: O_t(i-1) was issued before S_t(i), the tensor pipe runs them
                            // in order, and s_full (waited for above) came when all of them had finished; O_t(i) waits
                            // for this warp's p_full.
                            const float corr = move ? fast_exp2(m_ref - ref) : 1.0f;
                            l_run *= corr;
#pragma unroll 1
                            for (int c = 0; c < OC; c += 32) {
                                float v[32];
                                tmem_ld32(tmem_o[t] + lane_off + (unsigned)(ch * OC + c), v);
#pragma unroll
                                for (int e = 0; e < 32; ++e) v[e] *= corr;
                                tmem_st32(tmem_o[t] + lane_off + (unsigned)(ch * OC + c), v);
                            }
                        } else if (move) {
                            l_run *= fast_exp2(m_ref - ref);         // first tile: nothing accumulated yet (and l_run is 0)
                        }
                        m_ref = m_new;
                        if (ok) half_pass(ref, false);
                    }
                }
                if (ok) {
                    l_run += sum;
                    // the probabilities replace the first 32 of this thread's own 64 scores in tensor memory, two
                    // bfloat16 values per word (the matrix warp reads them from there as its A operand); nobody
                    // else reads these columns
                    tmem_st32u(tmem_s[t] + lane_off + (unsigned)(ch * BH), pk);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar->p_full[t]);
                }
            }
            if (ok) ok = mbar_wait(&bar->o_full, 0, abort_flag, 33);
            // the row's sum over both halves
            bar->row_sum[t][ch][row] = l_run;
            pair_sync();
            l_run += bar->row_sum[t][ch ^ 1][row];
            // The output goes through shared memory, through the Q tile's place, which nothing reads any more: a
            // thread holds half of ONE row, and rows lie 2 x HEAD_DIM bytes apart in the output, so that a warp's
            // store of 16 bytes a lane would touch 32 lines (1.4 us for the block's 16 warps).  The 16-byte pieces
            // of a row are swizzled with the row, so that neither the writes (eight rows, the same piece) nor the
            // reads (one row, pieces in turn) meet in a bank; the two warps of a (Q tile, quarter) then write their
            // 32 rows out whole, two rows to a store.
            constexpr int ROW_PIECES = HD / 8;
            unsigned char* stage = q_tiles + t * TILE_BYTES;     // [BM rows][2 x HEAD_DIM bytes]
            const bool good = ok && !*abort_flag;
            if (good) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float inv = 1.0f / l_run;
#pragma unroll 1
                for (int c = 0; c < OC; c += 32) {
                    float v[32];
                    tmem_ld32(tmem_o[t] + lane_off + (unsigned)(ch * OC + c), v);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 pk;
                        unsigned* pw = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 hh = __floats2bfloat162_rn(v[q4 * 8 + 2 * e] * inv, v[q4 * 8 + 2 * e + 1] * inv);
                            pw[e] = *reinterpret_cast<unsigned*>(&hh);
                        }
                        const int piece = (ch * OC + c) / 8 + q4;
                        *reinterpret_cast<uint4*>(stage + row * (HD * 2) + ((piece ^ (row & 7)) << 4)) = pk;
                    }
                }
            }
            pair_sync();
            if (good) {
                const int tid = ch * 32 + lane;                  // 0..63 among the two warps
#pragma unroll 4
                for (int k = 0; k < 32 * ROW_PIECES / 64; ++k) {
                    const int idx = k * 64 + tid;
                    const int r = quarter * 32 + idx / ROW_PIECES, piece = idx % ROW_PIECES;
                    const int mm = mt0 + r;
                    if (mm < M) {
                        const uint4 v = *reinterpret_cast<const uint4*>(stage + r * (HD * 2) + ((piece ^ (r & 7)) << 4));
                        *reinterpret_cast<uint4*>(a.out + ((size_t)(q0 + mm / G) * a.nh + kvh * G + mm % G) * HD + piece * 8) = v;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
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

constexpr size_t SMEM_BYTES = 1024 + (size_t)(QT + 4) * TILE_BYTES + sizeof(Barriers) + 64;
static_assert(SMEM_BYTES <= 232448, "the block's shared memory must fit an SM");

}  // namespace

LLME_API int llme_attention_tc_head_dim() { return HD; }

// Whether this kernel takes the problem: a page size that divides 128 and is at least 8 (a TMA box of whole
// pages with whole swizzle groups), and a group size (query heads per key/value head) that divides 128.
LLME_API int llme_attention_tc_supports(int nh, int nkv, int page_size) {
    if (nkv <= 0 || nh % nkv) return 0;
    const int G = nh / nkv;
    return page_size >= 8 && (page_size <= 128 ? 128 % page_size == 0 : page_size % 128 == 0) && 128 % G == 0 && G <= 128;
}

// q, out [T, nh, HD] bfloat16 (q_tokens = T rows in all); the other arguments as for the portion kernel of
// attention_fast.cu.  total_cache_rows = pages * 2 * nkv * page_size.
LLME_API int llme_attention_tc(const void* q, long long q_tokens, long long total_cache_rows, const TcAttnArgs* args,
                               int max_q_len, cudaStream_t stream) {
    const TcAttnArgs& a = *args;
    if (a.n_rows <= 0 || max_q_len <= 0) return 0;
    if (!q || !a.out || !a.cache || !a.rows || !a.cu_q_lens || !a.ctx_lens || !a.table_rows || !a.block_tables)
        LLME_REFUSE("attention_tc: null pointer");
    if (!llme_attention_tc_supports(a.nh, a.nkv, a.page_size)) LLME_REFUSE("attention_tc: %d/%d heads with pages of %d are not supported", a.nh, a.nkv, a.page_size);
    if (a.n_rows > 65535) LLME_REFUSE("attention_tc: grid too large");
    EncodeTiledFn enc = encode_fn();
    if (!enc) LLME_REFUSE("attention_tc: cuTensorMapEncodeTiled is not available in this driver");
    const int G = a.nh / a.nkv;
    alignas(64) CUtensorMap mq, mkv;
    {   // q as [token][head][column]; a box is 128/G tokens x G heads x 64 columns = 128 rows of 128 bytes
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)a.nh, (cuuint64_t)q_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)a.nh * HD * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(BM / G)};
        cuuint32_t es[3] = {1, 1, 1};
        CUresult r = enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) LLME_REFUSE("attention_tc: cuTensorMapEncodeTiled (q) failed with code %d", (int)r);
    }
    {   // the cache as rows of HD columns; a box is one page (or 128 rows of a larger page) x 64 columns
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)total_cache_rows};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)(a.page_size < BOX_ROWS ? a.page_size : BOX_ROWS)};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(&mkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(a.cache), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) LLME_REFUSE("attention_tc: cuTensorMapEncodeTiled (cache) failed with code %d", (int)r);
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) LLME_REFUSE("attention_tc: cannot reserve %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    const long long tiles = ((long long)max_q_len * G + QT * BM - 1) / (QT * BM);
    if (tiles * a.nkv > 2147483647LL) LLME_REFUSE("attention_tc: grid too large");
    dim3 grid((unsigned)(tiles * a.nkv), 1, a.n_rows);
    attention_tc_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(mq, mkv, a);
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_attention_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
