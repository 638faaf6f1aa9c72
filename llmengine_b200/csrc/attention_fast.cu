// Paged attention on the tensor cores for bfloat16 queries and caches, compiled for one head
// size (HEAD_DIM, a multiple of 16 up to 128, given on the nvcc command line).
//
//   attention_portion_kernel  prompt portions of any length at any start position: a tile of 64
//                             (token, query-head-of-the-group) rows per block, flash-attention
//                             style: keys and values stream through shared memory in tiles of 64,
//                             scores and the running softmax stay in registers, 32-bit.
//   attention_decode_kernel   one new token per request: the query heads of one key/value head
//                             form the (padded) 16-row tile, the context is split over blocks and
//                             over the four warps of a block (each warp streams its own 16-key
//                             sub-tiles).  Up to 8 splits are launched as a thread-block cluster
//                             and hand their partial (max, sum, output) triples to the cluster's
//                             first block through distributed shared memory; with more splits the
//                             triples go to scratch memory and the block that finishes last for a
//                             head merges them.  Nobody waits for anybody except at the cluster
//                             barrier, which every block of a cluster reaches.  The kernel can take
//                             the raw q|k|v projections of the new tokens instead of finished
//                             queries (FusedQkv): it then applies QK norm and rotation itself and
//                             stores the new key and value in the cache.
//
// Both read keys and values only from the cache pages through the block table, mask by the
// absolute position of each query (causal, optional window) and never let a cache row outside
// the needed range reach the arithmetic: such rows are replaced by zeros while loading, so
// stale or never-written memory (NaN included) cannot leak into a result.
//
// Reference counterparts: flash_sdpa_tiled_kernel (src/runtime/kernels/cuda_kernels.cu:558-645,
// one block per query row, scalar FMA) and paged_attention_decode_batch_kernel (:697-754, one
// block per head walking the keys one at a time).
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16, at most 128>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 128, "HEAD_DIM must be a multiple of 16 in 16..128");

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

constexpr int HD = HEAD_DIM;
constexpr int BM = 64;            // rows of a portion tile (4 warps x 16)
constexpr int BN = 64;            // keys per shared-memory tile
constexpr int LDS = HD + 8;       // padded row length in shared memory (elements): conflict-free ldmatrix
constexpr int THREADS = 128;
constexpr int KSTEPS = HD / 16;   // k-steps of Q K^T
constexpr int DTILES = HD / 8;    // n-tiles of P V
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

struct FastAttnArgs {
    const bf16* q;               // [T, nh, HD]
    const bf16* cache;           // [pages][K|V][nkv][page_size][HD]
    bf16* out;                   // [T, nh, HD]
    const int* rows;             // [n_rows] batch rows (requests) this launch serves
    const int* cu_q_lens;        // [R+1]
    const int* ctx_lens;         // [R] cached length after this step
    const int* table_rows;       // [R] row of block_tables of each request
    const int* block_tables;     // [*, max_blocks]
    float* scratch;              // decode partials
    int max_blocks, n_rows, nh, nkv, page_size, window, splits;
    float scale;
};

// The decode kernel can take the raw projections instead of finished queries: it then norms and rotates the
// query heads itself, and the block whose share holds the new token's position does the same for the key head
// and stores key and value in the cache (what the QK-norm/rotation/cache-write kernel would have done in a
// launch of its own, src/model/transformer_graph_builder.cpp:224-240).
struct FusedQkv {
    const bf16* qkv;             // nullable; [T, (nh + 2 nkv) * HD]: query heads, key heads, value heads
    long long stride;            // elements between tokens
    const void* q_gain;          // nullable: no norm; [HD]
    const void* k_gain;
    int gain_dtype;              // LLME_F32 or LLME_BF16
    float eps;
    const float* cos_sin;        // nullable: no rotation; [max_positions, HD] = cos | sin
    int max_positions;
    int write_kv;                // 0: the layer reads another layer's cache and stores nothing
};
#include "kernel_args.h"
static_assert(sizeof(FastAttnArgs) == sizeof(LlmeFastAttnArgs) && sizeof(FusedQkv) == sizeof(LlmeFusedQkv), "the argument blocks must match kernel_args.h");

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy; with valid == false the destination is filled with zeros.
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
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// D += A(16x16, row) * B(16x8, col), bfloat16 operands, 32-bit accumulators
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Load keys [j0, j0+BN) of one key/value head into a [BN][LDS] shared tile (K or V).  Keys outside
// [lo, hi] become zeros.
// `page_shift` is log2(page size) when that is a power of two, else -1 (then the page is found by division).
__device__ __forceinline__ void load_kv_tile(bf16* dst, const bf16* cache, const int* bt, int which, int kvh, int nkv,
                                             int ps, int page_shift, int j0, int lo, int hi) {
    constexpr int CHUNKS = HD / 8;                      // 16-byte chunks per key row
    const size_t head_off = ((size_t)which * nkv + kvh) * ps;      // row offset of this head inside a page
    const size_t page_rows = (size_t)2 * nkv * ps;                 // rows of a whole page (K and V, all heads)
#pragma unroll
    for (int c = threadIdx.x; c < BN * CHUNKS; c += THREADS) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const int j = j0 + r;
        const bool valid = j >= lo && j <= hi;
        const bf16* src = cache;
        if (valid) {
            const int blk = page_shift >= 0 ? (j >> page_shift) : (j / ps);
            src = cache + ((size_t)bt[blk] * page_rows + head_off + (j - blk * ps)) * HD + ch * 8;
        }
        cp_async_16(dst + r * LDS + ch * 8, src, valid);
    }
}

// One warp: scores of its 16 rows against NT*8 keys starting at shared row `key0` of the K tile.
template <int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const unsigned (&qf)[KSTEPS][4], const bf16* Ks, int key0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            unsigned b[4];
            const int mi = lane >> 3;
            ldmatrix_x4(b, Ks + (key0 + np * 16 + (lane & 7) + (mi >> 1) * 8) * LDS + kk * 16 + (mi & 1) * 8);
            mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
            mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
        }
    }
}

// One warp: o += P V for NT*8 keys starting at shared row `key0` of the V tile; p holds the
// probabilities in the accumulator layout of the scores.
template <int NT>
__device__ __forceinline__ void pv_tile(float (&o)[DTILES][4], const float (&p)[NT][4], const bf16* Vs, int key0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        unsigned a[4];
        a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
        a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
        a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
        a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
            unsigned b[4];
            const int mi = lane >> 3;
            ldmatrix_x4_trans(b, Vs + (key0 + kk * 16 + (lane & 7) + (mi & 1) * 8) * LDS + dp * 16 + (mi >> 1) * 8);
            mma_bf16(o[2 * dp], a, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ float fast_exp2(float x) {     // 2^x, x <= 0 here; results below the normal range become 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Running maximum and sum for the two rows a thread holds (r0 = lane/4, r1 = r0 + 8), and the rescaling of
// the output accumulators.  s holds raw scores (q.k) on entry and the probabilities on exit; `sc` is
// scale * log2(e), applied inside the exponent; m is kept in those base-2 units.  MASK: keys outside
// [plo, phi] of a row are excluded (needed only for tiles that touch the diagonal or a window's edge).
// key index of s[n][c] is jbase + n*8 + (lane%4)*2 + (c&1); rows c<2 -> r0, c>=2 -> r1.
template <int NT, bool MASK>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[DTILES][4],
                                               int jbase, const int (&plo)[2], const int (&phi)[2], float sc) {
    const int lane = threadIdx.x & 31;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (MASK) {
                const int j = jbase + n * 8 + (lane & 3) * 2 + (c & 1);
                const int r = c >> 1;
                if (j < plo[r] || j > phi[r]) s[n][c] = -INFINITY;
            }
            mx[c >> 1] = fmaxf(mx[c >> 1], s[n][c]);
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], ref[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float mnew = fmaxf(m[r], mx[r] * sc);
        // a row that has seen no key yet keeps m = -inf: use 0 as the reference point so that exp2 gives 0, not NaN
        ref[r] = mnew == -INFINITY ? 0.0f : mnew;
        corr[r] = fast_exp2(m[r] - ref[r]);
        m[r] = mnew;
    }
    float sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float e = fast_exp2(fmaf(s[n][c], sc, -ref[c >> 1]));
            s[n][c] = e;
            sum[c >> 1] += e;
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l[r] = l[r] * corr[r] + sum[r];
    }
    // once the maxima have settled the factors are exactly 1 for the whole warp: skip the multiplications
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            o[d][0] *= corr[0]; o[d][1] *= corr[0];
            o[d][2] *= corr[1]; o[d][3] *= corr[1];
        }
    }
}

// ----------------------------------------------------------------------------- portions
// One warp: scores of its 16 query rows (fragments read from the shared Q tile at `Qw`) against NT*8 keys
// starting at shared row `key0` of the K tile.  Reading the query fragments from shared memory at every
// step instead of holding them costs a few loads and saves 4*KSTEPS registers per thread.
template <int NT>
__device__ __forceinline__ void qk_tile_shared_q(float (&s)[NT][4], const bf16* Qw, const bf16* Ks, int key0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
        unsigned qf[4];
        ldmatrix_x4(qf, Qw + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            unsigned b[4];
            const int mi = lane >> 3;
            ldmatrix_x4(b, Ks + (key0 + np * 16 + (lane & 7) + (mi >> 1) * 8) * LDS + kk * 16 + (mi & 1) * 8);
            mma_bf16(s[2 * np], qf, b[0], b[1]);
            mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
        }
    }
}

// A block holds one copy of the K and V tiles (no double buffering) and at most 128 registers per
// thread, so that four blocks (16 warps) share an SM and hide each other's waits; the scores of a 64-key
// tile are formed 32 keys at a time.
constexpr int PORTION_BLOCKS_PER_SM = HD <= 64 ? 6 : 4;

__global__ void __launch_bounds__(THREADS, PORTION_BLOCKS_PER_SM) attention_portion_kernel(FastAttnArgs a) {
    pdl_wait();                // everything below reads or writes what earlier kernels touch
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [BM][LDS]
    bf16* Ks = Qs + BM * LDS;                              // [BN][LDS]
    bf16* Vs = Ks + BN * LDS;                              // [BN][LDS]

    const int r = a.rows[blockIdx.z];
    const int kvh = blockIdx.y;
    const int G = a.nh / a.nkv;
    const int q0 = a.cu_q_lens[r];
    const int q_len = a.cu_q_lens[r + 1] - q0;
    const int M = q_len * G;
    // the tiles with the most keys (the last rows of the portion) start first
    const int m0 = ((M + BM - 1) / BM - 1 - (int)blockIdx.x) * BM;
    if (m0 < 0) return;
    const int start = a.ctx_lens[r] - q_len;               // position of the portion's first token
    const int* bt = a.block_tables + (size_t)a.table_rows[r] * a.max_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // rows of the tile -> (token, head of the group)
    const int t_lo = m0 / G;
    const int t_hi = min(q_len - 1, (m0 + BM - 1) / G);
    const int hi_max = start + t_hi;
    const int lo_min = a.window > 0 ? max(0, start + t_lo - a.window + 1) : 0;

    // Q tile
    {
        constexpr int CHUNKS = HD / 8;
        for (int c = threadIdx.x; c < BM * CHUNKS; c += THREADS) {
            const int row = c / CHUNKS, ch = c - row * CHUNKS;
            const int m = m0 + row;
            const bool valid = m < M;
            const bf16* src = a.q;
            if (valid) src = a.q + ((size_t)(q0 + m / G) * a.nh + kvh * G + m % G) * HD + ch * 8;
            cp_async_16(Qs + row * LDS + ch * 8, src, valid);
        }
    }

    // this thread's two rows
    int plo[2], phi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + warp * 16 + (lane >> 2) + i * 8;
        const int p = start + min(m, M - 1) / G;
        phi[i] = m < M ? p : -1;                            // rows past the portion see no key
        plo[i] = a.window > 0 ? max(0, p - a.window + 1) : 0;
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
    const float sc = a.scale * LOG2E;
    const bf16* Qw = Qs + warp * 16 * LDS;
    const int ps = a.page_size;
    const int page_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
    // the positions of the warp's first and last row bound what its rows may see
    const int warp_p_lo = start + min(q_len - 1, (m0 + warp * 16) / G);
    const int warp_hi = start + min(q_len - 1, (m0 + warp * 16 + 15) / G);
    const int warp_lo = a.window > 0 ? max(0, warp_p_lo - a.window + 1) : 0;
    const int warp_lo_last = a.window > 0 ? max(0, warp_hi - a.window + 1) : 0;
    const bool warp_has_rows = m0 + warp * 16 < M;
    const bool warp_full = m0 + warp * 16 + 15 < M;          // no row of the warp lies past the portion

    for (int j0 = (lo_min / BN) * BN; j0 <= hi_max; j0 += BN) {
        load_kv_tile(Ks, a.cache, bt, 0, kvh, a.nkv, ps, page_shift, j0, lo_min, hi_max);
        cp_async_commit();                                  // (the first group also carries the Q tile)
        load_kv_tile(Vs, a.cache, bt, 1, kvh, a.nkv, ps, page_shift, j0, lo_min, hi_max);
        cp_async_commit();
        cp_async_wait<1>();                                 // the keys have landed, the values may still be on their way
        __syncthreads();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int jb = j0 + half * 32;
            // skip 32-key blocks that lie wholly after, or wholly before, what this warp's rows may see
            const bool live = warp_has_rows && jb <= warp_hi && jb + 31 >= warp_lo;
            float sreg[4][4];
            if (live) {
                qk_tile_shared_q<4>(sreg, Qw, Ks, half * 32);
                // a block of keys that every row of the warp sees entirely needs no mask
                if (warp_full && jb + 31 <= warp_p_lo && jb >= warp_lo_last)
                    softmax_update<4, false>(sreg, m_run, l_run, o, jb, plo, phi, sc);
                else
                    softmax_update<4, true>(sreg, m_run, l_run, o, jb, plo, phi, sc);
            }
            if (half == 0) {
                cp_async_wait<0>();                         // now the values are needed
                __syncthreads();
            }
            if (live) pv_tile<4>(o, sreg, Vs, half * 32);
        }
        __syncthreads();                                    // everyone is done with the tiles before they are refilled
    }

    pdl_launch_dependents();
    // write the rows
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + warp * 16 + (lane >> 2) + i * 8;
        if (m >= M) continue;
        const float inv = 1.0f / l_run[i];
        bf16* dst = a.out + ((size_t)(q0 + m / G) * a.nh + kvh * G + m % G) * HD;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            const int col = d * 8 + (lane & 3) * 2;
            *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
        }
    }
}

// ----------------------------------------------------------------------------- decode
// grid (splits, nkv * head_chunks, n_rows).  A block serves one request, one key/value head (up to 16 of
// its query heads) and one share of the context.  Its four warps work independently: warp w takes the
// 16-key sub-tiles w, w+4, w+8, ... of the block's share and streams them through a pipeline of its own
// (DSTAGES sub-tiles in flight per warp, no block-wide barrier inside the loop), so that enough bytes are
// in flight to cover the memory latency.  At the end the warps' partial results are merged in shared
// memory; with more than one split the block's result goes to the first block of its cluster (up to 8
// splits) or to scratch memory, where the last block to arrive merges the splits.
// Scratch per (request row, query head, split): HD outputs (not normalised), then max (base-2 units) and sum.
constexpr int PART = HD + 2;
// Scratch layout: COUNTER_WORDS ticket counters (one per (request, key/value head) of a call; they must be
// zero before the first call and every call leaves them zero), then the partial results.
constexpr int COUNTER_WORDS = 65536;
__device__ __forceinline__ float* partials(const FastAttnArgs& a) { return a.scratch + COUNTER_WORDS; }
constexpr int SUB = 16;           // keys per sub-tile
constexpr int PAGE_TAB = 512;     // block-table entries a block keeps in shared memory (longer ranges are read from global memory)
constexpr int DSTAGES = 2;        // stage buffers per warp (one sub-tile in flight while one is used; three measured the same)
constexpr int CL_SLOTS = 48;      // (split, row) partial results a cluster's first block can take in its shared memory
constexpr int STAGE_ELEMS = 2 * SUB * LDS;   // K rows then V rows

// One warp loads keys [j0, j0+16) (K and V) into its stage buffer; keys outside [lo, hi] become zeros.
// When the page size is a multiple of 16 (page_shift >= 4) the 16 keys lie in one page: one look-up in the
// block table, and every lane's addresses differ from one another only by constants.
// `bt` points at the entry of block `bt_first` (the request's row of the block table in global memory, or the
// part of it that the block has copied into shared memory).
__device__ __forceinline__ void load_sub_tile(bf16* dst, const bf16* cache, const int* bt, int bt_first, int kvh, int nkv, int ps,
                                              int page_shift, int j0, int lo, int hi) {
    const int lane = threadIdx.x & 31;
    constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per key row
    constexpr int TOTAL = SUB * CHUNKS;            // chunks of K (and as many of V)
    if (page_shift >= 4) {
        const int blk = j0 >> page_shift;
        const bool any = j0 + SUB - 1 >= lo && j0 <= hi;
        const bf16* kbase = cache;
        if (any) kbase = cache + ((((size_t)bt[blk - bt_first] * 2) * nkv + kvh) * ps + (j0 - (blk << page_shift))) * HD;
        const size_t v_off = (size_t)nkv * ps * HD;
#pragma unroll
        for (int c = lane; c < TOTAL; c += 32) {
            const int r = c / CHUNKS, ch = c - r * CHUNKS;
            const bool valid = j0 + r >= lo && j0 + r <= hi;
            const bf16* src = kbase + r * HD + ch * 8;
            cp_async_16(dst + r * LDS + ch * 8, valid ? src : cache, valid);
            cp_async_16(dst + (SUB + r) * LDS + ch * 8, valid ? src + v_off : cache, valid);
        }
        return;
    }
#pragma unroll
    for (int c = lane; c < TOTAL; c += 32) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const int j = j0 + r;
        const bool valid = j >= lo && j <= hi;
        const bf16* ksrc = cache;
        if (valid) {
            const int blk = page_shift >= 0 ? (j >> page_shift) : (j / ps);
            const int page = bt[blk - bt_first];
            ksrc = cache + ((((size_t)page * 2) * nkv + kvh) * ps + (j - blk * ps)) * HD + ch * 8;
        }
        cp_async_16(dst + r * LDS + ch * 8, ksrc, valid);
        cp_async_16(dst + (SUB + r) * LDS + ch * 8, valid ? ksrc + (size_t)nkv * ps * HD : cache, valid);
    }
}

// One head (HD values at src) through the per-head RMS norm and the rotate-half rotation, as the kernel of
// elementwise.cu does it (the same order of operations): lane l holds the pairs (d, d+1) and (d + HD/2, d + HD/2 + 1)
// for d = 2 (l + 32 i).  The result goes to dst_a and, if given, dst_b.  One warp.
__device__ __forceinline__ void norm_rotate_head(const bf16* src, const void* gain, int gain_dtype, float eps,
                                                 const float* cs, bf16* dst_a, bf16* dst_b) {
    constexpr int half = HD / 2;
    constexpr int NP = (half + 63) / 64;
    const int lane = threadIdx.x & 31;
    float2 lo[NP], hi[NP];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int d = 2 * (lane + 32 * i);
        if (d < half) {
            lo[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + d));
            hi[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + d + half));
            ss += lo[i].x * lo[i].x + lo[i].y * lo[i].y + hi[i].x * hi[i].x + hi[i].y * hi[i].y;
        }
    }
    if (gain) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rinv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < half) {
                float2 g0, g1;
                if (gain_dtype == LLME_F32) {
                    g0 = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(gain) + d);
                    g1 = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(gain) + d + half);
                } else {
                    g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const bf16*>(gain) + d));
                    g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const bf16*>(gain) + d + half));
                }
                lo[i].x = (lo[i].x * rinv) * g0.x; lo[i].y = (lo[i].y * rinv) * g0.y;
                hi[i].x = (hi[i].x * rinv) * g1.x; hi[i].y = (hi[i].y * rinv) * g1.y;
            }
        }
    }
    if (cs) {
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < half) {
                const float2 c = *reinterpret_cast<const float2*>(cs + d);
                const float2 sn = *reinterpret_cast<const float2*>(cs + half + d);
                const float2 x0 = lo[i], x1 = hi[i];
                lo[i] = make_float2(x0.x * c.x - x1.x * sn.x, x0.y * c.y - x1.y * sn.y);
                hi[i] = make_float2(x0.x * sn.x + x1.x * c.x, x0.y * sn.y + x1.y * c.y);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int d = 2 * (lane + 32 * i);
        if (d < half) {
            const __nv_bfloat162 a2 = __floats2bfloat162_rn(lo[i].x, lo[i].y), b2 = __floats2bfloat162_rn(hi[i].x, hi[i].y);
            *reinterpret_cast<__nv_bfloat162*>(dst_a + d) = a2;
            *reinterpret_cast<__nv_bfloat162*>(dst_a + d + half) = b2;
            if (dst_b) {
                *reinterpret_cast<__nv_bfloat162*>(dst_b + d) = a2;
                *reinterpret_cast<__nv_bfloat162*>(dst_b + d + half) = b2;
            }
        }
    }
}

__global__ void __launch_bounds__(THREADS) attention_decode_kernel(FastAttnArgs a, FusedQkv f) {
    // Launched while the kernel before it is still running (programmatic dependent launch), the kernel may read, before
    // pdl_wait(), only what that kernel does not write.  Taking the raw projections (f.qkv), it follows the product
    // that made them: the step's lengths and tables and the keys and values of earlier positions are older than that
    // product, so the block table and the first key/value loads need not wait for it; the projections do.  Otherwise
    // the kernel before it has written the cache, and everything waits.
    const bool early_loads = f.qkv != nullptr;
    if (!early_loads) pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);              // [16][LDS]
    bf16* stages = Qs + 16 * LDS;                              // [4 warps][DSTAGES][K 16 rows | V 16 rows][LDS]
    float* red = reinterpret_cast<float*>(stages);             // [4 warps][16 rows][PART], reuses the stages after the loop
    float* cl_part = reinterpret_cast<float*>(stages + 4 * DSTAGES * STAGE_ELEMS);   // [CL_SLOTS][PART]: written by the other blocks of a cluster
    // Launched as a cluster of `splits` blocks (one per split of a request and key/value head), the blocks hand
    // their partial results to the first block through distributed shared memory instead of global memory.
    unsigned cl_rank, cl_size;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cl_rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(cl_size));
    const bool clustered = cl_size > 1;
    // A block may store into the first block's shared memory only once that block is known to run.  Every
    // block of the cluster arrives here, at its very start, and waits for the others just before its first
    // remote store; by then the key/value loop has hidden the wait.
    if (clustered) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    const int zi = blockIdx.z;
    const int r = a.rows[zi];
    const int G = a.nh / a.nkv;
    const int chunks = (G + 15) / 16;
    const int kvh = blockIdx.y / chunks, g0 = (blockIdx.y % chunks) * 16;
    const int rows_here = min(16, G - g0);
    const int split = blockIdx.x;
    const int t = a.cu_q_lens[r];                          // the request's single token
    const int p = a.ctx_lens[r] - 1;                       // its position
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    const int* bt = a.block_tables + (size_t)a.table_rows[r] * a.max_blocks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ps = a.page_size;
    const int page_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;

    // this block's share of the 16-key sub-tiles, in whole groups of four (one per warp)
    const int sub_first = lo / SUB, sub_last = p / SUB;
    const int n_groups = (sub_last - sub_first + 4) / 4;
    const int per = (n_groups + a.splits - 1) / a.splits;
    const int my_first = sub_first + split * per * 4;
    const int my_last = min(sub_last, my_first + per * 4 - 1);

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;

    // The block's part of the block table goes to shared memory first, all entries at once: looked up in
    // global memory one by one, in front of every sub-tile's copies, each entry cost a warp a memory
    // round trip (8 of them per warp at 2,048 cached tokens, about a third of the kernel's time).
    __shared__ int page_tab[PAGE_TAB];
    const int* tab = bt;
    int tab_first = 0;
    if (my_first <= my_last) {
        const int blk_first = (max(my_first * SUB, lo)) / ps, blk_last = min(my_last * SUB + SUB - 1, p) / ps;
        if (blk_last - blk_first < PAGE_TAB) {
            for (int i = threadIdx.x; i <= blk_last - blk_first; i += THREADS) page_tab[i] = bt[blk_first + i];
            tab = page_tab;
            tab_first = blk_first;
            __syncthreads();
        }
    }
    const float* cs_row = nullptr;
    if (f.qkv && f.cos_sin) {
        const int pos = p < 0 ? 0 : (p >= f.max_positions ? f.max_positions - 1 : p);      // the host refuses such positions
        cs_row = f.cos_sin + (size_t)pos * HD;
    }
    // this block's share holds the new token's position: it stores the token's key and value
    const bool writer = f.qkv && f.write_kv && my_first <= my_last && my_last == sub_last;
    auto store_new_kv = [&]() {
        const int blk = p / ps;
        const size_t at = ((((size_t)bt[blk] * 2) * a.nkv + kvh) * ps + (p - blk * ps)) * HD;
        const bf16* tok = f.qkv + (size_t)t * f.stride;
        if (warp == 0)
            norm_rotate_head(tok + (size_t)(a.nh + kvh) * HD, f.k_gain, f.gain_dtype, f.eps, cs_row,
                             const_cast<bf16*>(a.cache) + at, nullptr);
        if (warp == 1) {
            const bf16* vsrc = tok + (size_t)(a.nh + a.nkv + kvh) * HD;
            bf16* vdst = const_cast<bf16*>(a.cache) + at + (size_t)a.nkv * ps * HD;
            for (int d = 2 * lane; d < HD; d += 64) *reinterpret_cast<unsigned*>(vdst + d) = *reinterpret_cast<const unsigned*>(vsrc + d);
        }
    };
    // With few sub-tiles the first loads below may already fetch the new token's position: then it is stored first.
    const bool store_early = writer && my_last - my_first < 4 * (DSTAGES - 1);
    bool waited = !early_loads;
    if (store_early) {
        if (!waited) pdl_wait();           // the new key and value come from the projections
        waited = true;
        store_new_kv();
        __threadfence_block();
        __syncthreads();
    }
    if (my_first <= my_last) {
        // the query rows, loaded by the whole block
        if (!f.qkv) {
            constexpr int CHUNKS = HD / 8;
            for (int c = threadIdx.x; c < 16 * CHUNKS; c += THREADS) {
                const int row = c / CHUNKS, ch = c - row * CHUNKS;
                const bool valid = row < rows_here;
                const bf16* src = a.q;
                if (valid) src = a.q + ((size_t)t * a.nh + kvh * G + g0 + row) * HD + ch * 8;
                cp_async_16(Qs + row * LDS + ch * 8, src, valid);
            }
        }
        cp_async_commit();
        bf16* mine = stages + (size_t)warp * DSTAGES * STAGE_ELEMS;
        // prologue: the first DSTAGES-1 sub-tiles of this warp
#pragma unroll
        for (int st = 0; st < DSTAGES - 1; ++st) {
            const int sub = my_first + warp + 4 * st;
            if (sub <= my_last) load_sub_tile(mine + st * STAGE_ELEMS, a.cache, tab, tab_first, kvh, a.nkv, ps, page_shift, sub * SUB, lo, p);
            cp_async_commit();
        }
        if (!waited) pdl_wait();           // the first key/value loads are under way: now the projections
        waited = true;
        if (f.qkv) {
            // the query heads from the raw projection: a warp per head; rows beyond the group's heads are zeros
            for (int row = warp; row < 16; row += 4) {
                if (row < rows_here)
                    norm_rotate_head(f.qkv + (size_t)t * f.stride + (size_t)(kvh * G + g0 + row) * HD, f.q_gain, f.gain_dtype, f.eps,
                                     cs_row, Qs + row * LDS, nullptr);
                else
                    for (int d = 2 * lane; d < HD; d += 64) *reinterpret_cast<unsigned*>(Qs + row * LDS + d) = 0u;
            }
            // the new token's key and value, before any load that may fetch them (those follow the barrier below)
            if (writer && !store_early) {
                store_new_kv();
                __threadfence_block();
            }
        }
        cp_async_wait<DSTAGES - 1>();                       // the query rows have landed
        __syncthreads();
        unsigned qf[KSTEPS][4];
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk)
            ldmatrix_x4(qf[kk], Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + kk * 16 + (lane >> 4) * 8);

        int plo[2] = {lo, lo}, phi[2];
        phi[0] = (lane >> 2) < rows_here ? p : -1;
        phi[1] = (lane >> 2) + 8 < rows_here ? p : -1;
        const float sc = a.scale * LOG2E;
        int n = 0;
        for (int sub = my_first + warp; sub <= my_last; sub += 4, ++n) {
            const int ahead = sub + 4 * (DSTAGES - 1);
            if (ahead <= my_last)
                load_sub_tile(mine + ((n + DSTAGES - 1) % DSTAGES) * STAGE_ELEMS, a.cache, tab, tab_first, kvh, a.nkv, ps, page_shift,
                              ahead * SUB, lo, p);
            cp_async_commit();
            cp_async_wait<DSTAGES - 1>();                   // this lane's copies of sub-tile n are done
            __syncwarp();                                   // ... and so are the other lanes'
            const bf16* Kt = mine + (n % DSTAGES) * STAGE_ELEMS;
            float sreg[2][4];
            qk_tile<2>(sreg, qf, Kt, 0);
            // only the sub-tiles at the two ends of the visible range hold keys that must be masked
            // (rows past the group's heads hold zero queries: finite, and never stored)
            if (sub * SUB >= lo && sub * SUB + SUB - 1 <= p)
                softmax_update<2, false>(sreg, m_run, l_run, o, sub * SUB, plo, phi, sc);
            else
                softmax_update<2, true>(sreg, m_run, l_run, o, sub * SUB, plo, phi, sc);
            pv_tile<2>(o, sreg, Kt + SUB * LDS, 0);
            __syncwarp();                                   // all lanes have read the stage before it is refilled
        }
        cp_async_wait<0>();
    }
    if (!waited) pdl_wait();               // a block without a share of the context: before it writes anything
    __syncthreads();

    // merge the four warps' partial results in shared memory, in a fixed order
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = (lane >> 2) + i * 8;
        float* dst = red + ((size_t)warp * 16 + row) * PART;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            const int col = d * 8 + (lane & 3) * 2;
            dst[col] = o[d][2 * i];
            dst[col + 1] = o[d][2 * i + 1];
        }
        if ((lane & 3) == 0) {
            dst[HD] = m_run[i];
            dst[HD + 1] = l_run[i];
        }
    }
    __syncthreads();
    if (clustered) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");     // all blocks of the cluster have started
    for (int row = warp; row < rows_here; row += 4) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[((size_t)w * 16 + row) * PART + HD]);
        const float ref = mm == -INFINITY ? 0.0f : mm;
        float wgt[4], ll = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            wgt[w] = exp2f(red[((size_t)w * 16 + row) * PART + HD] - ref);
            ll += wgt[w] * red[((size_t)w * 16 + row) * PART + HD + 1];
        }
        const int head = kvh * G + g0 + row;
        if (a.splits == 1) {
            bf16* dst = a.out + ((size_t)t * a.nh + head) * HD;
            const float inv = 1.0f / ll;
            for (int d = lane; d < HD; d += 32) {
                float acc = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + row) * PART + d];
                dst[d] = __float2bfloat16_rn(acc * inv);
            }
        } else if (clustered) {
            // into the shared memory of the cluster's first block, slot (split, row)
            const unsigned local = (unsigned)__cvta_generic_to_shared(cl_part + ((size_t)split * rows_here + row) * PART);
            unsigned remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(local));
            for (int d = lane; d < HD; d += 32) {
                float acc = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + row) * PART + d];
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * (unsigned)d), "f"(acc) : "memory");
            }
            if (lane == 0) {
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * (unsigned)HD), "f"(mm) : "memory");
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + 4u * (unsigned)(HD + 1)), "f"(ll) : "memory");
            }
        } else {
            float* dst = partials(a) + (((size_t)zi * a.nh + head) * a.splits + split) * PART;
            for (int d = lane; d < HD; d += 32) {
                float acc = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + row) * PART + d];
                dst[d] = acc;
            }
            if (lane == 0) {
                dst[HD] = mm;
                dst[HD + 1] = ll;
            }
        }
    }
    if (a.splits == 1) return;
    if (clustered) {
        // every block of the cluster comes here (none returns earlier); after the barrier the first block finds
        // all partial results in its own shared memory and merges them, in the order of the splits
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (cl_rank != 0) return;
        for (int row = warp; row < rows_here; row += 4) {
            const int head = kvh * G + g0 + row;
            const float* src = cl_part + (size_t)row * PART;           // split s at src + s * rows_here * PART
            const size_t step = (size_t)rows_here * PART;
            float mm = -INFINITY;
            for (int s2 = lane; s2 < a.splits; s2 += 32) mm = fmaxf(mm, src[s2 * step + HD]);
            mm = warp_max(mm);
            const float ref = mm == -INFINITY ? 0.0f : mm;
            constexpr int KREGS = (HD + 31) / 32;
            float ll = 0.0f, w_mine = 0.0f;
            if (lane < a.splits) {
                w_mine = exp2f(src[lane * step + HD] - ref);
                ll = w_mine * src[lane * step + HD + 1];
            }
            ll = warp_sum(ll);
            float acc[KREGS];
#pragma unroll
            for (int k = 0; k < KREGS; ++k) acc[k] = 0.0f;
            for (int s2 = 0; s2 < a.splits; ++s2) {                     // at most 8 splits in a cluster
                const float w = __shfl_sync(0xffffffffu, w_mine, s2);
#pragma unroll
                for (int k = 0; k < KREGS; ++k) {
                    const int d = lane + 32 * k;
                    if (d < HD) acc[k] += w * src[s2 * step + d];
                }
            }
            bf16* dst = a.out + ((size_t)t * a.nh + head) * HD;
            const float inv = 1.0f / ll;
#pragma unroll
            for (int k = 0; k < KREGS; ++k) {
                const int d = lane + 32 * k;
                if (d < HD) dst[d] = __float2bfloat16_rn(acc[k] * inv);
            }
        }
        return;
    }

    // The block that finishes last for this (request, key/value head) merges the splits.  No block waits
    // for another: each one publishes its partial results, takes a ticket, and only the holder of the last
    // ticket goes on (and puts the counter back to zero for the next call).
    __shared__ int last_block;
    __threadfence();                                       // this block's partial results are visible device-wide
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = reinterpret_cast<int*>(a.scratch) + (size_t)zi * gridDim.y + blockIdx.y;
        const int ticket = atomicAdd(counter, 1);
        last_block = ticket == a.splits - 1;
        if (last_block) *counter = 0;
    }
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    for (int row = warp; row < rows_here; row += 4) {
        const int head = kvh * G + g0 + row;
        const float* src = partials(a) + ((size_t)zi * a.nh + head) * a.splits * PART;
        float mm = -INFINITY;
        for (int s = lane; s < a.splits; s += 32) mm = fmaxf(mm, __ldcg(src + s * PART + HD));
        mm = warp_max(mm);
        const float ref = mm == -INFINITY ? 0.0f : mm;
        // Splits are added in their own order, so the result does not depend on which block came last.  Lane s of
        // a batch of 32 splits holds that split's weight; the partial outputs are fetched eight splits at a time
        // (loads that do not wait for one another) and added with the weight passed from its lane.  An empty
        // split holds zeros and has weight 0.
        constexpr int KREGS = (HD + 31) / 32;
        float ll = 0.0f;
        float acc[KREGS];
#pragma unroll
        for (int k = 0; k < KREGS; ++k) acc[k] = 0.0f;
        for (int s0 = 0; s0 < a.splits; s0 += 32) {
            float w_mine = 0.0f;
            if (s0 + lane < a.splits) {
                w_mine = exp2f(__ldcg(src + (s0 + lane) * PART + HD) - ref);
                ll += w_mine * __ldcg(src + (s0 + lane) * PART + HD + 1);
            }
            const int n = min(32, a.splits - s0);
            for (int j0 = 0; j0 < n; j0 += 8) {
                float v[8][KREGS];
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int k = 0; k < KREGS; ++k) {
                        const int d = lane + 32 * k;
                        v[j][k] = (j0 + j < n && d < HD) ? __ldcg(src + (size_t)(s0 + j0 + j) * PART + d) : 0.0f;
                    }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float w = __shfl_sync(0xffffffffu, w_mine, (j0 + j) & 31);
#pragma unroll
                    for (int k = 0; k < KREGS; ++k) acc[k] += w * v[j][k];
                }
            }
        }
        ll = warp_sum(ll);
        bf16* dst = a.out + ((size_t)t * a.nh + head) * HD;
        const float inv = 1.0f / ll;
#pragma unroll
        for (int k = 0; k < (HD + 31) / 32; ++k) {
            const int d = lane + 32 * k;
            if (d < HD) dst[d] = __float2bfloat16_rn(acc[k] * inv);
        }
    }
}

constexpr size_t PORTION_SMEM = (size_t)(BM + 2 * BN) * LDS * sizeof(bf16);
constexpr size_t DECODE_SMEM = (size_t)(16 * LDS + 4 * DSTAGES * STAGE_ELEMS) * sizeof(bf16) + (size_t)CL_SLOTS * PART * sizeof(float);
static_assert((size_t)4 * 16 * PART * sizeof(float) <= (size_t)4 * DSTAGES * STAGE_ELEMS * sizeof(bf16), "the merge buffer must fit the stage buffers");

int check_common(const FastAttnArgs& a, bool fused = false) {
    if ((!a.q && !fused) || !a.cache || !a.out || !a.rows || !a.cu_q_lens || !a.ctx_lens || !a.table_rows || !a.block_tables)
        LLME_REFUSE("attention: null pointer");
    if (a.nh <= 0 || a.nkv <= 0 || a.nh % a.nkv) LLME_REFUSE("attention: %d query heads are not a multiple of %d key/value heads", a.nh, a.nkv);
    if (a.page_size <= 0 || a.max_blocks <= 0) LLME_REFUSE("attention: non-positive size");
    if (a.n_rows > 65535) LLME_REFUSE("attention: more than 65535 requests in one launch");
    return 0;
}

}  // namespace

LLME_API int llme_attention_head_dim() { return HD; }

// Floats of scratch that the decode kernel needs for `n_rows` requests.
LLME_API long long llme_attention_decode_scratch_floats(int n_rows, int nh, int splits) {
    return splits <= 1 ? 0 : (long long)COUNTER_WORDS + (long long)n_rows * nh * splits * PART;
}

// How many clusters of `splits` blocks of the decode kernel the GPU holds at once (0: unknown).  A cluster's blocks
// must find room in one GPC together, so this is less than the blocks the SMs hold divided by the cluster's size.
LLME_API int llme_attention_decode_clusters(int splits) {
    if (splits < 2 || splits > 8) return 0;
    static int known[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (known[splits]) return known[splits];
    if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)splits, 1024, 1);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = DECODE_SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    known[splits] = n;
    return n;
}

LLME_API int llme_attention_portion(const FastAttnArgs* args, int max_q_len, cudaStream_t stream) {
    const FastAttnArgs& a = *args;
    if (a.n_rows <= 0 || max_q_len <= 0) return 0;
    if (int rc = check_common(a)) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_portion_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PORTION_SMEM);
        if (e != cudaSuccess) LLME_REFUSE("attention: cannot reserve %zu bytes of shared memory: %s", PORTION_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    const int G = a.nh / a.nkv;
    const long long tiles = ((long long)max_q_len * G + BM - 1) / BM;
    if (tiles > 2147483647LL || a.nkv > 65535) LLME_REFUSE("attention: grid too large");
    dim3 grid((unsigned)tiles, a.nkv, a.n_rows);
    llme_launch(attention_portion_kernel, dim3(grid), dim3(THREADS), PORTION_SMEM, stream, a);
    LLME_LAUNCH_STATUS();
}

static int launch_decode(const FastAttnArgs& a, const FusedQkv& f, cudaStream_t stream) {
    if (a.n_rows <= 0) return 0;
    if (int rc = check_common(a, f.qkv != nullptr)) return rc;
    if (a.splits < 1 || a.splits > 1024) LLME_REFUSE("attention: splits must be in 1..1024, got %d", a.splits);
    if (a.splits > 1 && !a.scratch) LLME_REFUSE("attention: split decoding needs scratch memory");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
        if (e != cudaSuccess) LLME_REFUSE("attention: cannot reserve %zu bytes of shared memory: %s", DECODE_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    const int G = a.nh / a.nkv;
    const int chunks = (G + 15) / 16;
    if ((long long)a.nkv * chunks > 65535) LLME_REFUSE("attention: grid too large");
    dim3 grid(a.splits, a.nkv * chunks, a.n_rows);
    if ((long long)a.n_rows * a.nkv * chunks > COUNTER_WORDS) LLME_REFUSE("attention: more than %d (request, head) pairs in one split launch", COUNTER_WORDS);
    const int rows_cap = G < 16 ? G : 16;
    if (a.splits >= 2 && a.splits <= 8 && a.splits * rows_cap <= CL_SLOTS) {
        // the splits of a (request, key/value head) as one thread-block cluster: they merge through the first
        // block's shared memory
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = DECODE_SMEM;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        // the kernel may begin while the product before it runs (its block table and first key/value loads do not
        // wait for it), but it never lets its successor in before it has finished: that cost the kernels around it 7
        // to 10 us (common.cuh)
        attr[0].val.programmaticStreamSerializationAllowed = llme_pdl_enabled() ? 1 : 0;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)a.splits;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        cudaLaunchKernelEx(&cfg, attention_decode_kernel, a, f);
        LLME_LAUNCH_STATUS();
    }
    llme_launch(attention_decode_kernel, dim3(grid), dim3(THREADS), DECODE_SMEM, stream, a, f);
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_attention_decode(const FastAttnArgs* args, cudaStream_t stream) {
    const FusedQkv none = {};
    return launch_decode(*args, none, stream);
}

// The same with the raw q|k|v projections of the new tokens instead of finished queries (args->q is ignored):
// the kernel norms and rotates the heads and stores the new keys and values itself.
LLME_API int llme_attention_decode_fused(const FastAttnArgs* args, const FusedQkv* fused, cudaStream_t stream) {
    const FusedQkv& f = *fused;
    if (!f.qkv) LLME_REFUSE("attention: the fused decode needs the raw projections");
    if (HD % 4) LLME_REFUSE("attention: the fused decode needs a head size that is a multiple of 4");
    if (f.stride % 2 || ((uintptr_t)f.qkv | (uintptr_t)f.q_gain | (uintptr_t)f.k_gain | (uintptr_t)f.cos_sin) % 8)
        LLME_REFUSE("attention: the fused decode needs 8-byte aligned rows");
    if ((f.q_gain || f.k_gain) && !(f.eps > 0.0f)) LLME_REFUSE("attention: eps must be positive");
    if ((f.q_gain == nullptr) != (f.k_gain == nullptr)) LLME_REFUSE("attention: the fused decode norms both queries and keys or neither");
    if (f.q_gain && f.gain_dtype != LLME_F32 && f.gain_dtype != LLME_BF16) LLME_REFUSE("attention: unsupported gain dtype %d", f.gain_dtype);
    if (f.cos_sin && f.max_positions <= 0) LLME_REFUSE("attention: rotation needs the table's length");
    return launch_decode(*args, f, stream);
}
