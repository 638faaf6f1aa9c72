// The tcgen05 plumbing of the matrix-product kernel (kept apart from the kernel itself): mbarrier and TMA wrappers with bounded
// waits, shared-memory matrix descriptors and the instruction descriptor of tcgen05.mma (kind::f16), loads
// from tensor memory, and the host side of a tiled tensor map.  Included inside the including file's
// unnamed namespace, after <cuda.h> and "common.cuh"; every library has its own error flag g_status.
#pragma once

typedef __nv_bfloat16 bf16;
constexpr int BM = 128;                 // rows of the A operand per tile (the lanes of tensor memory)
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

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}

// ---- a pair of blocks on one tile (a cluster of two, tcgen05 with .cta_group::2)
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of the same place in the shared memory of block `rank`
__device__ __forceinline__ unsigned map_to_cta(unsigned smem_addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A load into this block's shared memory whose bytes are counted on a barrier of the pair's other block (`bar`: an
// address in the cluster's shared window).  No multicast: every block fetches what it needs itself.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// One instruction over both blocks' operands: M = 256 (128 rows from each block's A tile), N from both blocks'
// halves of B; the accumulator's rows 0..127 live in the first block's tensor memory, 128..255 in the second's.
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                               unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, when the pair's instructions so far have finished, on the barrier at this place in BOTH blocks
__device__ __forceinline__ void umma_commit_pair(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
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

// A [rows, cols] matrix with row stride ld (elements of `elem_bytes`), cut into boxes of box_rows x box_cols,
// 128-byte swizzle (box_cols * elem_bytes = 128); parts of a box outside the matrix read as zeros and are
// not written.
int make_map(CUtensorMap* map, const void* base, CUtensorMapDataType type, int elem_bytes, long long rows, long long cols,
             long long ld, int box_rows, int box_cols) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) LLME_REFUSE("gemm_tc: cuTensorMapEncodeTiled is not available in this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) LLME_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) v = 148;
        return v;
    }();
    return n;
}

