// The step executor: walks a plan (the model's operation records) for one step and launches, per record, the kernel
// that serves the step's shape.  Host code only; the interface and the ideas are in
// include/llmengine_b200/executor.h.  The kernels live in libraries of their own and are reached through entry
// points registered by name, so this file knows their argument blocks (kernel_args.h) but not their code.
//
// Library matrix products (bfloat16 products of 17 to 127 tokens, and larger ones whose tiles would not fill the
// GPU) go to cuBLAS, as the reference's do (src/runtime/kernels/cuda_kernels.cu:892-908).  cuBLAS is not linked:
// the copy already in the process (PyTorch's) is looked up at run time, and the caller's handle is used when the
// step brings one, so that a captured step and an eager one take the same library path.
#include <cublas_v2.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "kernel_args.h"
#include "llmengine_b200/executor.h"

#define LLME_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// entry points of the kernel libraries
typedef int (*EmbeddingFn)(const int*, const void*, int, float*, int, int, int, cudaStream_t);
typedef int (*RmsNormFn)(float*, const void*, int, const void*, int, void*, int, const int*, int, int, float, cudaStream_t);
typedef int (*QkvPostFn)(const LlmeQkvArgs*, int, int, cudaStream_t);
typedef int (*SwigluFn)(const void*, int, void*, int, int, int, cudaStream_t);
typedef int (*GemmF32Fn)(const float*, const void*, int, float*, int, int, int, long long, long long, long long, cudaStream_t);
typedef int (*GemmBf16Fn)(const void*, long long, const void*, long long, void*, int, long long, int, int, int, cudaStream_t);
typedef int (*GemmTcSwigluFn)(const void*, long long, const void*, long long, void*, long long, int, int, int, cudaStream_t);
typedef int (*AttnPlainFn)(const LlmeAttnArgs*, int, cudaStream_t);
typedef int (*AttnPortionFn)(const LlmeFastAttnArgs*, int, cudaStream_t);
typedef int (*AttnDecodeFn)(const LlmeFastAttnArgs*, cudaStream_t);
typedef int (*AttnDecodeFusedFn)(const LlmeFastAttnArgs*, const LlmeFusedQkv*, cudaStream_t);
typedef long long (*AttnScratchFn)(int, int, int);
typedef int (*AttnTcFn)(const void*, long long, long long, const LlmeTcAttnArgs*, int, cudaStream_t);
typedef const char* (*LastErrorFn)();

struct Blas {
    void* lib = nullptr;
    cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
    cublasStatus_t (*destroy)(cublasHandle_t) = nullptr;
    cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
    cublasStatus_t (*set_math)(cublasHandle_t, cublasMath_t) = nullptr;
    cublasStatus_t (*set_workspace)(cublasHandle_t, void*, size_t) = nullptr;
    cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                              cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                              cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
    bool load() {
        if (lib) return gemm_ex != nullptr;
        for (const char* name : {"libcublas.so.12", "libcublas.so"}) {
            lib = dlopen(name, RTLD_NOW | RTLD_NOLOAD);          // the copy the process already has
            if (lib) break;
        }
        if (!lib)
            for (const char* name : {"libcublas.so.12", "libcublas.so", "/usr/local/cuda/lib64/libcublas.so.12", "/usr/local/cuda/lib64/libcublas.so"}) {
                lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
                if (lib) break;
            }
        if (!lib) return false;
        create = (decltype(create))dlsym(lib, "cublasCreate_v2");
        destroy = (decltype(destroy))dlsym(lib, "cublasDestroy_v2");
        set_stream = (decltype(set_stream))dlsym(lib, "cublasSetStream_v2");
        set_math = (decltype(set_math))dlsym(lib, "cublasSetMathMode");
        set_workspace = (decltype(set_workspace))dlsym(lib, "cublasSetWorkspace_v2");
        gemm_ex = (decltype(gemm_ex))dlsym(lib, "cublasGemmEx");
        return create && destroy && set_stream && set_math && set_workspace && gemm_ex;
    }
};

}  // namespace

struct LlmeExecutor {
    int device = 0, sms = 148;
    std::map<std::string, void*> entry;
    std::map<std::string, std::string> chosen;
    std::string error;
    long long launches = 0;
    Blas blas;
    cublasHandle_t own_handle = nullptr;
    void* own_workspace = nullptr;

    void* find(const std::string& name) const {
        auto it = entry.find(name);
        return it == entry.end() ? nullptr : it->second;
    }
    void* find_hd(const char* name, int hd) const { return find(std::string(name) + "/" + std::to_string(hd)); }
    const std::string& choice(const char* op) { return chosen[op]; }
    int fail(const char* fmt, ...) {
        char buf[768];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        error = buf;
        return -1;
    }
    // a kernel library's launcher returned rc: count the launch, keep the library's message on failure
    int launched(int rc, const char* kernel) {
        ++launches;
        if (rc == 0) return 0;
        const char* msg = "";
        std::string base(kernel);
        if (auto* f = (LastErrorFn)find("error/" + base)) msg = f();
        if (!msg || !*msg) msg = rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "refused";
        error = std::string(kernel) + ": " + msg + " (code " + std::to_string(rc) + ")";
        return rc;
    }
};

struct LlmePlan {
    LlmeExecutor* ex;
    struct Record {
        int kind;
        std::vector<unsigned char> bytes;
    };
    std::vector<Record> records;
};

namespace {

size_t record_size(int kind) {
    switch (kind) {
        case LLME_OP_EMBEDDING: return sizeof(LlmeEmbeddingOp);
        case LLME_OP_RMSNORM: return sizeof(LlmeRmsNormOp);
        case LLME_OP_LINEAR: return sizeof(LlmeLinearOp);
        case LLME_OP_LINEAR_SWIGLU: return sizeof(LlmeLinearSwigluOp);
        case LLME_OP_QKV_POST: return sizeof(LlmeQkvPostOp);
        case LLME_OP_ATTEND: return sizeof(LlmeAttendOp);
        case LLME_OP_ATTENTION: return sizeof(LlmeAttentionOp);
        case LLME_OP_CALL: return sizeof(LlmeCallOp);
    }
    return 0;
}
const char* kind_name(int kind) {
    static const char* names[] = {"?", "embedding", "rmsnorm", "linear", "linear_swiglu", "qkv_post", "attend", "attention", "call"};
    return kind >= 1 && kind <= 8 ? names[kind] : names[0];
}

constexpr int SKINNY_ROWS = 16;      // most rows the weight-streaming product takes (gemm_skinny.cu)

// Whether a product of M tokens goes to the weight-streaming kernel when the choice is "auto".  That kernel has one
// block per group of 16 weight rows (8 gate + 8 up rows with the activation), two blocks resident per SM: it wins
// against the library's product for up to 8 tokens when its blocks fill their waves (4096 rows: 256 blocks for 296
// places, 5.5 TB/s on 4096 x 12288 against 3.1), and loses when a second wave is nearly empty (5120 rows: 320 blocks,
// 4.5 TB/s on 5120 x 17408 against 5.6) or when 9 to 16 tokens double the operands it re-reads from L2 per block.
// Where its waves of 296 are badly filled the kernel has a lighter form with three blocks per SM (444 places: 6.1 TB/s
// on 5120 x 17408 / 25600, against 5.7 to 5.9 for the library); 7,168 rows (448 groups) fit neither and go to the library.
bool skinny_pays(const LlmeExecutor& ex, int M, long long row_groups) {
    const long long places = 2LL * ex.sms, waves = (row_groups + places - 1) / places;
    // 9 to 16 tokens: only where the row groups are one well-filled round (4,096 rows: 256 groups).  There the kernel
    // takes 8.0 / 20.0 us for 4096 x 4096 / 4096 x 12288 against 10.6 / 21.7 us; with more row groups, each re-reading
    // the tokens' operands, the library is ahead (6144 x 4096: 14.3 against 12.9 us; 24576 x 4096: 39.5 against 37.7).
    if (M > 8) return row_groups <= places && 10 * row_groups >= 8 * places;
    if (4 * row_groups <= places) return true;          // a small product is bound by its launch, not by its waves
    if (10 * row_groups >= 8 * waves * places) return true;
    // the kernel's lighter form, three blocks per SM: 444 places a round (gemm_skinny.cu chooses it by the same figures)
    const long long places3 = 3LL * ex.sms, waves3 = (row_groups + places3 - 1) / places3;
    return 10 * row_groups >= 7 * waves3 * places3;
}

bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr) {
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0;
}

// Whether a plain product of this size goes to this package's tcgen05 kernel rather than to cuBLAS when the choice is
// "auto".  The kernel walks over whole tiles: 256 x 256 per pair of SMs from 129 tokens and 129 columns on (128 x 256
// or 128 x 128 per SM below that).  128 tiles on 74 pairs take the time of two waves for 1.73 waves of work, and there
// cuBLAS, which has the same tiles but more shapes to choose from, is 4 % faster (2,048 tokens of the 8B shape: 53 / 75
// / 153 us for the output, q|k|v and down products against 51 / 72 / 156 us; at 8,192 tokens, where the waves are
// full, 194 / 289 / 704 us against 259 / 301 / 806 us).  "auto" takes the kernel when its last wave is at least 90 % full.
bool tc_fills_its_waves(const LlmeExecutor& ex, int M, int N) {
    const bool pairs = M > 128 && N > 128;
    const long long tiles = pairs ? (long long)((M + 255) / 256) * ((N + 255) / 256)
                                  : (long long)((M + 127) / 128) * ((N + (N > 128 ? 255 : 127)) / (N > 128 ? 256 : 128));
    const long long walkers = pairs ? ex.sms / 2 : ex.sms;
    const long long waves = (tiles + walkers - 1) / walkers;
    return 10 * tiles >= 9 * waves * walkers;
}

int cublas_product(LlmeExecutor& ex, const LlmeStep& step, const void* x, long long ldx, const void* w, long long ldw, void* out,
                   long long ldo, int out_dtype, int M, int N, int K, cudaStream_t stream) {
    if (!ex.blas.load()) return ex.fail("linear: cuBLAS is not available in this process");
    cublasHandle_t h = (cublasHandle_t)step.blas;
    if (!h) {
        if (!ex.own_handle) {
            if (ex.blas.create(&ex.own_handle) != CUBLAS_STATUS_SUCCESS) return ex.fail("linear: cublasCreate failed");
            // a workspace of its own, so that a captured step never allocates
            if (cudaMalloc(&ex.own_workspace, 32u << 20) == cudaSuccess) ex.blas.set_workspace(ex.own_handle, ex.own_workspace, 32u << 20);
        }
        h = ex.own_handle;
        ex.blas.set_stream(h, stream);
    }
    // partial sums are never added in bfloat16: some shapes (a few tokens, an odd width) otherwise come out a
    // thousand rounding steps off
    ex.blas.set_math(h, (cublasMath_t)(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
    const float alpha = 1.0f, beta = 0.0f;
    const cublasStatus_t st = ex.blas.gemm_ex(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, (int)ldw, x, CUDA_R_16BF,
                                              (int)ldx, &beta, out, out_dtype == LLME_DT_F32 ? CUDA_R_32F : CUDA_R_16BF, (int)ldo,
                                              CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ex.blas.set_math(h, CUBLAS_DEFAULT_MATH);
    if (st != CUBLAS_STATUS_SUCCESS) return ex.fail("linear: cublasGemmEx failed with status %d for M=%d N=%d K=%d", (int)st, M, N, K);
    return 0;
}

int rows_of(const LlmeStep& s, int rows) { return rows == LLME_ROWS_LOGITS ? s.num_logit_rows : s.num_tokens; }

// out[M, n] = x[M, k] w[n, k]^T
int product(LlmeExecutor& ex, const LlmeStep& step, const void* x, long long ldx, int x_dtype, const void* w, long long ldw,
            int w_dtype, void* out, long long ldo, int out_dtype, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (x_dtype == LLME_DT_F32) {
        // the 32-bit path: this package's FMA kernel, never a reduced-precision mode
        auto* f = (GemmF32Fn)ex.find("gemm_f32");
        if (!f) return ex.fail("linear: no 32-bit product kernel is registered");
        if (out_dtype != LLME_DT_F32) return ex.fail("linear: a 32-bit product writes 32-bit output");
        return ex.launched(f((const float*)x, w, w_dtype, (float*)out, M, N, K, ldx, ldw, ldo, stream), "gemm_f32");
    }
    if (w_dtype != LLME_DT_BF16) return ex.fail("linear: bfloat16 inputs need bfloat16 weights");
    const std::string& how = ex.choice("linear");
    const bool operands_ok = K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && aligned16(x, w);
    const std::string& dec = ex.choice("linear.decode");
    if (how != "plain" && M <= SKINNY_ROWS && operands_ok && (dec == "skinny" || (dec == "auto" && skinny_pays(ex, M, (N + 15) / 16)))) {
        if (auto* f = (GemmBf16Fn)ex.find("gemm_skinny"))     // a handful of tokens: the weight-streaming kernel
            return ex.launched(f(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, stream), "gemm_skinny");
    }
    if (M >= 128 && operands_ok && N >= 8 && ldo >= N && (how == "tcgen05" || (how == "auto" && tc_fills_its_waves(ex, M, N)))) {
        if (auto* f = (GemmBf16Fn)ex.find("gemm_tc"))         // many tokens: the tcgen05 kernel
            return ex.launched(f(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, stream), "gemm_tc");
    }
    return cublas_product(ex, step, x, ldx, w, ldw, out, ldo, out_dtype, M, N, K, stream);
}

int op_embedding(LlmeExecutor& ex, const LlmeEmbeddingOp& o, const LlmeStep& s, cudaStream_t st) {
    auto* f = (EmbeddingFn)ex.find("embedding");
    if (!f) return ex.fail("no embedding kernel is registered");
    return ex.launched(f(s.token_ids, o.table, o.table_dtype, o.out, s.num_tokens, o.hidden, o.vocab, st), "embedding");
}

int op_rmsnorm(LlmeExecutor& ex, const LlmeRmsNormOp& o, const LlmeStep& s, cudaStream_t st) {
    auto* f = (RmsNormFn)ex.find("rmsnorm");
    if (!f) return ex.fail("no rmsnorm kernel is registered");
    const bool some = o.rows == LLME_ROWS_LOGITS;
    return ex.launched(f(o.x, o.delta, o.delta_dtype, o.gain, o.gain_dtype, o.out, o.out_dtype, some ? s.logit_rows : nullptr,
                         rows_of(s, o.rows), o.size, o.eps, st), "rmsnorm");
}

int op_linear(LlmeExecutor& ex, const LlmeLinearOp& o, const LlmeStep& s, cudaStream_t st) {
    if (rows_of(s, o.rows) <= 0) return 0;
    void* out = o.out ? o.out : (void*)s.logits;
    if (!out) return ex.fail("linear: the step has no place for its logits");
    return product(ex, s, o.x, o.ldx, o.x_dtype, o.w, o.ldw, o.w_dtype, out, o.out ? o.ldo : o.n, o.out ? o.out_dtype : LLME_DT_F32,
                   rows_of(s, o.rows), o.n, o.k, st);
}

int op_linear_swiglu(LlmeExecutor& ex, const LlmeLinearSwigluOp& o, const LlmeStep& s, cudaStream_t st) {
    const int M = s.num_tokens;
    if (M <= 0) return 0;
    const bool fused = ex.choice("linear_swiglu") == "fused" && ex.choice("linear") != "plain" && o.dtype == LLME_DT_BF16;
    const bool operands_ok = o.k % 8 == 0 && o.ldx % 8 == 0 && o.ldw % 8 == 0 && aligned16(o.x, o.w_gate_up);
    const std::string& dec = ex.choice("linear.decode");
    if (fused && M <= SKINNY_ROWS && operands_ok && (dec == "skinny" || (dec == "auto" && skinny_pays(ex, M, (o.inter + 7) / 8)))) {
        if (auto* f = (GemmBf16Fn)ex.find("gemm_skinny_swiglu"))
            return ex.launched(f(o.x, o.ldx, o.w_gate_up, o.ldw, o.out, LLME_DT_BF16, o.ldo, M, o.inter, o.k, st), "gemm_skinny_swiglu");
    }
    // the tcgen05 kernel with the activation in its epilogue: its tile is 128 tokens x (128 gate + 128 up) rows; like
    // the plain product it is taken only when its last wave is nearly full (at 256 / 512 / 1,024 tokens of the 8B
    // shape the library product with the activation kernel behind it is faster)
    const std::string& how = ex.choice("linear");
    if (fused && M >= 128 && operands_ok && o.inter >= 8 && o.ldo % 8 == 0 && aligned16(o.out) &&
        (how == "tcgen05" || (how == "auto" && tc_fills_its_waves(ex, M, 2 * o.inter)))) {
        if (auto* f = (GemmTcSwigluFn)ex.find("gemm_tc_swiglu"))
            return ex.launched(f(o.x, o.ldx, o.w_gate_up, o.ldw, o.out, o.ldo, M, o.inter, o.k, st), "gemm_tc_swiglu");
    }
    if (!o.gate_up) return ex.fail("linear_swiglu: the unfused form needs a workspace for gate|up");
    if (int rc = product(ex, s, o.x, o.ldx, o.dtype, o.w_gate_up, o.ldw, o.dtype, o.gate_up, 2LL * o.inter, o.dtype, M, 2 * o.inter, o.k, st))
        return rc;
    auto* f = (SwigluFn)ex.find("swiglu");
    if (!f) return ex.fail("no swiglu kernel is registered");
    if (o.ldo != o.inter) return ex.fail("linear_swiglu: the unfused form writes dense rows");
    return ex.launched(f(o.gate_up, o.dtype, o.out, o.dtype, M, o.inter, st), "swiglu");
}

int op_qkv_post(LlmeExecutor& ex, const LlmeQkvPostOp& o, const LlmeStep& s, cudaStream_t st) {
    auto* f = (QkvPostFn)ex.find("qkv_post");
    if (!f) return ex.fail("no qkv_post kernel is registered");
    if (!o.q_out && !o.k_out && !o.cache) return 0;
    if (o.cache && (o.group < 0 || o.group >= s.num_groups)) return ex.fail("qkv_post: the step has no cache group %d", o.group);
    LlmeQkvArgs a = {};
    a.q_in = o.q_in; a.k_in = o.k_in; a.v_in = o.v_in;
    a.q_stride = o.q_stride; a.k_stride = o.k_stride; a.v_stride = o.v_stride;
    a.q_gain = o.q_gain; a.k_gain = o.k_gain; a.gain_dtype = o.gain_dtype; a.eps = o.eps;
    a.cos_sin = o.cos_sin; a.positions = s.positions; a.max_positions = o.max_positions;
    a.q_out = o.q_out; a.k_out = o.k_out; a.cache = o.cache;
    a.slot_mapping = o.cache ? s.groups[o.group].slot_mapping : nullptr;
    a.tokens = s.num_tokens; a.nh = o.nh; a.nkv = o.nkv; a.hd = o.hd;
    a.page_size = o.cache ? s.groups[o.group].page_size : 0;
    return ex.launched(f(&a, o.in_dtype, o.out_dtype, st), "qkv_post");
}

// Blocks per (request, key/value head) of the decode attention, chosen by what the kernel's time is made of.  A block
// streams its share of the keys at a rate of its own (about 27 GB/s: its warps' loads wait for one another), and
// needs about 6 us beside that, the time of some 300 keys; the blocks run in rounds of as many as the GPU holds at
// once.  Up to 8 splits are one thread-block cluster and merge through shared memory; the blocks of a cluster must find
// room in one GPC together, so the GPU holds fewer clusters than its SMs hold blocks (71 of four blocks, not 74; 93 of
// three, not 98: the kernel library says how many), and one cluster too many is a second round: 9 requests of 8
// key/value heads in clusters of four took 33 us a layer against 17 us for 8 requests, 19 us in clusters of three.
// More than 8 splits (at most 16) merge through scratch memory, where the block that finishes last adds the parts up,
// the dearer the more there are (batch 1, 8,200 keys: 15.1 us with 16 splits, 16.9 us with 37, 23.2 us with 64).
// Measured choices this reproduces: batch 1 / 8 / 9 / 12 / 16 / 24 / 40 at 2,048 keys: 8 / 4 / 3 / 2 / 2 / 1 / 3 splits.
typedef int (*AttnClustersFn)(int);

int decode_splits(const LlmeExecutor& ex, int requests, int nh, int nkv, int hd, int window, long long max_ctx) {
    const long long span = window > 0 && window < max_ctx ? window : max_ctx;
    const long long groups = (span + 63) / 64 + (window > 0 ? 1 : 0);      // 64-key groups of the longest context
    const int G = nh / nkv;
    const long long units = (long long)requests * nkv * ((G + 15) / 16);     // (request, key/value head, 16 query heads)
    auto* room = (AttnClustersFn)ex.find_hd("attention_decode_clusters", hd);
    long long best = 1, best_cost = -1;
    for (long long s = 1; s <= 16 && s <= groups; ++s) {
        long long held = 2LL * ex.sms;                                       // blocks the GPU holds at once
        if (s >= 2 && s <= 8 && room) {
            const int clusters = room((int)s);
            if (clusters > 0) held = s * clusters;
        }
        const long long rounds = (units * s + held - 1) / held;
        const long long keys = (groups + s - 1) / s * 64;
        const long long fixed = s <= 8 ? 300 : 300 + 25 * s;
        const long long cost = rounds * (keys + fixed) * (100 + 8 * (rounds - 1));      // later rounds are never quite full
        if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
    }
    return (int)best;
}

bool fast_attention(LlmeExecutor& ex, int dtype, int hd) {
    return ex.choice("attention") == "fast" && dtype == LLME_DT_BF16 && hd % 16 == 0 && hd >= 16 && hd <= 128 &&
           ex.find_hd("attention_decode", hd) && ex.find_hd("attention_portion", hd);
}

void fill_fast(LlmeFastAttnArgs& a, const LlmeAttendOp& o, const LlmeStep& s, const int* rows, int n_rows, int splits) {
    const LlmeStepGroup& g = s.groups[o.group];
    a.q = o.q; a.cache = o.cache; a.out = o.out; a.rows = rows; a.cu_q_lens = s.cu_q_lens; a.ctx_lens = s.ctx_lens;
    a.table_rows = s.state_slots; a.block_tables = g.block_tables; a.scratch = o.scratch;
    a.max_blocks = g.max_blocks; a.n_rows = n_rows; a.nh = o.nh; a.nkv = o.nkv; a.page_size = g.page_size; a.window = o.window;
    a.splits = splits; a.scale = o.scale;
}

int scratch_check(LlmeExecutor& ex, const LlmeAttendOp& o, int n_rows, int splits) {
    if (splits <= 1) return 0;
    auto* need = (AttnScratchFn)ex.find_hd("attention_decode_scratch", o.hd);
    const long long floats = need ? need(n_rows, o.nh, splits) : 65536 + (long long)n_rows * o.nh * splits * (o.hd + 2);
    if (!o.scratch || floats > o.scratch_floats)
        return ex.fail("attention: %d requests x %d splits need %lld scratch values, the record has %lld", n_rows, splits, floats, o.scratch_floats);
    return 0;
}

int op_attend(LlmeExecutor& ex, const LlmeAttendOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    if (o.group < 0 || o.group >= s.num_groups) return ex.fail("attention: the step has no cache group %d", o.group);
    const LlmeStepGroup& g = s.groups[o.group];
    if (!fast_attention(ex, o.dtype, o.hd)) {
        auto* f = (AttnPlainFn)ex.find("attention_plain");
        if (!f) return ex.fail("no plain attention kernel is registered");
        LlmeAttnArgs a = {o.q, o.cache, o.out, s.positions, s.token_request, g.block_tables, g.max_blocks, s.num_tokens, o.nh, o.nkv,
                          o.hd, g.page_size, o.window, o.scale};
        return ex.launched(f(&a, o.dtype, st), "attention_plain");
    }
    if (s.num_portion > 0) {
        const int G = o.nh / o.nkv, ps = g.page_size;
        const bool pages_ok = ps >= 8 && (ps <= 128 ? 128 % ps == 0 : ps % 128 == 0);
        auto* tc = (AttnTcFn)ex.find_hd("attention_tc", o.hd);
        if (tc && ex.choice("attention.portion") == "tcgen05" && (o.hd == 64 || o.hd == 128) && pages_ok && 128 % G == 0) {
            LlmeTcAttnArgs a = {o.out, o.cache, s.portion_rows, s.cu_q_lens, s.ctx_lens, s.state_slots, g.block_tables, g.max_blocks,
                                s.num_portion, o.nh, o.nkv, ps, o.window, o.scale};
            if (int rc = ex.launched(tc(o.q, s.num_tokens, o.cache_rows, &a, s.max_portion_len, st), "attention_tc")) return rc;
        } else {
            LlmeFastAttnArgs a = {};
            fill_fast(a, o, s, s.portion_rows, s.num_portion, 1);
            auto* f = (AttnPortionFn)ex.find_hd("attention_portion", o.hd);
            if (int rc = ex.launched(f(&a, s.max_portion_len, st), "attention_portion")) return rc;
        }
    }
    if (s.num_decode > 0) {
        const int splits = decode_splits(ex, s.num_decode, o.nh, o.nkv, o.hd, o.window, s.max_decode_ctx);
        if (int rc = scratch_check(ex, o, s.num_decode, splits)) return rc;
        LlmeFastAttnArgs a = {};
        fill_fast(a, o, s, s.decode_rows, s.num_decode, splits);
        auto* f = (AttnDecodeFn)ex.find_hd("attention_decode", o.hd);
        if (int rc = ex.launched(f(&a, st), "attention_decode")) return rc;
    }
    return 0;
}

int op_attention(LlmeExecutor& ex, const LlmeAttentionOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    const LlmeAttendOp& at = o.attend;
    auto* fused = (AttnDecodeFusedFn)ex.find_hd("attention_decode_fused", at.hd);
    // a step of single new tokens: norm, rotation and cache write happen inside the attention kernel
    if (fused && fast_attention(ex, at.dtype, at.hd) && ex.choice("attention.decode") == "fused" && s.num_portion == 0 &&
        s.num_decode == s.num_tokens && at.hd % 4 == 0 && o.qkv_stride % 2 == 0 &&
        (((uintptr_t)o.qkv | (uintptr_t)o.post.q_gain | (uintptr_t)o.post.k_gain | (uintptr_t)o.post.cos_sin) & 7) == 0) {
        if (at.group < 0 || at.group >= s.num_groups) return ex.fail("attention: the step has no cache group %d", at.group);
        const int splits = decode_splits(ex, s.num_decode, at.nh, at.nkv, at.hd, at.window, s.max_decode_ctx);
        if (int rc = scratch_check(ex, at, s.num_decode, splits)) return rc;
        LlmeFastAttnArgs a = {};
        fill_fast(a, at, s, s.decode_rows, s.num_decode, splits);
        a.q = nullptr;
        LlmeFusedQkv f = {o.qkv, o.qkv_stride, o.post.q_gain, o.post.k_gain, o.post.gain_dtype, o.post.eps,
                          o.rotary ? o.post.cos_sin : nullptr, o.rotary ? o.post.max_positions : 0, o.post.cache ? 1 : 0};
        return ex.launched(fused(&a, &f, st), "attention_decode_fused");
    }
    if (int rc = op_qkv_post(ex, o.post, s, st)) return rc;
    return op_attend(ex, at, s, st);
}

const std::map<std::string, std::vector<std::string>>& variants() {
    static const std::map<std::string, std::vector<std::string>> v = {
        {"linear", {"auto", "tcgen05", "cublas", "plain"}},
        {"linear.decode", {"auto", "skinny", "cublas"}},
        {"linear_swiglu", {"fused", "unfused"}},
        {"attention", {"fast", "plain"}},
        {"attention.portion", {"tcgen05", "mma"}},
        {"attention.decode", {"fused", "split"}},
    };
    return v;
}

}  // namespace

// (every library of this package has this symbol; the executor's own messages belong to an executor: llme_executor_error)
LLME_EXPORT const char* llme_last_error() { return ""; }

LLME_EXPORT LlmeExecutor* llme_executor_create(int device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
        cudaGetLastError();
        return nullptr;
    }
    auto* ex = new LlmeExecutor();
    ex->device = device;
    ex->sms = sms;
    for (auto& kv : variants()) ex->chosen[kv.first] = kv.second[0];
    return ex;
}

LLME_EXPORT void llme_executor_destroy(LlmeExecutor* ex) {
    if (!ex) return;
    if (ex->own_handle) ex->blas.destroy(ex->own_handle);
    if (ex->own_workspace) cudaFree(ex->own_workspace);
    delete ex;
}

LLME_EXPORT int llme_executor_register(LlmeExecutor* ex, const char* name, void* entry_point) {
    if (!name || !entry_point) return ex->fail("register: a name and an entry point are needed");
    ex->entry[name] = entry_point;
    return 0;
}

LLME_EXPORT int llme_executor_choose(LlmeExecutor* ex, const char* op, const char* variant) {
    const std::string o = op ? op : "", v = variant ? variant : "";
    if (o == "*") {
        if (v != "fast" && v != "plain") return ex->fail("choose: all operations at once take 'fast' or 'plain', got '%s'", v.c_str());
        for (auto& kv : variants()) ex->chosen[kv.first] = kv.second[0];
        if (v == "plain") {
            ex->chosen["linear"] = "plain";
            ex->chosen["linear_swiglu"] = "unfused";
            ex->chosen["attention"] = "plain";
        }
        return 0;
    }
    auto it = variants().find(o);
    if (it == variants().end()) {
        std::string known;
        for (auto& kv : variants()) known += (known.empty() ? "" : ", ") + kv.first;
        return ex->fail("choose: no operation '%s'; known: %s", o.c_str(), known.c_str());
    }
    for (auto& k : it->second)
        if (k == v) {
            ex->chosen[o] = v;
            return 0;
        }
    std::string known;
    for (auto& k : it->second) known += (known.empty() ? "" : ", ") + k;
    return ex->fail("choose: operation '%s' has no variant '%s'; it has: %s", o.c_str(), v.c_str(), known.c_str());
}

LLME_EXPORT const char* llme_executor_chosen(LlmeExecutor* ex, const char* op) {
    auto it = ex->chosen.find(op ? op : "");
    return it == ex->chosen.end() ? "" : it->second.c_str();
}

LLME_EXPORT const char* llme_executor_error(LlmeExecutor* ex) { return ex->error.c_str(); }
LLME_EXPORT long long llme_executor_launches(LlmeExecutor* ex) { return ex->launches; }

LLME_EXPORT int llme_decode_splits(LlmeExecutor* ex, int requests, int nh, int nkv, int hd, int window, int max_ctx) {
    if (requests <= 0 || nh <= 0 || nkv <= 0 || nh % nkv) return 1;
    return decode_splits(*ex, requests, nh, nkv, hd, window, max_ctx);
}

LLME_EXPORT long long llme_attention_scratch_floats(LlmeExecutor* ex, int max_requests, int nh, int nkv, int hd) {
    if (max_requests <= 0 || nh <= 0 || nkv <= 0 || nh % nkv) return 0;
    long long most = 0;
    for (int n = 1; n <= max_requests; ++n) {
        const int splits = decode_splits(*ex, n, nh, nkv, hd, 0, 1LL << 30);
        const long long need = splits <= 1 ? 0 : 65536 + (long long)n * nh * splits * (hd + 2);
        if (need > most) most = need;
    }
    return most;
}

LLME_EXPORT LlmePlan* llme_plan_create(LlmeExecutor* ex) {
    auto* p = new LlmePlan();
    p->ex = ex;
    return p;
}
LLME_EXPORT void llme_plan_destroy(LlmePlan* p) { delete p; }
LLME_EXPORT int llme_plan_size(LlmePlan* p) { return (int)p->records.size(); }

LLME_EXPORT int llme_plan_add(LlmePlan* p, int kind, const void* record, size_t bytes) {
    const size_t want = record_size(kind);
    if (!want) return p->ex->fail("plan: unknown record kind %d", kind);
    if (!record || bytes != want) return p->ex->fail("plan: a %s record has %zu bytes, got %zu", kind_name(kind), want, bytes);
    LlmePlan::Record r;
    r.kind = kind;
    r.bytes.assign((const unsigned char*)record, (const unsigned char*)record + bytes);
    p->records.push_back(std::move(r));
    return (int)p->records.size() - 1;
}

LLME_EXPORT int llme_plan_run(LlmePlan* p, const LlmeStep* step, int first, int count, cudaStream_t stream) {
    LlmeExecutor& ex = *p->ex;
    if (!step) return ex.fail("run: no step");
    const int n = (int)p->records.size();
    if (first < 0 || first > n) return ex.fail("run: record %d of %d", first, n);
    const int last = count < 0 || first + count > n ? n : first + count;
    const LlmeStep& s = *step;
    for (int i = first; i < last; ++i) {
        const LlmePlan::Record& r = p->records[i];
        const void* b = r.bytes.data();
        int rc = 0;
        switch (r.kind) {
            case LLME_OP_EMBEDDING: rc = op_embedding(ex, *(const LlmeEmbeddingOp*)b, s, stream); break;
            case LLME_OP_RMSNORM: rc = op_rmsnorm(ex, *(const LlmeRmsNormOp*)b, s, stream); break;
            case LLME_OP_LINEAR: rc = op_linear(ex, *(const LlmeLinearOp*)b, s, stream); break;
            case LLME_OP_LINEAR_SWIGLU: rc = op_linear_swiglu(ex, *(const LlmeLinearSwigluOp*)b, s, stream); break;
            case LLME_OP_QKV_POST: rc = op_qkv_post(ex, *(const LlmeQkvPostOp*)b, s, stream); break;
            case LLME_OP_ATTEND: rc = op_attend(ex, *(const LlmeAttendOp*)b, s, stream); break;
            case LLME_OP_ATTENTION: rc = op_attention(ex, *(const LlmeAttentionOp*)b, s, stream); break;
            case LLME_OP_CALL: {
                const LlmeCallOp& c = *(const LlmeCallOp*)b;
                rc = c.fn ? c.fn(c.user, step, stream) : 0;
                if (rc) ex.error = "a called part reported an error";
                break;
            }
        }
        if (rc) {
            ex.error = "record " + std::to_string(i) + " (" + kind_name(r.kind) + "): " + ex.error;
            return rc;
        }
    }
    return 0;
}
