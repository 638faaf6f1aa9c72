/* llmengine_b200: the step executor.
 *
 * A model is flattened once, when it is loaded, into a *plan*: a list of operation records (embedding, norm,
 * matrix product, attention, ...), each holding the device pointers of its weights and of its places in the
 * step's workspace.  `llme_plan_run` then walks that list for one step: a batch of (request, its next tokens)
 * that may mix prompt portions with single decoded tokens, described by an `LlmeStep`.  The walk is native code:
 * per operation it decides which kernel serves the step's shape (the kernel registry below) and launches it on
 * the given stream; nothing is allocated and the host never waits for the device.
 *
 * The reference walks a graph of nodes and looks every kernel up per node and run
 * (src/runtime/executor.cpp:112-142, include/minillm/runtime/kernel_registry.h:18-35); the plan is the same
 * idea with the lookup done once and the shapes left open until the step.
 *
 * Kernels are not linked into this library.  Whoever loaded the kernel libraries registers their entry points
 * by name (`llme_executor_register`); an operation with several implementations (this package's tcgen05 or
 * mma.sync kernels, the plain 32-bit twins, the library product) is switched per operation with
 * `llme_executor_choose`, so that any fast kernel can be exchanged for its plain twin inside the whole model.
 *
 * An operation this library does not know is a `LLME_OP_CALL` record: a function pointer with a user value,
 * called in its turn with the step and the stream.  Parts written outside this package (also in Python) run
 * through it, and a new kernel family needs no change here.
 */
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLME_MAX_GROUPS 8

enum { LLME_DT_F32 = 0, LLME_DT_BF16 = 1 };

/* One cache group (layers whose caches grow and shrink together) as a step sees it. */
typedef struct LlmeStepGroup {
    const int* block_tables;   /* device [slots, max_blocks]; -1 where no page is held */
    const int* slot_mapping;   /* device [T]: page * page_size + place in page of each token; < 0 = not stored */
    int max_blocks, page_size, window;
} LlmeStepGroup;

/* One step.  Pointers are device memory and stay the same from step to step (a captured step is replayed with
 * new contents behind them); the counts are host values. */
typedef struct LlmeStep {
    int num_tokens, num_requests, num_logit_rows, num_decode, num_portion;
    int max_portion_len;       /* longest prompt portion of the step (requests with more than one token) */
    int max_decode_ctx;        /* longest context among the requests with exactly one token; for a step that is
                                  captured for replay: the longest context a replay may meet */
    const int* token_ids;      /* [T] */
    const int* positions;      /* [T] absolute position of each token in its request */
    const int* token_request;  /* [T] block-table row (state slot) of the token's request */
    const int* cu_q_lens;      /* [R+1] */
    const int* ctx_lens;       /* [R] cached length of each request after this step */
    const int* state_slots;    /* [R] */
    const int* first_portion;  /* [R] */
    const int* logit_rows;     /* [NL] token rows whose logits are wanted */
    const int* decode_rows;    /* [ND] batch rows of the requests with exactly one token */
    const int* portion_rows;   /* [NP] the others */
    float* logits;             /* [NL, vocab] output of the step */
    void* blas;                /* cublasHandle_t bound to `stream` by the caller, or NULL: the executor's own */
    int num_groups;
    LlmeStepGroup groups[LLME_MAX_GROUPS];
} LlmeStep;

typedef int (*LlmeCallFn)(void* user, const LlmeStep* step, cudaStream_t stream);

enum LlmeOpKind {
    LLME_OP_EMBEDDING = 1, LLME_OP_RMSNORM, LLME_OP_LINEAR, LLME_OP_LINEAR_SWIGLU, LLME_OP_QKV_POST, LLME_OP_ATTEND,
    LLME_OP_ATTENTION, LLME_OP_CALL
};

enum { LLME_ROWS_TOKENS = 0, LLME_ROWS_LOGITS = 1 };

typedef struct LlmeEmbeddingOp {
    const void* table; int table_dtype, vocab, hidden;
    float* out;                /* [T, hidden] */
} LlmeEmbeddingOp;

typedef struct LlmeRmsNormOp {
    float* x;                  /* [T, size] the residual stream, updated in place when delta is given */
    const void* delta; int delta_dtype;
    const void* gain; int gain_dtype;
    void* out; int out_dtype;
    int size; float eps;
    int rows;                  /* LLME_ROWS_TOKENS: every row; LLME_ROWS_LOGITS: the step's logit rows only */
} LlmeRmsNormOp;

typedef struct LlmeLinearOp {
    const void* x; long long ldx; int x_dtype;
    const void* w; long long ldw; int w_dtype;
    void* out; long long ldo; int out_dtype;   /* out NULL: the step's logits, row stride n */
    int n, k;
    int rows;                  /* LLME_ROWS_TOKENS or LLME_ROWS_LOGITS */
} LlmeLinearOp;

typedef struct LlmeLinearSwigluOp {
    const void* x; long long ldx; int dtype;
    const void* w_gate_up; long long ldw;      /* [2 * inter, k]: gate rows, then up rows */
    void* gate_up;             /* [T, 2 * inter] workspace for the unfused form */
    void* out; long long ldo;  /* [T, inter] */
    int inter, k;
} LlmeLinearSwigluOp;

/* QK norm, rotation and cache write as a step of its own (the parts of it that are given). */
typedef struct LlmeQkvPostOp {
    const void* q_in; const void* k_in; const void* v_in; long long q_stride, k_stride, v_stride; int in_dtype;
    const void* q_gain; const void* k_gain; int gain_dtype; float eps;
    const float* cos_sin; int max_positions;
    void* q_out; void* k_out; int out_dtype;
    void* cache; int group;    /* cache NULL: nothing is stored */
    int nh, nkv, hd;
} LlmeQkvPostOp;

/* Attention of every token of the step over its request's cache, queries finished. */
typedef struct LlmeAttendOp {
    const void* q; void* out; int dtype;
    const void* cache; long long cache_rows;   /* pages * 2 * nkv * page_size */
    int group, nh, nkv, hd, window; float scale;
    float* scratch; long long scratch_floats;
} LlmeAttendOp;

/* The mixer's middle in one record: raw q|k|v projections in, attention output out.  A step of single new tokens
 * goes to the decode kernel that norms, rotates and stores by itself; any other step to QKV_POST then ATTEND. */
typedef struct LlmeAttentionOp {
    LlmeQkvPostOp post;        /* q_out is the finished-queries workspace */
    LlmeAttendOp attend;
    const void* qkv; long long qkv_stride;
    int rotary;                /* 1: cos_sin table; 0: no position encoding at all */
} LlmeAttentionOp;

typedef struct LlmeCallOp { LlmeCallFn fn; void* user; } LlmeCallOp;

typedef struct LlmeExecutor LlmeExecutor;
typedef struct LlmePlan LlmePlan;

LlmeExecutor* llme_executor_create(int device);
void llme_executor_destroy(LlmeExecutor*);
/* Entry points of the kernel libraries, by name: "embedding", "rmsnorm", "qkv_post", "swiglu", "gemm_f32",
 * "gemm_skinny", "gemm_skinny_swiglu", "gemm_tc", "gemm_tc_swiglu", "attention_plain", and per head size
 * "attention_portion/<hd>", "attention_decode/<hd>", "attention_decode_fused/<hd>", "attention_tc/<hd>". */
int llme_executor_register(LlmeExecutor*, const char* name, void* entry_point);
/* Which implementation an operation takes.  Operations and their variants:
 *   "linear":            "auto" | "tcgen05" | "cublas" | "plain"   (bfloat16 products of 128 tokens or more / all)
 *   "linear.decode":     "auto" | "skinny" | "cublas"               (bfloat16 products of up to 16 tokens)
 *   "linear_swiglu":     "fused" | "unfused"
 *   "attention.portion": "tcgen05" | "mma" | "plain"
 *   "attention.decode":  "fused" | "split" | "plain"
 *   "*":                 "fast" | "plain"                           (all of the above at once)
 * Returns 0, or -1 for an unknown operation or variant. */
int llme_executor_choose(LlmeExecutor*, const char* op, const char* variant);
const char* llme_executor_chosen(LlmeExecutor*, const char* op);
const char* llme_executor_error(LlmeExecutor*);
long long llme_executor_launches(LlmeExecutor*);      /* kernels of this package launched so far */
/* Scratch floats an attention record needs for steps of up to `max_requests` single tokens. */
long long llme_attention_scratch_floats(LlmeExecutor*, int max_requests, int nh, int nkv, int hd);
/* Blocks per (request, key/value head) that the decode attention would use. */
int llme_decode_splits(LlmeExecutor*, int requests, int nh, int nkv, int hd, int window, int max_ctx);

LlmePlan* llme_plan_create(LlmeExecutor*);
void llme_plan_destroy(LlmePlan*);
/* Appends a record (copied); `kind` says which of the structs above `record` is.  Returns its index, or -1. */
int llme_plan_add(LlmePlan*, int kind, const void* record, size_t bytes);
int llme_plan_size(LlmePlan*);
/* Runs records [first, first + count) (count < 0: to the end) for one step.  0, or the failing record's code;
 * `llme_executor_error` then names the record and the reason. */
int llme_plan_run(LlmePlan*, const LlmeStep* step, int first, int count, cudaStream_t stream);

#ifdef __cplusplus
}

#include <stdexcept>
#include <string>

namespace llmengine_b200 {

/* Thin C++ face of the functions above: owning handles, errors as exceptions. */
class Executor {
public:
    explicit Executor(int device = 0) : h_(llme_executor_create(device)) {
        if (!h_) throw std::runtime_error("llmengine_b200: cannot create an executor on this device");
    }
    ~Executor() { llme_executor_destroy(h_); }
    Executor(const Executor&) = delete;
    Executor& operator=(const Executor&) = delete;
    void register_kernel(const std::string& name, void* entry) {
        if (llme_executor_register(h_, name.c_str(), entry)) throw std::invalid_argument(error());
    }
    void choose(const std::string& op, const std::string& variant) {
        if (llme_executor_choose(h_, op.c_str(), variant.c_str())) throw std::invalid_argument(error());
    }
    std::string error() const { return llme_executor_error(h_); }
    LlmeExecutor* handle() const { return h_; }

private:
    LlmeExecutor* h_;
};

class Plan {
public:
    explicit Plan(Executor& ex) : ex_(ex), h_(llme_plan_create(ex.handle())) {}
    ~Plan() { llme_plan_destroy(h_); }
    Plan(const Plan&) = delete;
    Plan& operator=(const Plan&) = delete;
    int add(const LlmeEmbeddingOp& r) { return add(LLME_OP_EMBEDDING, &r, sizeof r); }
    int add(const LlmeRmsNormOp& r) { return add(LLME_OP_RMSNORM, &r, sizeof r); }
    int add(const LlmeLinearOp& r) { return add(LLME_OP_LINEAR, &r, sizeof r); }
    int add(const LlmeLinearSwigluOp& r) { return add(LLME_OP_LINEAR_SWIGLU, &r, sizeof r); }
    int add(const LlmeQkvPostOp& r) { return add(LLME_OP_QKV_POST, &r, sizeof r); }
    int add(const LlmeAttendOp& r) { return add(LLME_OP_ATTEND, &r, sizeof r); }
    int add(const LlmeAttentionOp& r) { return add(LLME_OP_ATTENTION, &r, sizeof r); }
    int add(const LlmeCallOp& r) { return add(LLME_OP_CALL, &r, sizeof r); }
    /* One step through the whole plan; throws with the failing record's message. */
    void run(const LlmeStep& step, cudaStream_t stream) {
        if (llme_plan_run(h_, &step, 0, -1, stream)) throw std::runtime_error(ex_.error());
    }

private:
    int add(int kind, const void* r, size_t n) {
        const int i = llme_plan_add(h_, kind, r, n);
        if (i < 0) throw std::invalid_argument(ex_.error());
        return i;
    }
    Executor& ex_;
    LlmePlan* h_;
};

}  // namespace llmengine_b200
#endif
