/* llmengine_b200: the engine as a C++ library.
 *
 *     #include "llmengine_b200/engine.h"
 *     using namespace llmengine_b200;
 *     auto engine = Engine::create(EngineOptions{}, ModelSource::folder("/models/qwen3"));
 *     std::vector<int> tokens = engine->generate({5, 17, 3}, 64, SamplingParams{});
 *
 * Everything between a request's token ids and its next token, without Python: the typed configuration read
 * from config.json and the registry from the architecture's name to its model, weights from safetensors by
 * tensor name (or from a seed), the paged cache with a block table per request, the step function for batches
 * that mix prompt portions with single decoded tokens, the continuous-batching scheduler and the sampler.  The
 * model's launch sequence is a plan of the step executor (executor.h), and the kernels are the libraries that
 * `python -m llmengine_b200.kernels.build` compiles for sm_100a: the same records and the same kernels that the
 * Python entry point runs.
 *
 * It stands where the reference has its umbrella header and executors (include/minillm/minillm.h:1-51,
 * include/minillm/runtime/executor.h:16-51): `Engine::create` for the reference's build-graph / load-weights /
 * compile sequence (examples/generate_cuda.cpp:155-245), `submit` / `step` for its ContinuousBatchScheduler driven
 * by hand (src/runtime/continuous_batch_scheduler.cpp:55-125), `generate` for the loop of examples/generate.cpp.
 *
 * This front serves the registered architecture with full causal attention in every layer; a configuration with
 * sliding-window layers or a `layer_order` of its own is refused here with a message (the Python front, which
 * keeps a page pool per kind of layer, serves those).  Errors are `llmengine_b200::Error` exceptions whose text
 * names the key, tensor or limit at fault.
 */
#pragma once

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace llmengine_b200 {

struct __attribute__((visibility("default"))) Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

/* Options of the engine itself; none is a property of the model.  Names and defaults of the Python EngineConfig. */
struct EngineOptions {
    std::string dtype = "bfloat16";        /* "bfloat16" or "float32" (a true 32-bit path: no reduced-precision product) */
    int page_size = 64;                    /* tokens per cache page */
    long long max_cached_tokens = 0;       /* cache pool in tokens; 0 = from free device memory */
    double gpu_memory_fraction = 0.85;
    int max_num_seqs = 64;                 /* requests alive at once */
    int max_num_batched_tokens = 2048;     /* token budget of one step */
    int prefill_chunk = 2048;              /* longest prompt portion of one request in one step */
    int max_model_len = 0;                 /* 0 = the model's max_position_embeddings */
    unsigned long long seed = 42;          /* default sampling seed */
    std::string kernels = "fast";          /* "fast" or "plain" */
    int device = 0;
    std::string kernel_dir;                /* folder with the compiled kernel libraries and their manifest.json;
                                              empty = the folder this library was loaded from */
};

struct ModelSource {
    std::string model_dir;                 /* a folder with config.json and model.safetensors (or shards + index) */
    std::string config_json;               /* or: the text of a config.json, with random weights from `random_seed` */
    long long random_seed = -1;
    static ModelSource folder(const std::string& dir) { ModelSource s; s.model_dir = dir; return s; }
    static ModelSource random(const std::string& config_text, long long seed) {
        ModelSource s; s.config_json = config_text; s.random_seed = seed; return s;
    }
};

/* Fields, defaults and order of application of the reference's SamplingConfig (include/minillm/runtime/sampler.h:9-20). */
struct SamplingParams {
    bool greedy = true;
    int top_k = 0;
    float top_p = 0.0f;
    float temperature = 1.0f;
    float repetition_penalty = 1.0f;
    unsigned long long seed = 42;
};

struct Request {
    std::vector<int> prompt_tokens;
    int max_tokens = 64;
    long long id = -1;                     /* -1 = the next free id */
    SamplingParams sampling;
    int eos_token_id = -1;                 /* -1 = none */
};

struct TokenEvent {
    long long id;
    int token;                             /* -1 when the request ended on its end token (which is not kept) */
    bool finished;
    std::string finish_reason;             /* "", "length", "eos" */
};

/* One request's share of a step of the low-level interface: its next tokens and the places among them whose logits
 * are wanted. */
struct StepEntry {
    long long request;
    std::vector<int> tokens;
    std::vector<int> want;
};

class __attribute__((visibility("default"))) Engine {
public:
    static std::unique_ptr<Engine> create(const EngineOptions& options, const ModelSource& source);
    virtual ~Engine() = default;

    /* Continuous batching: waiting -> prefilling -> decoding -> finished. */
    virtual long long submit(const Request& request) = 0;
    virtual std::vector<TokenEvent> step() = 0;            /* admit, run one batch, sample, finish and free */
    virtual bool idle() const = 0;                         /* nothing active, nothing waiting */
    /* One prompt to its end (EOS or max_tokens): the generated tokens. */
    virtual std::vector<int> generate(const std::vector<int>& prompt_tokens, int max_tokens,
                                      const SamplingParams& sampling = SamplingParams(), int eos_token_id = -1) = 0;

    /* The step function itself: the entries' tokens as one batch from the cache that earlier steps left; 32-bit
     * logits [wanted, vocab] in the order of the entries and of their `want` lists, copied to the host.  Requests in
     * `end` give back what they hold after the step.  A refused batch changes nothing. */
    virtual std::vector<float> step_batch(const std::vector<StepEntry>& entries, const std::vector<long long>& end) = 0;

    virtual int vocab_size() const = 0;
    virtual int free_pages() const = 0;
    virtual int num_pages() const = 0;
    virtual long long kernel_launches() const = 0;
    virtual std::string architecture() const = 0;
};

}  // namespace llmengine_b200
