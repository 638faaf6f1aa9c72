// The engine as a C++ library (include/llmengine_b200/engine.h): configuration, weights, cache, step function,
// scheduler and sampler in native host code, over the step executor's plan and the compiled kernel libraries.
// No Python, no PyTorch.  The launch sequence is the executor's records (the ones the Python parts emit), the
// kernels are the same shared libraries; what this file restates in C++ is the host logic around them.
//
// Reference counterparts: the graph builder's layer list (src/model/transformer_graph_builder.cpp:129-294), the weight
// binding by name (src/io/gguf_weight_loader.cpp:195-240), PagedKVCache's free list and reservation
// (src/runtime/cache/paged_kv_cache.cpp:48-52,327-349), ContinuousBatchScheduler (src/runtime/continuous_batch_scheduler.cpp)
// and Sampler (src/runtime/sampler.cpp:11-141).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <math.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <deque>
#include <fstream>
#include <map>
#include <set>
#include <sstream>

#include "json.h"
#include "llmengine_b200/engine.h"
#include "llmengine_b200/executor.h"
#include "sha256.h"

namespace llmengine_b200 {
namespace {

#define CUDA_OK(call)                                                                                    \
    do {                                                                                                 \
        cudaError_t e__ = (call);                                                                        \
        if (e__ != cudaSuccess) throw Error(std::string(#call) + ": " + cudaGetErrorString(e__));       \
    } while (0)

std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw Error(path + " does not exist or cannot be read");
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}
bool exists(const std::string& path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0;
}

// ----------------------------------------------------------------------------- configuration and registry
struct ModelConfig {                      // the Qwen3 dense architecture's own config.json keys
    std::string architecture;
    int vocab_size = 0, hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0, num_attention_heads = 0,
        num_key_value_heads = 0, head_dim = 0, max_position_embeddings = 0, eos_token_id = -1;
    double rms_norm_eps = 0, rope_theta = 0;
    bool tie_word_embeddings = false;
};

int positive_int(const json::Value& d, const char* key) {
    const json::Value* v = d.find(key);
    if (!v || v->kind != json::Value::Number || v->num <= 0 || v->num != floor(v->num))
        throw Error(std::string("config key '") + key + "' must be a positive integer");
    return (int)v->num;
}

ModelConfig read_qwen3(const json::Value& d) {
    std::string missing;
    for (const char* k : {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                          "rms_norm_eps", "max_position_embeddings"})
        if (!d.find(k)) missing += std::string(missing.empty() ? "" : ", ") + k;
    if (!missing.empty()) throw Error("config.json lacks required key(s): " + missing);
    ModelConfig c;
    c.hidden_size = positive_int(d, "hidden_size");
    c.num_attention_heads = positive_int(d, "num_attention_heads");
    const json::Value* kv = d.find("num_key_value_heads");
    c.num_key_value_heads = kv && !kv->is_null() ? positive_int(d, "num_key_value_heads") : c.num_attention_heads;
    const json::Value* hd = d.find("head_dim");
    if (hd && !hd->is_null()) c.head_dim = positive_int(d, "head_dim");
    else if (c.hidden_size % c.num_attention_heads) throw Error("config has no 'head_dim' and hidden_size is not a multiple of num_attention_heads");
    else c.head_dim = c.hidden_size / c.num_attention_heads;
    if (c.num_attention_heads % c.num_key_value_heads)
        throw Error("num_attention_heads must be a multiple of num_key_value_heads");
    if (c.head_dim % 2) throw Error("head_dim must be even for rotary position encoding");
    if (const json::Value* a = d.find("hidden_act"))
        if (a->kind == json::Value::String && a->str != "silu") throw Error("hidden_act='" + a->str + "' is not supported: the feed-forward gate is SiLU");
    if (const json::Value* b = d.find("attention_bias"))
        if (b->kind == json::Value::Bool && b->b) throw Error("attention_bias=true is not supported: the projections have no bias");
    for (const char* name : {"rope_scaling", "rope_parameters"})
        if (const json::Value* r = d.find(name))
            if (r->kind == json::Value::Object) {
                const json::Value* t = r->find("rope_type");
                if (!t) t = r->find("type");
                if (t && t->kind == json::Value::String && t->str != "default")
                    throw Error(std::string(name) + " of type '" + t->str + "' is not supported: only plain rotary encoding");
            }
    const json::Value* theta = d.find("rope_theta");
    if (!theta)
        if (const json::Value* r = d.find("rope_parameters")) theta = r->find("rope_theta");
    if (!theta || theta->kind != json::Value::Number) throw Error("config.json lacks required key(s): rope_theta");
    c.rope_theta = theta->num;
    if (!(c.rope_theta > 0)) throw Error("rope_theta must be positive");
    c.num_hidden_layers = positive_int(d, "num_hidden_layers");
    c.vocab_size = positive_int(d, "vocab_size");
    c.intermediate_size = positive_int(d, "intermediate_size");
    c.max_position_embeddings = positive_int(d, "max_position_embeddings");
    c.rms_norm_eps = d.find("rms_norm_eps")->num;
    if (!(c.rms_norm_eps > 0)) throw Error("rms_norm_eps must be positive");
    if (const json::Value* t = d.find("tie_word_embeddings")) c.tie_word_embeddings = t->kind == json::Value::Bool && t->b;
    if (const json::Value* e = d.find("eos_token_id")) {
        if (e->kind == json::Value::Number) c.eos_token_id = (int)e->num;
        if (e->kind == json::Value::Array && !e->arr.empty() && e->arr[0].kind == json::Value::Number) c.eos_token_id = (int)e->arr[0].num;
    }
    if (const json::Value* w = d.find("use_sliding_window"))
        if (w->kind == json::Value::Bool && w->b)
            throw Error("this configuration has sliding-window layers: the C++ front keeps one page pool for layers that see "
                        "every key; use the Python entry point, which keeps a pool per kind of layer");
    if (d.find("layer_order")) throw Error("this configuration has a layer_order of its own: use the Python entry point");
    return c;
}

// architecture name (config.json: architectures[0]) -> how its configuration is read
typedef ModelConfig (*ConfigReader)(const json::Value&);
const std::map<std::string, ConfigReader>& architectures() {
    static const std::map<std::string, ConfigReader> m = {{"Qwen3ForCausalLM", read_qwen3}};
    return m;
}

ModelConfig read_config(const std::string& text) {
    json::Value d;
    try {
        d = json::parse(text);
    } catch (const std::exception& e) {
        throw Error(std::string("config.json is not valid JSON: ") + e.what());
    }
    const json::Value* a = d.find("architectures");
    if (!a || a->kind != json::Value::Array || a->arr.empty() || a->arr[0].kind != json::Value::String)
        throw Error("config.json lacks required key(s): architectures");
    auto it = architectures().find(a->arr[0].str);
    if (it == architectures().end()) {
        std::string known;
        for (auto& kv : architectures()) known += (known.empty() ? "" : ", ") + kv.first;
        throw Error("unknown architecture '" + a->arr[0].str + "'; registered: " + known);
    }
    ModelConfig c = it->second(d);
    c.architecture = a->arr[0].str;
    return c;
}

// ----------------------------------------------------------------------------- safetensors
struct FileTensor {
    std::string dtype;
    std::vector<long long> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
};

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path) : path_(path) {
        fd_ = open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw Error(path + ": cannot be opened");
        struct stat st;
        fstat(fd_, &st);
        size_ = (size_t)st.st_size;
        if (size_ < 8) throw Error(path + ": too short to hold a safetensors header");
        map_ = (const unsigned char*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (map_ == MAP_FAILED) throw Error(path + ": cannot be mapped");
        unsigned long long hlen = 0;
        memcpy(&hlen, map_, 8);
        if (hlen == 0 || 8 + hlen > size_) throw Error(path + ": header length " + std::to_string(hlen) + " does not fit a file of " + std::to_string(size_) + " bytes");
        json::Value header;
        try {
            header = json::Parser((const char*)map_ + 8, (size_t)hlen).parse();
        } catch (const std::exception& e) {
            throw Error(path + ": header is not valid JSON: " + e.what());
        }
        const size_t data_start = 8 + (size_t)hlen, data_size = size_ - data_start;
        for (auto& kv : header.obj) {
            if (kv.first == "__metadata__") continue;
            const json::Value *dt = kv.second.find("dtype"), *sh = kv.second.find("shape"), *off = kv.second.find("data_offsets");
            if (!dt || !sh || !off || off->arr.size() != 2) throw Error(path + ": malformed header entry for tensor '" + kv.first + "'");
            FileTensor t;
            t.dtype = dt->str;
            size_t numel = 1;
            for (auto& s : sh->arr) {
                t.shape.push_back((long long)s.num);
                numel *= (size_t)s.num;
            }
            const size_t item = t.dtype == "F32" ? 4 : (t.dtype == "BF16" || t.dtype == "F16") ? 2 : 0;
            if (!item) throw Error(path + ": tensor '" + kv.first + "' has unsupported dtype " + t.dtype);
            const size_t b = (size_t)off->arr[0].num, e = (size_t)off->arr[1].num;
            if (e < b || e > data_size || e - b != numel * item)
                throw Error(path + ": tensor '" + kv.first + "' has data offsets that do not match its size or lie outside the file");
            t.data = map_ + data_start + b;
            t.bytes = e - b;
            tensors[kv.first] = t;
        }
    }
    ~SafetensorsFile() {
        if (map_ && map_ != MAP_FAILED) munmap((void*)map_, size_);
        if (fd_ >= 0) close(fd_);
    }
    std::map<std::string, FileTensor> tensors;

private:
    std::string path_;
    int fd_ = -1;
    size_t size_ = 0;
    const unsigned char* map_ = nullptr;
};

float half_to_float(unsigned short h) {
    const unsigned sign = (h >> 15) & 1, exp = (h >> 10) & 31, man = h & 1023;
    float v;
    if (exp == 0) v = ldexpf((float)man, -24);
    else if (exp == 31) v = man ? NAN : INFINITY;
    else v = ldexpf((float)(man | 1024), (int)exp - 25);
    return sign ? -v : v;
}
unsigned short float_to_bf16(float f) {            // round to nearest even
    unsigned u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (unsigned short)((u >> 16) | 0x40);
    return (unsigned short)((u + 0x7fffu + ((u >> 16) & 1)) >> 16);
}
float bf16_to_float(unsigned short h) {
    unsigned u = (unsigned)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// ----------------------------------------------------------------------------- device tensors and kernel libraries
struct DeviceTensor {
    void* ptr = nullptr;
    long long rows = 0, cols = 0;
    int dtype = LLME_DT_F32;
    size_t bytes() const { return (size_t)rows * cols * (dtype == LLME_DT_F32 ? 4 : 2); }
};

struct Memory {                                  // everything the engine allocates on the device, freed together
    std::vector<void*> blocks;
    ~Memory() {
        for (void* p : blocks) cudaFree(p);
    }
    void* alloc(size_t bytes, bool zero = false) {
        void* p = nullptr;
        CUDA_OK(cudaMalloc(&p, bytes ? bytes : 16));
        blocks.push_back(p);
        if (zero) CUDA_OK(cudaMemset(p, 0, bytes));
        return p;
    }
    DeviceTensor tensor(long long rows, long long cols, int dtype, bool zero = false) {
        DeviceTensor t;
        t.rows = rows; t.cols = cols; t.dtype = dtype;
        t.ptr = alloc(t.bytes(), zero);
        return t;
    }
};

struct ExecutorApi {                             // the executor library's C interface, looked up at run time
    void* lib = nullptr;
    decltype(&llme_executor_create) create;
    decltype(&llme_executor_destroy) destroy;
    decltype(&llme_executor_register) reg;
    decltype(&llme_executor_choose) choose;
    decltype(&llme_executor_error) error;
    decltype(&llme_executor_launches) launches;
    decltype(&llme_attention_scratch_floats) scratch_floats;
    decltype(&llme_plan_create) plan_create;
    decltype(&llme_plan_destroy) plan_destroy;
    decltype(&llme_plan_add) plan_add;
    decltype(&llme_plan_run) plan_run;
};

class KernelLibraries {
public:
    explicit KernelLibraries(std::string dir) : dir_(std::move(dir)) {
        if (dir_.empty()) {
            Dl_info info;
            if (dladdr((void*)&read_qwen3, &info) && info.dli_fname) {
                dir_ = info.dli_fname;
                dir_ = dir_.substr(0, dir_.find_last_of('/'));
            }
        }
        const std::string path = dir_ + "/manifest.json";
        if (!exists(path))
            throw Error("no kernel manifest at " + path + ": compile the kernel libraries first (python -m llmengine_b200.kernels.build)");
        manifest_ = json::parse(read_file(path));
    }
    void* open(const std::string& key) {
        auto it = open_.find(key);
        if (it != open_.end()) return it->second;
        const json::Value* f = manifest_.find(key);
        if (!f || f->kind != json::Value::String || !exists(dir_ + "/" + f->str))
            throw Error("the kernel library '" + key + "' is not built in " + dir_ + ": run python -m llmengine_b200.kernels.build " + key);
        void* h = dlopen((dir_ + "/" + f->str).c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!h) throw Error("cannot load " + dir_ + "/" + f->str + ": " + dlerror());
        open_[key] = h;
        return h;
    }
    void* symbol(const std::string& key, const char* name) {
        void* s = dlsym(open(key), name);
        if (!s) throw Error("the kernel library '" + key + "' has no entry point " + name);
        return s;
    }

private:
    std::string dir_;
    json::Value manifest_;
    std::map<std::string, void*> open_;
};

// ----------------------------------------------------------------------------- the page cache
// Host-authoritative: a last-in-first-out free list that hands out page 0 first, a used bitmap that catches a double
// free, all-or-nothing reservation, one block table per request shared by all layers.
class PageCache {
public:
    PageCache(int page_size, long long max_cached_tokens, int max_requests, int max_request_len)
        : page_size(page_size), num_pages((int)((max_cached_tokens + page_size - 1) / page_size)),
          max_blocks((max_request_len + page_size - 1) / page_size), max_requests(max_requests), max_request_len(max_request_len) {
        for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);
        used_.assign(num_pages, false);
        for (int s = max_requests - 1; s >= 0; --s) free_slots_.push_back(s);
        tables.assign((size_t)max_requests * max_blocks, -1);
    }
    struct Held {
        int slot = 0;
        int length = 0;
        std::vector<int> blocks;
        int committed = 0;
    };
    bool has(long long id) const { return requests.count(id) != 0; }
    int free_pages() const { return (int)free_.size(); }
    Held& add(long long id) {
        if (has(id)) throw Error("request " + std::to_string(id) + " is already live");
        if (free_slots_.empty()) throw Error("all " + std::to_string(max_requests) + " request slots are in use");
        Held h;
        h.slot = free_slots_.back();
        free_slots_.pop_back();
        return requests[id] = h;
    }
    void forget(long long id) {                       // undo `add` for a request that never ran
        free_slots_.push_back(requests.at(id).slot);
        requests.erase(id);
    }
    bool reserve(long long id, int new_length) {      // all or nothing
        Held& h = requests.at(id);
        const int need = (new_length + page_size - 1) / page_size - (int)h.blocks.size();
        if (need <= 0) return true;
        if (need > (int)free_.size()) return false;
        for (int i = 0; i < need; ++i) {
            const int p = free_.back();
            free_.pop_back();
            used_[p] = true;
            tables[(size_t)h.slot * max_blocks + h.blocks.size()] = p;
            h.blocks.push_back(p);
        }
        dirty = true;
        return true;
    }
    void shrink(long long id, size_t blocks) {        // take back the newest pages (a refused batch)
        Held& h = requests.at(id);
        while (h.blocks.size() > blocks) {
            const int p = h.blocks.back();
            h.blocks.pop_back();
            used_[p] = false;
            free_.push_back(p);
            tables[(size_t)h.slot * max_blocks + h.blocks.size()] = -1;
        }
        dirty = true;
    }
    void free_request(long long id) {
        auto it = requests.find(id);
        if (it == requests.end()) throw Error("request " + std::to_string(id) + " is not live");
        Held& h = it->second;
        for (size_t b = 0; b < h.blocks.size(); ++b) {
            const int p = h.blocks[b];
            if (p < 0 || p >= num_pages || !used_[p]) throw Error("page " + std::to_string(p) + " is freed but is not in use");
            used_[p] = false;
            free_.push_back(p);
            tables[(size_t)h.slot * max_blocks + b] = -1;
        }
        committed_ -= h.committed;
        free_slots_.push_back(h.slot);
        requests.erase(it);
        dirty = true;
    }
    // admission control: promise the pages a request can ever need, or nothing
    bool try_commit(long long id, int total_tokens) {
        const int pages = (total_tokens + page_size - 1) / page_size;
        if (committed_ + pages > num_pages) return false;
        committed_ += pages;
        requests.at(id).committed = pages;
        return true;
    }
    bool fits_at_all(int total_tokens) const {
        return total_tokens <= max_request_len && (total_tokens + page_size - 1) / page_size <= num_pages;
    }
    const int page_size, num_pages, max_blocks, max_requests, max_request_len;
    std::map<long long, Held> requests;
    std::vector<int> tables;                          // [max_requests, max_blocks], -1 where no page is held
    bool dirty = true;

private:
    std::vector<int> free_, free_slots_;
    std::vector<bool> used_;
    int committed_ = 0;
};

// ----------------------------------------------------------------------------- sampling
float uniform_draw(unsigned long long seed, unsigned long long draw) {        // sampling/sampler.py:uniform
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + (draw + 1) * 0xBF58476D1CE4E5B9ull;
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(((double)(z >> 40) + 0.5) / 16777216.0);
}

struct SampleArgs {
    const float* logits; long long ld;
    int rows, vocab;
    const int* greedy; const float* temperature; const int* top_k; const float* top_p; const float* u;
    int* out;
};
typedef int (*SampleFn)(const SampleArgs*, cudaStream_t);
typedef int (*PenaltyFn)(float*, long long, const int*, const int*, const int*, const float*, int, int, cudaStream_t);
typedef int (*RandomFillFn)(void*, int, unsigned long long, long long, long long, float, float, int, cudaStream_t);

// ----------------------------------------------------------------------------- the engine
enum class Phase { Waiting, Prefilling, Decoding, Finished };

struct Sequence {
    long long id = 0;
    std::vector<int> prompt, generated;
    int max_tokens = 0, prefilled = 0, eos = -1;
    SamplingParams sampling;
    Phase phase = Phase::Waiting;
    std::string finish_reason;
    std::map<int, int> counts;                        // prompt + generated, for the repetition penalty
};

class EngineImpl final : public Engine {
public:
    EngineImpl(const EngineOptions& o, const ModelSource& src) : opt_(o), libs_(o.kernel_dir) {
        if (opt_.dtype == "bf16") opt_.dtype = "bfloat16";
        if (opt_.dtype == "fp32" || opt_.dtype == "f32") opt_.dtype = "float32";
        if (opt_.dtype != "bfloat16" && opt_.dtype != "float32") throw Error("dtype must be bfloat16 or float32, got '" + opt_.dtype + "'");
        if (opt_.page_size <= 0 || opt_.page_size > 256) throw Error("page_size must be in 1..256");
        if (opt_.max_num_seqs <= 0 || opt_.max_num_batched_tokens <= 0 || opt_.prefill_chunk <= 0)
            throw Error("max_num_seqs, max_num_batched_tokens and prefill_chunk must be positive");
        if (opt_.max_num_batched_tokens < opt_.max_num_seqs)
            throw Error("max_num_batched_tokens must be at least max_num_seqs: every decoding request needs one token a step");
        dt_ = opt_.dtype == "bfloat16" ? LLME_DT_BF16 : LLME_DT_F32;
        CUDA_OK(cudaSetDevice(opt_.device));
        CUDA_OK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        const bool folder = !src.model_dir.empty();
        if (!folder && (src.config_json.empty() || src.random_seed < 0)) throw Error("a model needs a folder, or a configuration with a random seed");
        cfg_ = read_config(folder ? read_file(src.model_dir + "/config.json") : src.config_json);
        max_model_len_ = opt_.max_model_len > 0 ? std::min(opt_.max_model_len, cfg_.max_position_embeddings) : cfg_.max_position_embeddings;
        load_executor();
        load_weights(src);
        make_cache();
        make_workspace();
        make_plan();
        prefill_chunk_ = std::min(opt_.prefill_chunk, opt_.max_num_batched_tokens);
    }
    ~EngineImpl() override {
        if (plan_) x_.plan_destroy(plan_);
        if (ex_) x_.destroy(ex_);
        if (pinned_) cudaFreeHost(pinned_);
        if (stream_) cudaStreamDestroy(stream_);
    }

    // ------------------------------------------------------------------ public interface
    int vocab_size() const override { return cfg_.vocab_size; }
    int free_pages() const override { return cache_->free_pages(); }
    int num_pages() const override { return cache_->num_pages; }
    long long kernel_launches() const override { return x_.launches(ex_) + direct_launches_; }
    std::string architecture() const override { return cfg_.architecture; }
    bool idle() const override { return active_.empty() && waiting_.empty(); }

    long long submit(const Request& r) override {
        if (r.prompt_tokens.empty()) throw Error("a request must have at least one prompt token");
        if (r.max_tokens <= 0) throw Error("a request's max_tokens must be positive");
        for (int t : r.prompt_tokens)
            if (t < 0 || t >= cfg_.vocab_size) throw Error("token id " + std::to_string(t) + " is outside the vocabulary [0, " + std::to_string(cfg_.vocab_size) + ")");
        const int total = (int)r.prompt_tokens.size() + r.max_tokens;
        if (!cache_->fits_at_all(total))
            throw Error("the request needs " + std::to_string(total) + " tokens: more than the model's length limit " +
                        std::to_string(max_model_len_) + " or than the whole cache holds");
        long long id = r.id;
        if (id >= 0) {
            if (seqs_.count(id)) throw Error("request id is already in use: " + std::to_string(id));
            next_id_ = std::max(next_id_, id + 1);
        } else {
            id = next_id_++;
        }
        Sequence s;
        s.id = id;
        s.prompt = r.prompt_tokens;
        s.max_tokens = r.max_tokens;
        s.sampling = r.sampling;
        s.eos = r.eos_token_id;
        for (int t : s.prompt) ++s.counts[t];
        seqs_[id] = std::move(s);
        waiting_.push_back(id);
        return id;
    }

    std::vector<TokenEvent> step() override {
        // admit from the head of the queue while a batch place and the pages can be promised (head-of-line blocking)
        while (!waiting_.empty() && (int)active_.size() < opt_.max_num_seqs) {
            Sequence& s = seqs_.at(waiting_.front());
            cache_->add(s.id);
            if (!cache_->try_commit(s.id, (int)s.prompt.size() + s.max_tokens)) {
                cache_->forget(s.id);
                break;
            }
            s.phase = Phase::Prefilling;
            active_.push_back(s.id);
            waiting_.pop_front();
        }
        // the batch: one token for every decoding request, then prompt portions in admission order under the budget
        int budget = opt_.max_num_batched_tokens;
        std::vector<StepEntry> entries;
        std::vector<bool> samples;
        for (long long id : active_) {
            Sequence& s = seqs_.at(id);
            if (s.phase != Phase::Decoding) continue;
            entries.push_back({id, {s.generated.back()}, {0}});
            samples.push_back(true);
            --budget;
        }
        for (long long id : active_) {
            Sequence& s = seqs_.at(id);
            if (s.phase != Phase::Prefilling || budget <= 0) continue;
            const int left = (int)s.prompt.size() - s.prefilled, n = std::min({left, prefill_chunk_, budget});
            StepEntry e{id, std::vector<int>(s.prompt.begin() + s.prefilled, s.prompt.begin() + s.prefilled + n), {}};
            if (n == left) e.want = {n - 1};
            entries.push_back(std::move(e));
            samples.push_back(n == left);
            budget -= n;
        }
        std::vector<TokenEvent> events;
        if (entries.empty()) return events;
        const int rows = run(entries, {});
        std::vector<int> tokens = sample(entries, samples, rows);
        size_t k = 0;
        for (size_t i = 0; i < entries.size(); ++i) {
            Sequence& s = seqs_.at(entries[i].request);
            if (s.phase == Phase::Prefilling) {
                s.prefilled += (int)entries[i].tokens.size();
                if (s.prefilled >= (int)s.prompt.size()) s.phase = Phase::Decoding;
            }
            if (!samples[i]) continue;
            const int tok = tokens[k++];
            if (s.eos >= 0 && tok == s.eos) {        // the end token is not kept (examples/generate.cpp:334)
                s.finish_reason = "eos";
                s.phase = Phase::Finished;
                events.push_back({s.id, -1, true, "eos"});
                continue;
            }
            s.generated.push_back(tok);
            ++s.counts[tok];
            if ((int)s.generated.size() >= s.max_tokens) {
                s.finish_reason = "length";
                s.phase = Phase::Finished;
            }
            events.push_back({s.id, tok, s.phase == Phase::Finished, s.finish_reason});
        }
        // finished requests leave the batch and give back their pages and their slot at once
        for (size_t i = 0; i < active_.size();) {
            if (seqs_.at(active_[i]).phase == Phase::Finished) {
                cache_->free_request(active_[i]);
                finished_[active_[i]] = std::move(seqs_.at(active_[i]));
                seqs_.erase(active_[i]);
                active_.erase(active_.begin() + i);
            } else {
                ++i;
            }
        }
        return events;
    }

    std::vector<int> generate(const std::vector<int>& prompt, int max_tokens, const SamplingParams& sp, int eos) override {
        Request r;
        r.prompt_tokens = prompt;
        r.max_tokens = max_tokens;
        r.sampling = sp;
        r.eos_token_id = eos >= 0 ? eos : -1;
        const long long id = submit(r);
        while (!finished_.count(id)) step();
        std::vector<int> out = std::move(finished_.at(id).generated);
        finished_.erase(id);
        return out;
    }

    std::vector<float> step_batch(const std::vector<StepEntry>& entries, const std::vector<long long>& end) override {
        const int rows = run(entries, end);
        std::vector<float> host((size_t)rows * cfg_.vocab_size);
        if (rows) CUDA_OK(cudaMemcpyAsync(host.data(), logits_.ptr, host.size() * 4, cudaMemcpyDeviceToHost, stream_));
        CUDA_OK(cudaStreamSynchronize(stream_));
        return host;
    }

private:
    // ------------------------------------------------------------------ set-up
    void load_executor() {
        x_.lib = libs_.open("executor");
#define SYM(field, name) x_.field = (decltype(x_.field))libs_.symbol("executor", name)
        SYM(create, "llme_executor_create"); SYM(destroy, "llme_executor_destroy"); SYM(reg, "llme_executor_register");
        SYM(choose, "llme_executor_choose"); SYM(error, "llme_executor_error"); SYM(launches, "llme_executor_launches");
        SYM(scratch_floats, "llme_attention_scratch_floats"); SYM(plan_create, "llme_plan_create");
        SYM(plan_destroy, "llme_plan_destroy"); SYM(plan_add, "llme_plan_add"); SYM(plan_run, "llme_plan_run");
#undef SYM
        ex_ = x_.create(opt_.device);
        if (!ex_) throw Error("the step executor cannot use device " + std::to_string(opt_.device));
        if (x_.choose(ex_, "*", opt_.kernels.c_str())) throw Error(x_.error(ex_));
        auto reg = [&](const std::string& lib, const char* entry, const char* symbol) {
            x_.reg(ex_, entry, libs_.symbol(lib, symbol));
            std::string base(entry);
            base = "error/" + base.substr(0, base.find('/'));
            x_.reg(ex_, base.c_str(), libs_.symbol(lib, "llme_last_error"));
        };
        reg("elementwise", "embedding", "llme_embedding");
        reg("elementwise", "rmsnorm", "llme_rmsnorm");
        reg("elementwise", "qkv_post", "llme_qkv_post");
        reg("elementwise", "swiglu", "llme_swiglu");
        const std::string hd = std::to_string(cfg_.head_dim);
        const bool fast_attn = dt_ == LLME_DT_BF16 && opt_.kernels == "fast" && cfg_.head_dim % 16 == 0 && cfg_.head_dim >= 16 && cfg_.head_dim <= 128;
        if (dt_ == LLME_DT_F32) {
            reg("gemm_f32", "gemm_f32", "llme_gemm_nt_f32");
        } else if (opt_.kernels == "fast") {
            reg("gemm_skinny", "gemm_skinny", "llme_gemm_skinny_bf16");
            reg("gemm_skinny", "gemm_skinny_swiglu", "llme_gemm_skinny_swiglu_bf16");
            reg("gemm_tcgen05", "gemm_tc", "llme_gemm_tc_bf16");
            reg("gemm_tcgen05", "gemm_tc_swiglu", "llme_gemm_tc_swiglu_bf16");
        }
        if (fast_attn) {
            const std::string lib = "attention_fast@HEAD_DIM=" + hd;
            reg(lib, ("attention_portion/" + hd).c_str(), "llme_attention_portion");
            reg(lib, ("attention_decode/" + hd).c_str(), "llme_attention_decode");
            reg(lib, ("attention_decode_fused/" + hd).c_str(), "llme_attention_decode_fused");
            reg(lib, ("attention_decode_scratch/" + hd).c_str(), "llme_attention_decode_scratch_floats");
            reg(lib, ("attention_decode_clusters/" + hd).c_str(), "llme_attention_decode_clusters");
            if (cfg_.head_dim == 64 || cfg_.head_dim == 128) reg("attention_tc@HEAD_DIM=" + hd, ("attention_tc/" + hd).c_str(), "llme_attention_tc");
        } else {
            reg("attention_plain", "attention_plain", "llme_attention_plain");
        }
        sample_fn_ = (SampleFn)libs_.symbol("sampling", "llme_sample");
        penalty_fn_ = (PenaltyFn)libs_.symbol("sampling", "llme_repetition_penalty");
    }

    // The model's tensors by checkpoint name: what must be in the file, with its shape and whether it is a matrix
    // (stored in the compute type) or a gain vector (32-bit in the file stays 32-bit).
    struct Wanted {
        std::vector<long long> shape;
        bool matrix;
    };
    std::map<std::string, Wanted> wanted() const {
        const ModelConfig& c = cfg_;
        const long long H = c.hidden_size, I = c.intermediate_size, V = c.vocab_size, hd = c.head_dim;
        const long long qs = (long long)c.num_attention_heads * hd, kvs = (long long)c.num_key_value_heads * hd;
        std::map<std::string, Wanted> w;
        w["model.embed_tokens.weight"] = {{V, H}, true};
        for (int l = 0; l < c.num_hidden_layers; ++l) {
            const std::string p = "model.layers." + std::to_string(l) + ".";
            w[p + "input_layernorm.weight"] = {{H}, false};
            w[p + "self_attn.q_proj.weight"] = {{qs, H}, true};
            w[p + "self_attn.k_proj.weight"] = {{kvs, H}, true};
            w[p + "self_attn.v_proj.weight"] = {{kvs, H}, true};
            w[p + "self_attn.o_proj.weight"] = {{H, qs}, true};
            w[p + "self_attn.q_norm.weight"] = {{hd}, false};
            w[p + "self_attn.k_norm.weight"] = {{hd}, false};
            w[p + "post_attention_layernorm.weight"] = {{H}, false};
            w[p + "mlp.gate_proj.weight"] = {{I, H}, true};
            w[p + "mlp.up_proj.weight"] = {{I, H}, true};
            w[p + "mlp.down_proj.weight"] = {{H, I}, true};
        }
        w["model.norm.weight"] = {{H}, false};
        if (!c.tie_word_embeddings) w["lm_head.weight"] = {{V, H}, true};
        return w;
    }

    // names of the reference's graph and of its GGUF files for the same tensors (src/io/gguf_weight_loader.cpp:36-52,362-380)
    static std::string canonical(const std::string& name) {
        static const std::map<std::string, std::string> global = {
            {"tok_embeddings.weight", "model.embed_tokens.weight"}, {"token_embd.weight", "model.embed_tokens.weight"},
            {"output_norm.weight", "model.norm.weight"}, {"output.weight", "lm_head.weight"}};
        static const std::map<std::string, std::string> layer = {
            {"attn_norm", "input_layernorm"}, {"q_proj", "self_attn.q_proj"}, {"k_proj", "self_attn.k_proj"},
            {"v_proj", "self_attn.v_proj"}, {"o_proj", "self_attn.o_proj"}, {"q_norm", "self_attn.q_norm"},
            {"k_norm", "self_attn.k_norm"}, {"ffn_norm", "post_attention_layernorm"}, {"gate_proj", "mlp.gate_proj"},
            {"up_proj", "mlp.up_proj"}, {"down_proj", "mlp.down_proj"}, {"attn_q", "self_attn.q_proj"},
            {"attn_k", "self_attn.k_proj"}, {"attn_v", "self_attn.v_proj"}, {"attn_output", "self_attn.o_proj"},
            {"attn_q_norm", "self_attn.q_norm"}, {"attn_k_norm", "self_attn.k_norm"}, {"ffn_gate", "mlp.gate_proj"},
            {"ffn_up", "mlp.up_proj"}, {"ffn_down", "mlp.down_proj"}};
        auto g = global.find(name);
        if (g != global.end()) return g->second;
        for (const char* lead : {"layer_", "blk."}) {
            const size_t n = strlen(lead);
            if (name.compare(0, n, lead)) continue;
            const size_t dot = name.find('.', n);
            if (dot == std::string::npos) break;
            const std::string idx = name.substr(n, dot - n), tail = name.substr(dot + 1);
            if (idx.empty() || idx.find_first_not_of("0123456789") != std::string::npos)
                throw Error("tensor name '" + name + "': layer index '" + idx + "' is not a number");
            const size_t last = tail.rfind('.');
            if (last == std::string::npos) break;
            auto it = layer.find(tail.substr(0, last));
            if (it != layer.end()) return "model.layers." + std::to_string(atoi(idx.c_str())) + "." + it->second + tail.substr(last);
        }
        return name;
    }

    // one tensor of the file -> `rows` rows of a device tensor starting at row `at`, in the device tensor's type
    void upload(const FileTensor& t, DeviceTensor& dst, long long at) {
        size_t numel = 1;
        for (long long d : t.shape) numel *= (size_t)d;
        char* to = (char*)dst.ptr + (size_t)at * dst.cols * (dst.dtype == LLME_DT_F32 ? 4 : 2);
        if ((t.dtype == "BF16" && dst.dtype == LLME_DT_BF16) || (t.dtype == "F32" && dst.dtype == LLME_DT_F32)) {
            CUDA_OK(cudaMemcpy(to, t.data, t.bytes, cudaMemcpyHostToDevice));
            return;
        }
        if (dst.dtype == LLME_DT_F32) {                       // widened exactly
            std::vector<float> tmp(numel);
            const unsigned short* s = (const unsigned short*)t.data;
            for (size_t i = 0; i < numel; ++i) tmp[i] = t.dtype == "BF16" ? bf16_to_float(s[i]) : half_to_float(s[i]);
            CUDA_OK(cudaMemcpy(to, tmp.data(), numel * 4, cudaMemcpyHostToDevice));
        } else {                                              // rounded to nearest even
            std::vector<unsigned short> tmp(numel);
            for (size_t i = 0; i < numel; ++i)
                tmp[i] = float_to_bf16(t.dtype == "F32" ? ((const float*)t.data)[i] : half_to_float(((const unsigned short*)t.data)[i]));
            CUDA_OK(cudaMemcpy(to, tmp.data(), numel * 2, cudaMemcpyHostToDevice));
        }
    }

    struct LayerWeights {
        DeviceTensor qkv, o, gate_up, down, attn_norm, ffn_norm, q_norm, k_norm;
    };

    int vector_dtype(const std::string& file_dtype) const {
        // a gain vector stored in 32 bits stays so; 16-bit ones stay bfloat16 (float16 is widened); the 32-bit engine widens all
        return dt_ == LLME_DT_F32 ? LLME_DT_F32 : (file_dtype == "BF16" ? LLME_DT_BF16 : LLME_DT_F32);
    }

    void load_weights(const ModelSource& src) {
        const ModelConfig& c = cfg_;
        const long long H = c.hidden_size, I = c.intermediate_size, V = c.vocab_size, hd = c.head_dim;
        const long long qs = (long long)c.num_attention_heads * hd, kvs = (long long)c.num_key_value_heads * hd;
        const auto want = wanted();
        std::vector<std::unique_ptr<SafetensorsFile>> files;
        std::map<std::string, FileTensor> found;
        if (!src.model_dir.empty()) {
            std::vector<std::string> paths;
            if (exists(src.model_dir + "/model.safetensors")) {
                paths.push_back(src.model_dir + "/model.safetensors");
            } else if (exists(src.model_dir + "/model.safetensors.index.json")) {
                const json::Value idx = json::parse(read_file(src.model_dir + "/model.safetensors.index.json"));
                std::set<std::string> names;
                if (const json::Value* m = idx.find("weight_map"))
                    for (auto& kv : m->obj) names.insert(kv.second.str);
                for (auto& n : names) paths.push_back(src.model_dir + "/" + n);
            } else {
                throw Error(src.model_dir + ": neither model.safetensors nor model.safetensors.index.json found");
            }
            for (auto& p : paths) {
                files.emplace_back(new SafetensorsFile(p));
                for (auto& kv : files.back()->tensors) {
                    const std::string name = canonical(kv.first);
                    if (found.count(name)) throw Error("tensor '" + name + "' appears twice in " + src.model_dir);
                    found[name] = kv.second;
                }
            }
            // one error that lists everything wrong
            std::string missing, unexpected, wrong;
            int n_missing = 0, n_unexpected = 0, n_wrong = 0;
            for (auto& kv : want)
                if (!found.count(kv.first)) {
                    missing += (n_missing++ ? ", " : "") + kv.first;
                } else if (found[kv.first].shape != kv.second.shape) {
                    auto show = [](const std::vector<long long>& s) {
                        std::string o = "[";
                        for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + std::to_string(s[i]);
                        return o + "]";
                    };
                    wrong += std::string(n_wrong++ ? "; " : "") + kv.first + " is " + show(found[kv.first].shape) + ", expected " + show(kv.second.shape);
                }
            for (auto& kv : found)
                if (!want.count(kv.first)) {
                    if (kv.first == "lm_head.weight" && c.tie_word_embeddings) {
                        fprintf(stderr, "[llmengine_b200] lm_head.weight is tied to model.embed_tokens.weight: the file's copy is ignored\n");
                        continue;
                    }
                    unexpected += (n_unexpected++ ? ", " : "") + kv.first;
                }
            if (n_missing || n_unexpected || n_wrong) {
                std::string msg = "the weight file does not fit the model:";
                if (n_missing) msg += "\n  missing tensors (" + std::to_string(n_missing) + "): " + missing;
                if (n_unexpected) msg += "\n  unexpected tensors (" + std::to_string(n_unexpected) + "): " + unexpected;
                if (n_wrong) msg += "\n  wrong shapes (" + std::to_string(n_wrong) + "): " + wrong;
                throw Error(msg);
            }
        }
        RandomFillFn fill = src.model_dir.empty() ? (RandomFillFn)libs_.symbol("utility", "llme_random_fill") : nullptr;
        // a tensor (or several, stacked by rows: q|k|v, gate|up) from the file or from the seed
        auto make = [&](const std::vector<std::string>& names, long long cols, bool matrix) {
            long long rows = 0;
            for (auto& n : names) rows += want.at(n).shape[0];
            if (!matrix) rows = 1, cols = want.at(names[0]).shape[0];
            int dtype = matrix ? dt_ : vector_dtype(fill ? "BF16" : found.at(names[0]).dtype);
            DeviceTensor t = mem_.tensor(rows, cols, dtype);
            long long at = 0;
            for (auto& n : names) {
                const long long r = matrix ? want.at(n).shape[0] : 1;
                if (fill) {
                    // the values `make_random_model` writes for this seed (a bfloat16 file), as the loader would store them
                    char* to = (char*)t.ptr + (size_t)at * cols * (dtype == LLME_DT_F32 ? 4 : 2);
                    const int rc = fill(to, dtype, tensor_seed(src.random_seed, n), 0, r * cols, matrix ? 0.02f : 0.1f, matrix ? 0.0f : 1.0f,
                                        dtype == LLME_DT_F32 ? 1 : 0, stream_);
                    if (rc) throw Error("random weights: the generator kernel failed for " + n);
                    ++direct_launches_;
                } else {
                    upload(found.at(n), t, at);
                }
                at += r;
            }
            return t;
        };
        embedding_ = make({"model.embed_tokens.weight"}, H, true);
        layers_.resize(c.num_hidden_layers);
        for (int l = 0; l < c.num_hidden_layers; ++l) {
            const std::string p = "model.layers." + std::to_string(l) + ".";
            LayerWeights& w = layers_[l];
            w.attn_norm = make({p + "input_layernorm.weight"}, 0, false);
            w.qkv = make({p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"}, H, true);
            w.q_norm = make({p + "self_attn.q_norm.weight"}, 0, false);
            w.k_norm = make({p + "self_attn.k_norm.weight"}, 0, false);
            if (w.q_norm.dtype != w.k_norm.dtype) throw Error(p + "self_attn: the two QK-norm gains must be stored in one type");
            w.o = make({p + "self_attn.o_proj.weight"}, qs, true);
            w.ffn_norm = make({p + "post_attention_layernorm.weight"}, 0, false);
            w.gate_up = make({p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"}, H, true);
            w.down = make({p + "mlp.down_proj.weight"}, I, true);
        }
        final_norm_ = make({"model.norm.weight"}, 0, false);
        head_ = c.tie_word_embeddings ? embedding_ : make({"lm_head.weight"}, H, true);     // tied: stored once, used twice
        (void)V; (void)kvs;
        CUDA_OK(cudaStreamSynchronize(stream_));
    }

    void make_cache() {
        const ModelConfig& c = cfg_;
        const size_t item = dt_ == LLME_DT_BF16 ? 2 : 4;
        const size_t per_token = (size_t)c.num_hidden_layers * 2 * c.num_key_value_heads * c.head_dim * item;
        long long tokens = opt_.max_cached_tokens;
        if (tokens <= 0) {
            size_t free_b = 0, total_b = 0;
            CUDA_OK(cudaMemGetInfo(&free_b, &total_b));
            const double workspace = (double)opt_.max_num_batched_tokens * c.hidden_size * 64 + 2e9;
            const double usable = (double)free_b * opt_.gpu_memory_fraction - workspace;
            tokens = usable > 0 ? (long long)(usable / per_token) : 0;
            tokens = std::min(tokens, (long long)opt_.max_num_seqs * max_model_len_);
            if (tokens < opt_.page_size) throw Error("no device memory is left for the cache after the weights");
        }
        cache_.reset(new PageCache(opt_.page_size, tokens, opt_.max_num_seqs, max_model_len_));
        // one tensor per layer, [pages][K|V][kv heads][page_size][head_dim]
        for (int l = 0; l < c.num_hidden_layers; ++l)
            kv_.push_back(mem_.tensor((long long)cache_->num_pages * 2 * c.num_key_value_heads * opt_.page_size, c.head_dim, dt_, true));
        tables_dev_ = (int*)mem_.alloc((size_t)cache_->tables.size() * 4);
    }

    void make_workspace() {
        const ModelConfig& c = cfg_;
        const long long T = opt_.max_num_batched_tokens, R = opt_.max_num_seqs, H = c.hidden_size;
        const long long qs = (long long)c.num_attention_heads * c.head_dim, kvs = (long long)c.num_key_value_heads * c.head_dim;
        x_buf_ = mem_.tensor(T, H, LLME_DT_F32);
        normed_ = mem_.tensor(T, H, dt_);
        normed_rows_ = mem_.tensor(T, H, dt_);
        qkv_ = mem_.tensor(T, qs + 2 * kvs, dt_);
        q_ = mem_.tensor(T, qs, dt_);
        attn_out_ = mem_.tensor(T, qs, dt_);
        mixer_out_ = mem_.tensor(T, H, LLME_DT_F32);
        gate_up_ = mem_.tensor(T, 2LL * c.intermediate_size, dt_);
        act_ = mem_.tensor(T, c.intermediate_size, dt_);
        ffn_out_ = mem_.tensor(T, H, LLME_DT_F32);
        // logits only for the rows that are ever wanted at once: every decoding request, or every row of a low-level step
        logit_rows_cap_ = T;
        logits_ = DeviceTensor();
        scratch_floats_ = x_.scratch_floats(ex_, (int)R, c.num_attention_heads, c.num_key_value_heads, c.head_dim);
        scratch_ = scratch_floats_ > 0 ? (float*)mem_.alloc((size_t)scratch_floats_ * 4, true) : nullptr;
        // rotary table: the 32-bit angle the reference forms (32-bit power, 32-bit product), cosine and sine evaluated in
        // 64-bit and rounded once (src/runtime/kernels/cpu_kernels.cpp:302-336)
        const int half = c.head_dim / 2, P = c.max_position_embeddings;
        std::vector<float> table((size_t)P * c.head_dim);
        std::vector<float> inv(half);
        for (int d = 0; d < half; ++d) {
            const float expo = (-2.0f * (float)d) / (float)c.head_dim;
            inv[d] = (float)pow((double)(float)c.rope_theta, (double)expo);
        }
        for (int p = 0; p < P; ++p)
            for (int d = 0; d < half; ++d) {
                const float ang = (float)p * inv[d];
                table[(size_t)p * c.head_dim + d] = (float)cos((double)ang);
                table[(size_t)p * c.head_dim + half + d] = (float)sin((double)ang);
            }
        cos_sin_ = (float*)mem_.alloc(table.size() * 4);
        CUDA_OK(cudaMemcpy(cos_sin_, table.data(), table.size() * 4, cudaMemcpyHostToDevice));
        // step metadata: one pinned block, one device block, one copy per step
        const long long n = 5 * T + 6 * R + 1;
        meta_len_ = (size_t)n;
        CUDA_OK(cudaMallocHost(&pinned_, meta_len_ * 4));
        meta_dev_ = (int*)mem_.alloc(meta_len_ * 4, true);
        sample_host_.assign(6 * R, 0);
        sample_dev_ = (float*)mem_.alloc((size_t)6 * R * 4, true);
        sampled_dev_ = (int*)mem_.alloc((size_t)R * 4, true);
    }

    template <typename Op> void add(int kind, const Op& op) {
        if (x_.plan_add(plan_, kind, &op, sizeof op) < 0) throw Error(x_.error(ex_));
    }

    // The layer list of src/model/transformer_graph_builder.cpp:129-294 with QK norm on, as executor records: the
    // records the Python parts emit for the same configuration.
    void make_plan() {
        const ModelConfig& c = cfg_;
        const int H = c.hidden_size, hd = c.head_dim, nh = c.num_attention_heads, nkv = c.num_key_value_heads;
        const long long qs = (long long)nh * hd, kvs = (long long)nkv * hd;
        const float eps = (float)c.rms_norm_eps;
        plan_ = x_.plan_create(ex_);
        LlmeEmbeddingOp emb = {embedding_.ptr, embedding_.dtype, c.vocab_size, H, (float*)x_buf_.ptr};
        add(LLME_OP_EMBEDDING, emb);
        const void* delta = nullptr;
        const size_t item = dt_ == LLME_DT_BF16 ? 2 : 4;
        for (int l = 0; l < c.num_hidden_layers; ++l) {
            const LayerWeights& w = layers_[l];
            LlmeRmsNormOp n1 = {(float*)x_buf_.ptr, delta, LLME_DT_F32, w.attn_norm.ptr, w.attn_norm.dtype, normed_.ptr, dt_, H, eps, LLME_ROWS_TOKENS};
            add(LLME_OP_RMSNORM, n1);
            LlmeLinearOp pq = {normed_.ptr, H, dt_, w.qkv.ptr, H, dt_, qkv_.ptr, qs + 2 * kvs, dt_, (int)(qs + 2 * kvs), H, LLME_ROWS_TOKENS};
            add(LLME_OP_LINEAR, pq);
            LlmeAttentionOp at = {};
            at.post.q_in = qkv_.ptr;
            at.post.k_in = (char*)qkv_.ptr + qs * item;
            at.post.v_in = (char*)qkv_.ptr + (qs + kvs) * item;
            at.post.q_stride = at.post.k_stride = at.post.v_stride = qs + 2 * kvs;
            at.post.in_dtype = dt_;
            at.post.q_gain = w.q_norm.ptr; at.post.k_gain = w.k_norm.ptr; at.post.gain_dtype = w.q_norm.dtype; at.post.eps = eps;
            at.post.cos_sin = cos_sin_; at.post.max_positions = c.max_position_embeddings;
            at.post.q_out = q_.ptr; at.post.k_out = nullptr; at.post.out_dtype = dt_;
            at.post.cache = kv_[l].ptr; at.post.group = 0; at.post.nh = nh; at.post.nkv = nkv; at.post.hd = hd;
            at.attend.q = q_.ptr; at.attend.out = attn_out_.ptr; at.attend.dtype = dt_;
            at.attend.cache = kv_[l].ptr; at.attend.cache_rows = kv_[l].rows;
            at.attend.group = 0; at.attend.nh = nh; at.attend.nkv = nkv; at.attend.hd = hd; at.attend.window = 0;
            at.attend.scale = (float)(1.0 / sqrt((double)hd));
            at.attend.scratch = scratch_; at.attend.scratch_floats = scratch_floats_;
            at.qkv = qkv_.ptr; at.qkv_stride = qs + 2 * kvs; at.rotary = 1;
            add(LLME_OP_ATTENTION, at);
            LlmeLinearOp po = {attn_out_.ptr, qs, dt_, w.o.ptr, qs, dt_, mixer_out_.ptr, H, LLME_DT_F32, H, (int)qs, LLME_ROWS_TOKENS};
            add(LLME_OP_LINEAR, po);
            LlmeRmsNormOp n2 = {(float*)x_buf_.ptr, mixer_out_.ptr, LLME_DT_F32, w.ffn_norm.ptr, w.ffn_norm.dtype, normed_.ptr, dt_, H, eps, LLME_ROWS_TOKENS};
            add(LLME_OP_RMSNORM, n2);
            LlmeLinearSwigluOp gu = {normed_.ptr, H, dt_, w.gate_up.ptr, H, gate_up_.ptr, act_.ptr, c.intermediate_size, c.intermediate_size, H};
            add(LLME_OP_LINEAR_SWIGLU, gu);
            LlmeLinearOp pd = {act_.ptr, c.intermediate_size, dt_, w.down.ptr, c.intermediate_size, dt_, ffn_out_.ptr, H, LLME_DT_F32, H, c.intermediate_size, LLME_ROWS_TOKENS};
            add(LLME_OP_LINEAR, pd);
            delta = ffn_out_.ptr;
        }
        LlmeRmsNormOp nf = {(float*)x_buf_.ptr, delta, LLME_DT_F32, final_norm_.ptr, final_norm_.dtype, normed_rows_.ptr, dt_, H, eps, LLME_ROWS_LOGITS};
        add(LLME_OP_RMSNORM, nf);
        LlmeLinearOp ph = {normed_rows_.ptr, H, dt_, head_.ptr, H, dt_, nullptr, 0, LLME_DT_F32, c.vocab_size, H, LLME_ROWS_LOGITS};
        add(LLME_OP_LINEAR, ph);
    }

    // ------------------------------------------------------------------ the step function
    // Validates on the host (a refused batch changes nothing), reserves pages all or nothing, writes the step's metadata
    // into pinned memory (one copy), runs the plan, advances lengths once, frees ended requests.  Returns the number of
    // logit rows; the logits are in `logits_`.
    int run(const std::vector<StepEntry>& entries, const std::vector<long long>& end) {
        const int T_cap = opt_.max_num_batched_tokens, R_cap = opt_.max_num_seqs;
        std::set<long long> seen;
        long long total = 0, wanted = 0;
        for (auto& e : entries) {
            if (e.tokens.empty()) throw Error("request " + std::to_string(e.request) + ": an entry needs at least one token");
            if (!seen.insert(e.request).second) throw Error("request " + std::to_string(e.request) + " appears twice in one step");
            total += (long long)e.tokens.size();
            for (int t : e.tokens)
                if (t < 0 || t >= cfg_.vocab_size) throw Error("request " + std::to_string(e.request) + ": a token id is outside the vocabulary");
            std::set<int> places;
            for (int w : e.want) {
                if (w < 0 || w >= (int)e.tokens.size()) throw Error("request " + std::to_string(e.request) + ": wanted place " + std::to_string(w) + " is outside its tokens");
                if (!places.insert(w).second) throw Error("request " + std::to_string(e.request) + ": a place is wanted twice");
            }
            wanted += (long long)e.want.size();
        }
        for (long long r : end)
            if (!seen.count(r) && !cache_->has(r)) throw Error("request " + std::to_string(r) + " is ended but is not live");
        if (total > T_cap) throw Error("the step has " + std::to_string(total) + " tokens, the budget is " + std::to_string(T_cap));
        if ((int)entries.size() > R_cap) throw Error("the step has " + std::to_string(entries.size()) + " requests, the limit is " + std::to_string(R_cap));
        std::vector<int> starts;
        for (auto& e : entries) {
            const int s = cache_->has(e.request) ? cache_->requests.at(e.request).length : 0;
            if (s + (int)e.tokens.size() > max_model_len_)
                throw Error("request " + std::to_string(e.request) + " would reach " + std::to_string(s + e.tokens.size()) + " tokens, the model's limit is " + std::to_string(max_model_len_));
            starts.push_back(s);
        }
        // reserve: new requests and pages, undone together (last first) if anything is short
        std::vector<long long> created;
        std::vector<std::pair<long long, size_t>> grown;
        auto undo = [&]() {
            for (auto it = grown.rbegin(); it != grown.rend(); ++it) cache_->shrink(it->first, it->second);
            for (auto it = created.rbegin(); it != created.rend(); ++it) cache_->forget(*it);
        };
        for (size_t i = 0; i < entries.size(); ++i) {
            const StepEntry& e = entries[i];
            try {
                if (!cache_->has(e.request)) {
                    cache_->add(e.request);
                    created.push_back(e.request);
                }
            } catch (const Error& err) {
                undo();
                throw Error(std::string("the step does not fit the cache: ") + err.what());
            }
            grown.emplace_back(e.request, cache_->requests.at(e.request).blocks.size());
            if (!cache_->reserve(e.request, starts[i] + (int)e.tokens.size())) {
                undo();
                throw Error("the step does not fit the cache: request " + std::to_string(e.request) + " needs more pages than are free");
            }
        }
        const int T = (int)total, R = (int)entries.size(), NL = (int)wanted;
        if (R) {
            if (NL > 0 && (!logits_.ptr || logits_.rows < NL)) {
                // grown on demand (a decode step wants a row per request, a replayed trace every row of a prompt)
                logits_ = mem_.tensor(std::max<long long>(NL, std::min<long long>(R_cap, logit_rows_cap_)), cfg_.vocab_size, LLME_DT_F32);
            }
            // metadata layout: token_ids, positions, token_request, slot_mapping, logit_rows [T_cap each]; then
            // cu_q_lens [R_cap+1], ctx_lens, state_slots, first_portion, decode_rows, portion_rows [R_cap each]
            CUDA_OK(cudaStreamSynchronize(stream_));                 // the pinned block is free again (the last step has run)
            int* m = pinned_;
            int *tok = m, *pos = m + T_cap, *treq = m + 2 * T_cap, *slot = m + 3 * T_cap, *lrows = m + 4 * T_cap;
            int* cu = m + 5 * T_cap;
            int *ctx = cu + R_cap + 1, *slots = ctx + R_cap, *first = slots + R_cap, *dec = first + R_cap, *por = dec + R_cap;
            int a = 0, nl = 0, nd = 0, np = 0, max_portion = 0, max_decode_ctx = 0;
            cu[0] = 0;
            for (int r = 0; r < R; ++r) {
                const StepEntry& e = entries[r];
                const PageCache::Held& h = cache_->requests.at(e.request);
                const int n = (int)e.tokens.size(), s = starts[r];
                for (int i = 0; i < n; ++i) {
                    tok[a + i] = e.tokens[i];
                    pos[a + i] = s + i;
                    treq[a + i] = h.slot;
                    slot[a + i] = h.blocks[(s + i) / opt_.page_size] * opt_.page_size + (s + i) % opt_.page_size;
                }
                for (int w : e.want) lrows[nl++] = a + w;
                a += n;
                cu[r + 1] = a;
                ctx[r] = s + n;
                slots[r] = h.slot;
                first[r] = s == 0;
                if (n == 1) {
                    dec[nd++] = r;
                    max_decode_ctx = std::max(max_decode_ctx, s + 1);
                } else {
                    por[np++] = r;
                    max_portion = std::max(max_portion, n);
                }
            }
            CUDA_OK(cudaMemcpyAsync(meta_dev_, pinned_, meta_len_ * 4, cudaMemcpyHostToDevice, stream_));
            if (cache_->dirty) {
                CUDA_OK(cudaMemcpyAsync(tables_dev_, cache_->tables.data(), cache_->tables.size() * 4, cudaMemcpyHostToDevice, stream_));
                cache_->dirty = false;
            }
            LlmeStep st = {};
            st.num_tokens = T; st.num_requests = R; st.num_logit_rows = NL; st.num_decode = nd; st.num_portion = np;
            st.max_portion_len = max_portion; st.max_decode_ctx = max_decode_ctx;
            int* d = meta_dev_;
            st.token_ids = d; st.positions = d + T_cap; st.token_request = d + 2 * T_cap; st.logit_rows = d + 4 * T_cap;
            int* dcu = d + 5 * T_cap;
            st.cu_q_lens = dcu; st.ctx_lens = dcu + R_cap + 1; st.state_slots = dcu + 2 * R_cap + 1; st.first_portion = dcu + 3 * R_cap + 1;
            st.decode_rows = dcu + 4 * R_cap + 1; st.portion_rows = dcu + 5 * R_cap + 1;
            st.logits = (float*)logits_.ptr;
            st.blas = nullptr;
            st.num_groups = 1;
            st.groups[0].block_tables = tables_dev_;
            st.groups[0].slot_mapping = d + 3 * T_cap;
            st.groups[0].max_blocks = cache_->max_blocks;
            st.groups[0].page_size = opt_.page_size;
            st.groups[0].window = 0;
            if (x_.plan_run(plan_, &st, 0, -1, stream_)) {
                undo();
                throw Error(x_.error(ex_));
            }
            for (int r = 0; r < R; ++r) cache_->requests.at(entries[r].request).length = starts[r] + (int)entries[r].tokens.size();
        }
        for (long long r : end) cache_->free_request(r);
        return R ? NL : 0;
    }

    // ------------------------------------------------------------------ sampling
    std::vector<int> sample(const std::vector<StepEntry>& entries, const std::vector<bool>& samples, int rows) {
        std::vector<int> out;
        if (rows <= 0) return out;
        const int R = opt_.max_num_seqs;
        float* h = sample_host_.data();
        int* hi = (int*)h;
        std::vector<int> prow, ptok, pcount;
        int r = 0;
        for (size_t i = 0; i < entries.size(); ++i) {
            if (!samples[i]) continue;
            const Sequence& s = seqs_.at(entries[i].request);
            const SamplingParams& p = s.sampling;
            h[0 * R + r] = p.temperature;
            h[1 * R + r] = p.top_p;
            h[2 * R + r] = p.greedy ? 0.5f : uniform_draw(p.seed, (unsigned long long)s.generated.size());
            h[3 * R + r] = p.repetition_penalty;
            hi[4 * R + r] = p.greedy ? 1 : 0;
            hi[5 * R + r] = p.top_k;
            if (p.repetition_penalty != 1.0f)
                for (auto& kv : s.counts) {
                    prow.push_back(r);
                    ptok.push_back(kv.first);
                    pcount.push_back(kv.second);
                }
            ++r;
        }
        CUDA_OK(cudaMemcpyAsync(sample_dev_, h, (size_t)6 * R * 4, cudaMemcpyHostToDevice, stream_));
        if (!prow.empty()) {
            const size_t n = prow.size();
            std::vector<int> packed;
            packed.insert(packed.end(), prow.begin(), prow.end());
            packed.insert(packed.end(), ptok.begin(), ptok.end());
            packed.insert(packed.end(), pcount.begin(), pcount.end());
            if (packed.size() > penalty_cap_) {
                penalty_cap_ = packed.size() * 2;
                penalty_dev_ = (int*)mem_.alloc(penalty_cap_ * 4);
            }
            int* dev = penalty_dev_;
            CUDA_OK(cudaMemcpyAsync(dev, packed.data(), packed.size() * 4, cudaMemcpyHostToDevice, stream_));
            if (penalty_fn_((float*)logits_.ptr, cfg_.vocab_size, dev, dev + n, dev + 2 * n, sample_dev_ + 3 * R, (int)n, cfg_.vocab_size, stream_))
                throw Error("the repetition-penalty kernel failed");
            ++direct_launches_;
        }
        SampleArgs a = {(const float*)logits_.ptr, cfg_.vocab_size, rows, cfg_.vocab_size, (const int*)(sample_dev_ + 4 * R), sample_dev_,
                        (const int*)(sample_dev_ + 5 * R), sample_dev_ + R, sample_dev_ + 2 * R, sampled_dev_};
        if (sample_fn_(&a, stream_)) throw Error("the sampling kernel failed");
        ++direct_launches_;
        out.resize(rows);
        CUDA_OK(cudaMemcpyAsync(out.data(), sampled_dev_, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream_));
        CUDA_OK(cudaStreamSynchronize(stream_));
        return out;
    }

    EngineOptions opt_;
    KernelLibraries libs_;
    ModelConfig cfg_;
    ExecutorApi x_ = {};
    LlmeExecutor* ex_ = nullptr;
    LlmePlan* plan_ = nullptr;
    cudaStream_t stream_ = nullptr;
    Memory mem_;
    int dt_ = LLME_DT_BF16, max_model_len_ = 0, prefill_chunk_ = 0;
    DeviceTensor embedding_, head_, final_norm_;
    std::vector<LayerWeights> layers_;
    std::vector<DeviceTensor> kv_;
    std::unique_ptr<PageCache> cache_;
    int* tables_dev_ = nullptr;
    DeviceTensor x_buf_, normed_, normed_rows_, qkv_, q_, attn_out_, mixer_out_, gate_up_, act_, ffn_out_, logits_;
    long long logit_rows_cap_ = 0, scratch_floats_ = 0;
    float *scratch_ = nullptr, *cos_sin_ = nullptr;
    int *pinned_ = nullptr, *meta_dev_ = nullptr;
    size_t meta_len_ = 0;
    std::vector<float> sample_host_;
    float* sample_dev_ = nullptr;
    int* sampled_dev_ = nullptr;
    SampleFn sample_fn_ = nullptr;
    PenaltyFn penalty_fn_ = nullptr;
    long long direct_launches_ = 0;
    int* penalty_dev_ = nullptr;
    size_t penalty_cap_ = 0;
    // the scheduler's state
    std::map<long long, Sequence> seqs_, finished_;
    std::deque<long long> waiting_;
    std::vector<long long> active_;
    long long next_id_ = 0;
};

}  // namespace

__attribute__((visibility("default"))) std::unique_ptr<Engine> Engine::create(const EngineOptions& options, const ModelSource& source) {
    try {
        return std::unique_ptr<Engine>(new EngineImpl(options, source));
    } catch (const Error&) {
        throw;
    } catch (const std::exception& e) {
        throw Error(e.what());
    }
}

}  // namespace llmengine_b200

// every library of this package has this symbol
extern "C" __attribute__((visibility("default"))) const char* llme_last_error() { return ""; }
