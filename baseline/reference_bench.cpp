// Times the reference project's own CUDA path on the benchmark's workload: its TransformerGraphBuilder graph
// (use_qk_norm on), its CudaExecutor and its contiguous CUDA KVCache, exactly as examples/generate_cuda.cpp
// wires them (src/runtime/executor.cpp:83-142, examples/generate_cuda.cpp:155-306), with random weights
// bound by name instead of a GGUF file (no tokenizer, no file).  Nothing of llmengine_b200 is on this path:
// the program links the reference's static libraries only.
//
// The reference serves one sequence per run, so a batch of B requests is B sequences, each with a cache of
// its own, decoded one after the other (the round-robin of examples/generate_paged.cpp:381-430); a "step"
// here is one new token for every sequence.  Weights are 32-bit: that is the reference's library-GEMM path
// (sgemm_nt -> cublasSgemm); bfloat16 weights would take its 16x16 plain kernel.
//
// usage: reference_bench L H nh nkv hd I V batch cached prefill_tokens steps warmup
// prints one line of JSON with the device-timed and the end-to-end decode time per step and the prefill time.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "minillm/minillm.h"

using namespace minillm;

static void die(const std::string& what) {
    std::cout << "{\"error\": \"" << what << "\"}" << std::endl;
    std::exit(3);
}
static void ok(const Status& st, const char* what) {
    if (!st.ok()) die(std::string(what) + ": " + st.to_string());
}
static void cu(cudaError_t e, const char* what) {
    if (e != cudaSuccess) die(std::string(what) + ": " + cudaGetErrorString(e));
}

struct Net {
    Graph graph;
    ValueId logits;
    RuntimeContext ctx;
    ValueId input;
};

int main(int argc, char** argv) {
    if (argc < 13) die("usage: reference_bench L H nh nkv hd I V batch cached prefill_tokens steps warmup");
    TransformerConfig cfg;
    cfg.num_layers = std::atoll(argv[1]);
    cfg.hidden_size = std::atoll(argv[2]);
    cfg.num_heads = std::atoll(argv[3]);
    cfg.num_kv_heads = std::atoll(argv[4]);
    cfg.head_dim = std::atoll(argv[5]);
    cfg.intermediate_size = std::atoll(argv[6]);
    cfg.vocab_size = std::atoll(argv[7]);
    const int batch = std::atoi(argv[8]), cached = std::atoi(argv[9]), prefill_tokens = std::atoi(argv[10]);
    const int steps = std::atoi(argv[11]), warmup = std::atoi(argv[12]);
    cfg.batch_size = 1;
    cfg.rms_norm_eps = 1e-6;
    cfg.rope_base = 1000000.0;
    cfg.use_qk_norm = true;
    cfg.dtype = DType::Float32;
    cfg.device = Device::cuda(0);
    if (cached != prefill_tokens) die("the cached tokens come from the prefill: both counts must be equal");
    cu(cudaSetDevice(0), "cudaSetDevice");

    // random weights on the device, one tensor per constant name, shared by the two graphs
    std::vector<std::pair<std::string, std::unique_ptr<Tensor>>> weights;
    std::mt19937 rng(1234);
    std::normal_distribution<float> normal(0.0f, 1.0f);
    const size_t block = size_t(1) << 22;
    std::vector<float> host_block(block), gains(block);
    for (auto& v : host_block) v = 0.02f * normal(rng);
    for (auto& v : gains) v = 1.0f + 0.1f * normal(rng);
    auto weight_for = [&](const Value& v) -> Tensor* {
        for (auto& w : weights)
            if (w.first == v.name) return w.second.get();
        auto t = std::make_unique<Tensor>(v.name, v.shape, DType::Float32, Device::cuda(0));
        ok(t->allocate_cuda(), "allocate weight");
        auto n = t->numel();
        if (!n) die("weight without a size");
        const bool gain = v.shape.rank() == 1;
        for (size_t at = 0; at < *n; at += block) {
            const size_t m = std::min(block, *n - at);
            // every block of a tensor starts elsewhere in the host pattern, so rows differ
            const size_t shift = (at / block * 7919) % (block / 2);
            const float* src = (gain ? gains.data() : host_block.data()) + (m + shift <= block ? shift : 0);
            cu(cudaMemcpy(static_cast<float*>(t->data()) + at, src, m * sizeof(float), cudaMemcpyHostToDevice), "copy weight");
        }
        weights.emplace_back(v.name, std::move(t));
        return weights.back().second.get();
    };
    auto build = [&](Net& net, int seq_len) {
        TransformerConfig c = cfg;
        c.seq_len = seq_len;
        GraphBuilder gb(net.graph);
        TransformerGraphBuilder tb(gb);
        auto out = tb.build_transformer(c);
        if (!out) die(out.error().to_string());
        net.logits = *out;
        ok(net.graph.validate(), "graph validation");
        for (auto& v : net.graph.values()) {
            if (v.kind == ValueKind::Constant) ok(net.ctx.bind(v.id, weight_for(v)), "bind weight");
        }
        auto plan = net.ctx.allocate_intermediates_planned(net.graph);
        if (!plan) die(plan.error().to_string());
        for (auto& v : net.graph.values()) {
            if (v.kind != ValueKind::Input) continue;
            auto t = std::make_unique<Tensor>(v.name, v.shape, v.dtype, v.device);
            ok(v.device.type == DeviceType::CUDA ? t->allocate_cuda() : t->allocate_cpu(), "allocate input");
            net.input = v.id;
            ok(net.ctx.emplace(v.id, std::move(t)), "bind input");
        }
    };
    Net prefill, decode;
    build(prefill, prefill_tokens);
    build(decode, 1);
    prefill.ctx.set_kv_cache_advance_tokens(prefill_tokens);
    decode.ctx.set_kv_cache_advance_tokens(1);

    KernelRegistry registry;
    register_cuda_kernels(registry);
    auto backend = std::make_shared<CudaBackend>();
    CudaExecutor prefill_exec(backend, registry), decode_exec(backend, registry);
    ok(prefill_exec.compile(prefill.graph), "compile prefill");
    ok(decode_exec.compile(decode.graph), "compile decode");

    const int max_seq = cached + warmup + steps + 8;
    std::vector<std::shared_ptr<KVCache>> caches;
    for (int b = 0; b < batch; ++b) {
        auto c = std::make_shared<KVCache>();
        ok(c->init_cuda(int(cfg.num_layers), int(cfg.num_kv_heads), int(cfg.head_dim), max_seq, 0), "KV cache");
        caches.push_back(c);
    }
    std::uniform_int_distribution<int> tok(0, int(cfg.vocab_size) - 1);
    std::vector<int32_t> prompt(prefill_tokens);
    cudaEvent_t e0, e1;
    cu(cudaEventCreate(&e0), "event");
    cu(cudaEventCreate(&e1), "event");

    // prefill every sequence with the reference's own prefill run; each is timed
    std::vector<float> prefill_ms;
    for (int b = 0; b < batch; ++b) {
        for (auto& t : prompt) t = tok(rng);
        prefill.ctx.set_kv_cache(caches[b]);
        cu(cudaMemcpy(prefill.ctx.get(prefill.input)->data(), prompt.data(), prompt.size() * 4, cudaMemcpyHostToDevice), "copy prompt");
        cu(cudaEventRecord(e0), "record");
        ok(prefill_exec.run(prefill.ctx), "prefill run");
        cu(cudaEventRecord(e1), "record");
        cu(cudaDeviceSynchronize(), "prefill sync");
        float ms = 0;
        cu(cudaEventElapsedTime(&ms, e0, e1), "elapsed");
        prefill_ms.push_back(ms);
        if (caches[b]->cached_len() != cached) die("the cache does not hold the prompt after the prefill");
    }
    std::sort(prefill_ms.begin(), prefill_ms.end());

    // decode: one token for every sequence per step, as generate_cuda.cpp does it for one sequence: token id
    // host -> device, run, synchronise, logits device -> host, greedy choice on the host
    std::vector<int32_t> next(batch);
    for (auto& t : next) t = tok(rng);
    std::vector<float> row(cfg.vocab_size);
    SamplingConfig sc;
    sc.greedy = true;
    Sampler sampler(42);
    std::vector<int32_t> history;
    size_t h2d = 0, d2h = 0;
    auto one_step = [&]() {
        for (int b = 0; b < batch; ++b) {
            decode.ctx.set_kv_cache(caches[b]);
            cu(cudaMemcpy(decode.ctx.get(decode.input)->data(), &next[b], 4, cudaMemcpyHostToDevice), "copy token");
            ok(decode_exec.run(decode.ctx), "decode run");
            cu(cudaDeviceSynchronize(), "decode sync");
            cu(cudaMemcpy(row.data(), decode.ctx.get(decode.logits)->data(), row.size() * 4, cudaMemcpyDeviceToHost), "copy logits");
            next[b] = sampler.sample(row.data(), int32_t(cfg.vocab_size), sc, history);
        }
        h2d = size_t(batch) * 4;
        d2h = size_t(batch) * row.size() * 4;
    };
    for (int i = 0; i < warmup; ++i) one_step();
    cu(cudaDeviceSynchronize(), "sync");
    const auto t0 = std::chrono::steady_clock::now();
    cu(cudaEventRecord(e0), "record");
    for (int i = 0; i < steps; ++i) one_step();
    cu(cudaEventRecord(e1), "record");
    cu(cudaDeviceSynchronize(), "sync");
    const auto t1 = std::chrono::steady_clock::now();
    float dev_ms = 0;
    cu(cudaEventElapsedTime(&dev_ms, e0, e1), "elapsed");
    const double host_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    std::printf("{\"decode_ms_per_step\": %.4f, \"e2e_ms_per_step\": %.4f, \"prefill_ms\": %.3f, \"prefill_ms_all\": [",
                dev_ms / steps, host_ms / steps, prefill_ms[prefill_ms.size() / 2]);
    for (size_t i = 0; i < prefill_ms.size(); ++i) std::printf("%s%.3f", i ? ", " : "", prefill_ms[i]);
    std::printf("], \"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu, \"cached_after\": %d}\n", h2d, d2h,
                caches[0]->cached_len());
    return 0;
}
