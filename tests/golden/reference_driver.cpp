// Drives the reference project's own model code on the CPU: TransformerGraphBuilder::build_transformer
// (use_qk_norm on) + CpuExecutor over fp32 weights bound by name, once for the whole prompt without a
// cache and once in portions through its PagedKVCache.  Built and run only by make_golden.py; it links
// against the reference's static libraries and is not part of the engine.
//
// usage: reference_driver <in.bin> <out_whole.bin> <out_portions.bin> <page_size> <max_pages> <portion sizes...>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <vector>

#include "minillm/minillm.h"

using namespace minillm;

struct Loaded {
    TransformerConfig cfg;
    bool tied = false;
    std::vector<int32_t> tokens;
    std::map<std::string, std::unique_ptr<Tensor>> weights;
};

static Loaded load(const std::string& path) {
    Loaded m;
    std::ifstream f(path, std::ios::binary);
    int hdr[10];
    double d[2];
    f.read(reinterpret_cast<char*>(hdr), sizeof hdr);
    f.read(reinterpret_cast<char*>(d), sizeof d);
    m.cfg.num_layers = hdr[0]; m.cfg.hidden_size = hdr[1]; m.cfg.num_heads = hdr[2]; m.cfg.num_kv_heads = hdr[3];
    m.cfg.head_dim = hdr[4]; m.cfg.intermediate_size = hdr[5]; m.cfg.vocab_size = hdr[6]; m.tied = hdr[7] != 0;
    m.cfg.rope_base = d[0]; m.cfg.rms_norm_eps = d[1]; m.cfg.use_qk_norm = true; m.cfg.batch_size = 1;
    m.tokens.resize(hdr[8]);
    f.read(reinterpret_cast<char*>(m.tokens.data()), hdr[8] * 4);
    for (int i = 0; i < hdr[9]; ++i) {
        int n = 0;
        f.read(reinterpret_cast<char*>(&n), 4);
        std::string name(n, ' ');
        f.read(name.data(), n);
        int nd = 0;
        f.read(reinterpret_cast<char*>(&nd), 4);
        std::vector<int64_t> dims;
        size_t numel = 1;
        for (int j = 0; j < nd; ++j) { int x; f.read(reinterpret_cast<char*>(&x), 4); dims.push_back(x); numel *= x; }
        auto t = std::make_unique<Tensor>(name, Shape(dims), DType::Float32);
        t->allocate_cpu();
        f.read(reinterpret_cast<char*>(t->data()), numel * 4);
        m.weights[name] = std::move(t);
    }
    return m;
}

static void die(const std::string& what) { std::cerr << what << "\n"; std::exit(1); }

// n tokens starting at tokens[start]; paged == nullptr: whole prompt, no cache.
static std::vector<float> run(Loaded& m, int start, int n, PagedKVCache* paged, KernelRegistry& reg) {
    TransformerConfig cfg = m.cfg;
    cfg.seq_len = n;
    Graph g;
    GraphBuilder gb(g);
    TransformerGraphBuilder tb(gb);
    auto out = tb.build_transformer(cfg);
    if (!out) die(out.error().to_string());
    RuntimeContext ctx;
    for (auto& v : g.values()) {
        if (v.kind == ValueKind::Constant) {
            std::string name = v.name;
            if (name == "lm_head.weight" && m.tied) name = "tok_embeddings.weight";
            auto it = m.weights.find(name);
            if (it == m.weights.end()) die("missing " + name);
            if (!(it->second->shape() == v.shape)) die("shape mismatch " + name);
            ctx.bind(v.id, it->second.get());
        }
        if (v.kind == ValueKind::Input) {
            auto t = std::make_unique<Tensor>(v.name, v.shape, v.dtype);
            t->allocate_cpu();
            std::memcpy(t->data(), m.tokens.data() + start, n * 4);
            ctx.emplace(v.id, std::move(t));
        }
    }
    auto plan = ctx.allocate_intermediates_planned(g);
    if (!plan) die(plan.error().to_string());
    if (paged) { ctx.set_paged_kv_cache(paged); ctx.set_paged_sequence_id(0); }
    CpuExecutor ex(std::make_shared<CpuBackend>(), reg);
    auto st = ex.compile(g);
    if (!st.ok()) die(st.to_string());
    st = ex.run(ctx);
    if (!st.ok()) die(st.to_string());
    auto* t = ctx.get(*out);
    const float* p = reinterpret_cast<const float*>(t->data());
    return std::vector<float>(p, p + static_cast<size_t>(n) * m.cfg.vocab_size);
}

int main(int argc, char** argv) {
    if (argc < 7) die("usage: reference_driver in whole portions page_size max_pages sizes...");
    Loaded m = load(argv[1]);
    KernelRegistry reg;
    register_cpu_kernels(reg);
    const int T = static_cast<int>(m.tokens.size());
    auto whole = run(m, 0, T, nullptr, reg);
    std::ofstream(argv[2], std::ios::binary).write(reinterpret_cast<char*>(whole.data()), whole.size() * 4);
    std::vector<int> sizes;
    for (int i = 6; i < argc; ++i) sizes.push_back(std::atoi(argv[i]));
    PagedKVCache pc;
    auto st = pc.init(m.cfg.num_layers, m.cfg.num_kv_heads, m.cfg.head_dim, std::atoi(argv[4]), std::atoi(argv[5]));
    if (!st.ok()) die(st.to_string());
    pc.ensure_sequence(0);
    std::vector<float> portions;
    int pos = 0, i = 0;
    while (pos < T) {
        const int n = std::min(sizes[i++ % sizes.size()], T - pos);
        auto r = run(m, pos, n, &pc, reg);
        portions.insert(portions.end(), r.begin(), r.end());
        pos += n;
    }
    std::ofstream(argv[3], std::ios::binary).write(reinterpret_cast<char*>(portions.data()), portions.size() * 4);
    std::cout << "cached " << pc.sequence_length(0) << " tokens, " << pc.free_block_count() << " pages free\n";
    return 0;
}
