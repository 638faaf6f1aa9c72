// Command line in the manner of the reference's `generate` (examples/generate.cpp:57-65:
// `generate <model.gguf> [prompt] [max_tokens]`), on the C++ interface of this engine: no Python in the process.
//
//     generate <model_dir> [prompt] [max_tokens] [--dtype bfloat16|float32] [--no-greedy] [--temperature t] [--top-k k]
//              [--top-p p] [--repetition-penalty r] [--seed s] [--page-size n] [--max-cached-tokens n] [--kernels fast|plain]
//     generate --random-config config.json --seed 7 [prompt] [max_tokens] ...
//
// The engine works on token ids (it has no tokenizer): `prompt` is a list of ids separated by commas or spaces, default "1";
// several prompts are separated by ';' and run together through the continuous-batching scheduler.  Progress goes to
// stderr, one line of generated token ids per prompt to stdout, then "[Generated N tokens total]".
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "llmengine_b200/engine.h"

using namespace llmengine_b200;

static std::vector<std::vector<int>> parse_prompts(const std::string& text) {
    std::vector<std::vector<int>> out;
    std::stringstream all(text);
    std::string part;
    while (std::getline(all, part, ';')) {
        for (char& c : part)
            if (c == ',') c = ' ';
        std::stringstream ss(part);
        std::vector<int> ids;
        int v;
        while (ss >> v) ids.push_back(v);
        if (!ids.empty()) out.push_back(ids);
    }
    if (out.empty()) throw Error("the prompt holds no token ids");
    return out;
}

int main(int argc, char** argv) {
    EngineOptions opt;
    opt.max_num_seqs = 64;
    SamplingParams sp;
    std::vector<std::string> positional;
    std::string random_config;
    long long seed = 42;
    bool ignore_eos = false;
    try {
        for (int i = 1; i < argc; ++i) {
            const std::string a = argv[i];
            auto value = [&]() -> std::string {
                if (i + 1 >= argc) throw Error("option " + a + " needs a value");
                return argv[++i];
            };
            if (a == "--dtype") opt.dtype = value();
            else if (a == "--no-greedy") sp.greedy = false;
            else if (a == "--greedy") sp.greedy = true;
            else if (a == "--temperature") sp.temperature = (float)atof(value().c_str());
            else if (a == "--top-k") sp.top_k = atoi(value().c_str());
            else if (a == "--top-p") sp.top_p = (float)atof(value().c_str());
            else if (a == "--repetition-penalty") sp.repetition_penalty = (float)atof(value().c_str());
            else if (a == "--seed") seed = atoll(value().c_str());
            else if (a == "--page-size") opt.page_size = atoi(value().c_str());
            else if (a == "--max-cached-tokens") opt.max_cached_tokens = atoll(value().c_str());
            else if (a == "--max-num-seqs") opt.max_num_seqs = atoi(value().c_str());
            else if (a == "--max-num-batched-tokens") opt.max_num_batched_tokens = atoi(value().c_str());
            else if (a == "--prefill-chunk") opt.prefill_chunk = atoi(value().c_str());
            else if (a == "--kernels") opt.kernels = value();
            else if (a == "--kernel-dir") opt.kernel_dir = value();
            else if (a == "--random-config") random_config = value();
            else if (a == "--ignore-eos") ignore_eos = true;
            else if (a.rfind("--", 0) == 0) throw Error("unknown option " + a);
            else positional.push_back(a);
        }
        sp.seed = (unsigned long long)seed;
        opt.seed = sp.seed;
        ModelSource src;
        size_t next = 0;
        if (!random_config.empty()) {
            std::ifstream f(random_config);
            if (!f) throw Error(random_config + " cannot be read");
            std::stringstream ss;
            ss << f.rdbuf();
            src = ModelSource::random(ss.str(), seed);
        } else {
            if (positional.empty()) throw Error("usage: generate <model_dir> [prompt] [max_tokens] [options]");
            src = ModelSource::folder(positional[next++]);
        }
        const std::string prompt = next < positional.size() ? positional[next++] : "1";
        const int max_tokens = next < positional.size() ? atoi(positional[next++].c_str()) : 64;
        const auto prompts = parse_prompts(prompt);

        std::cerr << "[1/3] Loading model...\n";
        auto engine = Engine::create(opt, src);
        std::cerr << "[2/3] Generating (" << prompts.size() << " prompt(s), up to " << max_tokens << " tokens each)...\n";
        std::map<long long, size_t> which;
        std::vector<std::vector<int>> out(prompts.size());
        for (size_t i = 0; i < prompts.size(); ++i) {
            Request r;
            r.prompt_tokens = prompts[i];
            r.max_tokens = max_tokens;
            r.sampling = sp;
            r.eos_token_id = -1;
            (void)ignore_eos;                   // a model folder's own end token is not read by this example: ids only
            which[engine->submit(r)] = i;
        }
        while (!engine->idle())
            for (const TokenEvent& e : engine->step())
                if (e.token >= 0) out[which.at(e.id)].push_back(e.token);
        std::cerr << "[3/3] Done\n";
        size_t total = 0;
        for (auto& toks : out) {
            for (size_t i = 0; i < toks.size(); ++i) std::cout << (i ? " " : "") << toks[i];
            std::cout << "\n";
            total += toks.size();
        }
        std::cout << "\n[Generated " << total << " tokens total]\n";
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "generate: " << e.what() << "\n";
        return 1;
    }
}
