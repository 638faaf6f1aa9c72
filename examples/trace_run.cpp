// Trace replay on the C++ interface: the protocol of bin/trace_run (one JSON object a line on standard input,
// `{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}`; `<out>/<step>.f32` with the
// logits at the wanted places; `done <step>` after every step), driven through Engine::step_batch: it samples nothing
// and has no forward pass, cache or loader of its own.
//
//     trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size P] [--max-requests R]
#include <sys/stat.h>

#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "json.h"
#include "llmengine_b200/engine.h"

using namespace llmengine_b200;

int main(int argc, char** argv) {
    std::string model, dtype, out;
    long long max_tokens = 0;
    int page = 64, max_requests = 8;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string a = argv[i], v = argv[i + 1];
        if (a == "--model") model = v;
        else if (a == "--dtype") dtype = v;
        else if (a == "--out") out = v;
        else if (a == "--max-tokens") max_tokens = atoll(v.c_str());
        else if (a == "--page-size") page = atoi(v.c_str());
        else if (a == "--max-requests") max_requests = atoi(v.c_str());
        else { std::cerr << "trace_run: unknown option " << a << "\n"; return 2; }
    }
    if (model.empty() || dtype.empty() || out.empty() || max_tokens <= 0) {
        std::cerr << "usage: trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N\n";
        return 2;
    }
    try {
        mkdir(out.c_str(), 0777);
        EngineOptions opt;
        opt.dtype = dtype;
        opt.page_size = page;
        const long long pool = std::max<long long>(page, (max_tokens + page - 1) / page * page);
        opt.max_cached_tokens = pool;
        opt.max_num_seqs = max_requests;
        opt.max_num_batched_tokens = (int)std::max<long long>(pool, max_requests);
        opt.prefill_chunk = opt.max_num_batched_tokens;
        auto engine = Engine::create(opt, ModelSource::folder(model));
        std::map<std::string, long long> ids;          // the trace's request names -> request numbers
        auto id_of = [&](const json::Value& v) {
            const std::string key = v.kind == json::Value::String ? v.str : std::to_string((long long)v.num);
            auto it = ids.find(key);
            if (it == ids.end()) it = ids.emplace(key, (long long)ids.size()).first;
            return it->second;
        };
        std::string line;
        while (std::getline(std::cin, line)) {
            if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
            json::Value rec;
            try {
                rec = json::parse(line);
            } catch (const std::exception& e) {
                std::cerr << "trace_run: bad input line: " << e.what() << "\n";
                return 2;
            }
            const json::Value* step = rec.find("step");
            if (!step) { std::cerr << "trace_run: bad input line: no step\n"; return 2; }
            std::vector<StepEntry> entries;
            std::vector<long long> end;
            if (const json::Value* es = rec.find("entries"))
                for (auto& e : es->arr) {
                    StepEntry se;
                    se.request = id_of(*e.find("id"));
                    for (auto& t : e.find("tokens")->arr) se.tokens.push_back((int)t.num);
                    if (const json::Value* w = e.find("want"))
                        for (auto& x : w->arr) se.want.push_back((int)x.num);
                    if (!se.tokens.empty()) entries.push_back(std::move(se));
                }
            if (const json::Value* en = rec.find("end"))
                for (auto& r : en->arr) end.push_back(id_of(r));
            std::vector<float> logits;
            try {
                logits = engine->step_batch(entries, end);
            } catch (const Error& e) {
                std::cerr << "trace_run: step " << (long long)step->num << " refused: " << e.what() << "\n";
                return 3;
            }
            if (!logits.empty()) {
                const std::string path = out + "/" + std::to_string((long long)step->num) + ".f32";
                FILE* f = fopen(path.c_str(), "wb");
                if (!f || fwrite(logits.data(), 4, logits.size(), f) != logits.size()) {
                    std::cerr << "trace_run: cannot write " << path << "\n";
                    return 1;
                }
                fclose(f);
            }
            std::cout << "done " << (long long)step->num << std::endl;
        }
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "trace_run: " << e.what() << "\n";
        return 1;
    }
}
