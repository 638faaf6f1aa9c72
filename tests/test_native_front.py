"""The engine's C++ interface (include/llmengine_b200/engine.h) through its command line (examples/generate.cpp,
bin/generate_native): a process without Python loads a model folder (or makes random weights from a seed), runs the
scheduler, the step function and the sampler in native code over the same executor records and kernels, and must
generate the tokens that the Python entry point generates."""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import make_model_dir, random_ids
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OPTIONS = ["--page-size", "16", "--max-cached-tokens", "1024", "--max-num-seqs", "4", "--max-num-batched-tokens", "64",
           "--prefill-chunk", "48"]


def _native(args, expect=0):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate_native"), *args], capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == expect, p.stderr[-3000:]
    return p


def _tokens(p, n):
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert lines[-1].startswith("[Generated ")
    return [[int(x) for x in l.split()] for l in lines[:n]]


def _python(model, prompts, dtype, sp=None, max_tokens=10, **more):
    from llmengine_b200 import LLM
    llm = LLM(model, dtype=dtype, page_size=16, max_cached_tokens=1024, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=48, pipeline_decode=False, **more)
    return [o.token_ids for o in llm.generate(prompts, sp, max_tokens=max_tokens, eos_token_id=None)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_D], ids=["A", "B", "D"])
def test_the_cpp_front_generates_the_tokens_of_the_python_front(tmp_path, cfg, dtype):
    d = make_model_dir(str(tmp_path / "m"), cfg, 5, dtype="bfloat16", sharpen=1.5)
    prompts = [random_ids(n, cfg["vocab_size"], i) for i, n in enumerate([1, 5, 64, 130, 33, 7])]
    text = ";".join(",".join(map(str, p)) for p in prompts)
    p = _native([d, text, "10", "--dtype", dtype, *OPTIONS])
    assert _tokens(p, len(prompts)) == _python(d, prompts, dtype)
    assert p.stdout.strip().splitlines()[-1] == "[Generated 60 tokens total]"


def test_drawn_tokens_and_random_weights_from_a_seed(tmp_path):
    """Temperature sampling from a fixed seed, on weights that both fronts make from the seed alone (no file)."""
    from llmengine_b200 import SamplingParams
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_B))
    prompts = [random_ids(n, 1000, 30 + i) for i, n in enumerate([9, 40, 3])]
    text = ";".join(",".join(map(str, p)) for p in prompts)
    p = _native(["--random-config", str(cfg), "--seed", "123", text, "12", "--dtype", "float32", "--no-greedy", "--temperature", "0.7",
                 "--top-k", "50", *OPTIONS])
    from llmengine_b200 import LLM
    llm = LLM(config=TINY_B, random_seed=123, dtype="float32", page_size=16, max_cached_tokens=1024, max_num_seqs=4,
              max_num_batched_tokens=64, prefill_chunk=48, pipeline_decode=False)
    sp = SamplingParams(greedy=False, temperature=0.7, top_k=50, seed=123)
    want = [o.token_ids for o in llm.generate(prompts, sp, max_tokens=12, eos_token_id=None)]
    assert _tokens(p, 3) == want


def test_the_cpp_front_names_what_is_wrong(tmp_path):
    from llmengine_b200.weights import SafetensorsFile, write_safetensors
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 1)
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    del f
    del t["model.layers.1.self_attn.k_norm.weight"]
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(96, 200, dtype=torch.bfloat16)
    t["extra.weight"] = torch.zeros(3)
    write_safetensors(path, t)
    err = _native([d, "1,2,3", "4", *OPTIONS], expect=1).stderr
    assert "missing tensors (1)" in err and "model.layers.1.self_attn.k_norm.weight" in err
    assert "unexpected tensors (1)" in err and "extra.weight" in err
    assert "wrong shapes (1)" in err and "[96, 200]" in err and "[96, 224]" in err
    # an unknown architecture, a configuration this front does not serve, a token outside the vocabulary
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps(dict(TINY_A, architectures=["NoSuchModel"])))
    assert "unknown architecture 'NoSuchModel'; registered: Qwen3ForCausalLM" in _native(["--random-config", str(bad), "1"], expect=1).stderr
    win = tmp_path / "win.json"
    win.write_text(json.dumps(TINY_C))
    assert "sliding-window" in _native(["--random-config", str(win), "1"], expect=1).stderr
    ok = tmp_path / "ok.json"
    ok.write_text(json.dumps(TINY_A))
    assert "outside the vocabulary" in _native(["--random-config", str(ok), "5,512", "2", *OPTIONS], expect=1).stderr
    no_key = tmp_path / "nokey.json"
    no_key.write_text(json.dumps({k: v for k, v in TINY_A.items() if k != "rms_norm_eps"}))
    assert "lacks required key(s): rms_norm_eps" in _native(["--random-config", str(no_key), "1"], expect=1).stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_the_cpp_step_function_replays_a_mixed_trace(tmp_path, name, dtype):
    """examples/trace_run.cpp: the replay protocol on Engine::step_batch.  Up to four live requests, portions of some
    beside single tokens of others, so few pages that they are used again; logits against the plain implementation."""
    import numpy as np

    from helpers import compare, max_live_tokens
    from test_replay import CONFIGS, _setup, _traces
    d, page, reqs, ref, tol = _setup(tmp_path, name, dtype, 2.0)
    steps = _traces(reqs)["mixed"]
    out = tmp_path / "out"
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in e], "end": end})
             for i, (e, end) in enumerate(steps)]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate_native"), "--program", "trace_run", "--model", d,
                        "--dtype", dtype, "--out", str(out), "--max-tokens", str(max_live_tokens(steps, 64)), "--page-size", str(page)],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = CONFIGS[name][0]["vocab_size"]
    rows = {}
    for i, (e, _) in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V))
        k = 0
        for r, t, w in e:
            rows.setdefault(r, []).append(arr[k:k + len(w)])
            k += len(w)
        assert k == arr.shape[0]
    compare({r: torch.cat(v) for r, v in rows.items()}, ref, tol, f"C++ trace_run/{name}/{dtype}")
