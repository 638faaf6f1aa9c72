"""On the GPU: generation through the Python entry point and the command line, long decoding
one token at a time from the very first token, and drawn tokens from a fixed seed."""
import os
import subprocess
import sys

import pytest
import torch

from helpers import compare, engine_for, make_model_dir, random_ids, replay
from llmengine_b200 import LLM, SamplingParams
from llmengine_b200.sampling import uniform
from plain_model import PlainQwen3, plain_sample
from tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _check_greedy(plain, prompt, tokens, dtype, rounded=None):
    """Every generated token is the plain implementation's argmax given the tokens before it.  In bfloat16 the
    reference is the plain implementation with bfloat16 rounding at the engine's places, and another token is
    accepted only where that reference nearly ties: the engine's logits may lie up to `tol` from the
    reference's (the bound of the replay tests: three quarters of the distance between the rounded and the
    32-bit plain run, on this very sequence), so its choice can differ only where the reference's gap is at most
    2 tol.  Returns the largest gap that was accepted."""
    ids, worst = list(prompt), 0.0
    for t in tokens:
        row = plain.logits(ids)
        margin = 1e-4
        if dtype == "bfloat16":
            row16 = rounded.logits(ids)
            margin = 2 * max(5e-3, 0.75 * float((row16 - row).abs().max()))
            row = row16
        row = row[-1]
        best = int(row.argmax())
        gap = float(row[best] - row[t])
        assert t == best or gap <= margin, (len(ids), t, best, gap, margin)
        worst = max(worst, gap)
        ids.append(t)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,page,chunk", [(TINY_A, 16, 64), (TINY_B, 8, 48), (TINY_C, 16, 40)])
def test_greedy_generation_through_the_entry_point(tmp_path, cfg, page, chunk, dtype):
    d = make_model_dir(str(tmp_path / "m"), cfg, 5, dtype="bfloat16", sharpen=1.5)
    llm = LLM(d, dtype=dtype, page_size=page, max_cached_tokens=1024, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=chunk)
    prompts = [random_ids(n, cfg["vocab_size"], i) for i, n in enumerate([1, 5, 64, 130, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=16, eos_token_id=None)
    plain, rounded = PlainQwen3(d), PlainQwen3(d, round_to=torch.bfloat16)
    worst = 0.0
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 16 and o.finish_reason == "length"
        worst = max(worst, _check_greedy(plain, p, o.token_ids, dtype, rounded))
    print(f"greedy {dtype}: largest gap of an accepted token to the reference's best {worst:.2e}")
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests
    assert llm.engine.ops.launches > 0


@pytest.mark.parametrize("cfg", [TINY_B, TINY_C], ids=["B", "C"])
@pytest.mark.parametrize("short_context", [8192, 48])
def test_cuda_graph_decoding_gives_the_same_tokens(tmp_path, monkeypatch, short_context, cfg):
    """Captured decode steps against eager ones; with the small limit the requests grow past it while they decode,
    so that both kinds of capture (short contexts, any context) are made and replayed."""
    from llmengine_b200.engine.engine import Engine
    monkeypatch.setattr(Engine, "SHORT_CONTEXT", short_context)
    d = make_model_dir(str(tmp_path / "m"), cfg, 8, dtype="bfloat16", sharpen=1.5)
    prompts = [random_ids(n, cfg["vocab_size"], i) for i, n in enumerate([9, 40, 3])]
    runs = []
    for graphs in (False, True):
        llm = LLM(d, dtype="bfloat16", page_size=8, max_cached_tokens=1024, max_num_seqs=4, max_num_batched_tokens=64,
                  use_cuda_graphs=graphs)
        runs.append([o.token_ids for o in llm.generate(prompts, max_tokens=40, eos_token_id=None)])
    assert runs[0] == runs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(tmp_path, dtype):
    """One token a step from position 0 on, for 230 steps, two requests side by side: the first tokens
    of a sequence, every page edge and a long run of single-token steps."""
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 6, dtype="bfloat16", sharpen=2.0)
    reqs = {"a": random_ids(230, 512, 1), "b": random_ids(190, 512, 2)}
    steps = []
    for i in range(230):
        entries = [(r, ids[i:i + 1], [0]) for r, ids in reqs.items() if i < len(ids)]
        steps.append((entries, [r for r, ids in reqs.items() if i == len(ids) - 1]))
    eng = engine_for(d, dtype, 512, page_size=16)
    got = replay(eng, steps, poison=True)
    if dtype == "float32":
        plain = PlainQwen3(d)
        compare(got, {r: plain.logits(ids) for r, ids in reqs.items()}, 1e-4, "long decode")
    else:
        from test_replay import bf16_tolerance
        p32, p16 = PlainQwen3(d), PlainQwen3(d, round_to=torch.bfloat16)
        ref16 = {r: p16.logits(ids) for r, ids in reqs.items()}
        compare(got, ref16, bf16_tolerance(ref16, {r: p32.logits(ids) for r, ids in reqs.items()}), "long decode bf16")


def test_drawn_tokens_from_a_fixed_seed(tmp_path):
    """Temperature 0.7 from a fixed seed (32-bit): the tokens are those of the plain sampler fed the
    plain logits and the same uniform numbers, whatever else is in the batch."""
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 7, dtype="bfloat16")
    llm = LLM(d, dtype="float32", page_size=8, max_cached_tokens=1024, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=48)
    prompts = [random_ids(n, 1000, 10 + i) for i, n in enumerate([1, 5, 64, 130, 200])]
    sps = [SamplingParams(greedy=False, temperature=0.7, seed=1000 + i) for i in range(5)]
    outs = llm.generate(prompts, sps, max_tokens=24, eos_token_id=None)
    plain = PlainQwen3(d)
    for p, sp, o in zip(prompts, sps, outs):
        ids = list(p)
        for i, t in enumerate(o.token_ids):
            row = plain.logits(ids)[-1]
            want = plain_sample(row, greedy=False, temperature=0.7, u=uniform(sp.seed, i))
            if t != want:       # only possible when u sits on the boundary between the two tokens
                pr = torch.softmax(row.double() / 0.7, 0)
                cdf = torch.cumsum(pr, 0)
                assert abs(float(cdf[min(t, want)]) - uniform(sp.seed, i)) < 1e-4, (i, t, want)
            ids.append(t)


def test_top_k_top_p_and_penalty_through_the_entry_point(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 9, dtype="bfloat16")
    llm = LLM(d, dtype="float32", max_cached_tokens=512, max_num_seqs=2, max_num_batched_tokens=64)
    plain = PlainQwen3(d)
    p = random_ids(12, 512, 3)
    sp = SamplingParams(greedy=False, temperature=1.3, top_k=5, top_p=0.9, repetition_penalty=1.2, seed=5)
    toks = llm.generate(p, sp, max_tokens=12, eos_token_id=None)[0].token_ids
    ids = list(p)
    for i, t in enumerate(toks):
        row = plain.logits(ids)[-1]
        z = row.clone()
        for h in ids:
            z[h] = z[h] / 1.2 if z[h] > 0 else z[h] * 1.2
        top5 = torch.topk(z, 5).indices.tolist()
        assert t in top5, (i, t, top5)
        ids.append(t)
    greedy_pen = llm.generate(p, SamplingParams(repetition_penalty=1.2), max_tokens=8, eos_token_id=None)[0].token_ids
    ids = list(p)
    for t in greedy_pen:
        want = plain_sample(plain.logits(ids)[-1], repetition_penalty=1.2, history=ids)
        assert t == want
        ids.append(t)


def test_command_line(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 5, dtype="bfloat16", sharpen=1.5)
    p = subprocess.run([sys.executable, "-m", "llmengine_b200.generate", d, "5,17,3;9 8 7 6", "6", "--dtype", "float32",
                        "--ignore-eos"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert lines[-1] == "[Generated 12 tokens total]"
    plain = PlainQwen3(d)
    for prompt, line in zip(([5, 17, 3], [9, 8, 7, 6]), lines):
        _check_greedy(plain, prompt, [int(x) for x in line.split()], "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_requests_that_end_on_eos_at_different_steps_with_pipelined_decoding(tmp_path, dtype, graphs):
    """4 live requests and 2 waiting, end tokens picked so that the requests end at different steps (one before its
    first token): pipelined decoding, which learns of an end one step late, gives the tokens of the unpipelined run,
    frees every page and admits the waiting requests."""
    from helpers import eos_scenario
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 15, dtype="bfloat16", sharpen=1.5)
    mk = lambda pipelined: LLM(d, dtype=dtype, page_size=8, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
                               prefill_chunk=48, use_cuda_graphs=graphs, pipeline_decode=pipelined)
    prompts = [random_ids(n, 1000, 40 + i) for i, n in enumerate([9, 70, 3, 25, 1, 50])]
    expected, piped, unpiped, base = eos_scenario(mk, prompts)
    assert piped == expected and unpiped == expected
    assert len({len(t) for t, _ in expected}) >= 4
    plain, rounded = PlainQwen3(d), PlainQwen3(d, round_to=torch.bfloat16)
    for p, toks in zip(prompts, base):
        _check_greedy(plain, p, toks, dtype, rounded)
