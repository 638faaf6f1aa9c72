"""The Python entry point and the command line on the host (a CPU stand-in replaces the kernels):
greedy generation equals the plain implementation's greedy loop, under a small token budget that
forces prompts to be cut and batches to mix."""
import pytest
import torch

from helpers import make_model_dir, random_ids
from host_ops import HostOps
from llmengine_b200 import LLM, SamplingParams
from llmengine_b200.generate import parse_prompts
from plain_model import PlainQwen3, plain_sample
from tiny_configs import TINY_A, TINY_B


def plain_generate(plain, prompt, n, **sampling):
    ids, out = list(prompt), []
    for i in range(n):
        t = plain_sample(plain.logits(ids)[-1], **sampling(i) if callable(sampling.get("f")) else sampling)
        out.append(t)
        ids.append(t)
    return out


@pytest.mark.parametrize("cfg,page,chunk", [(TINY_A, 16, 64), (TINY_B, 8, 48)])
def test_greedy_generation_matches_the_plain_loop(tmp_path, cfg, page, chunk):
    d = make_model_dir(str(tmp_path / "m"), cfg, 5, dtype="float32", sharpen=2.0)
    llm = LLM(d, dtype="float32", page_size=page, max_cached_tokens=640, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=chunk, device="cpu", ops=HostOps(), use_cuda_graphs=False)
    prompts = [random_ids(n, cfg["vocab_size"], i) for i, n in enumerate([1, 5, 64, 130, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=5, eos_token_id=None)
    plain = PlainQwen3(d)
    for p, o in zip(prompts, outs):
        assert o.prompt_token_ids == p and o.finish_reason == "length"
        assert o.token_ids == plain_generate(plain, p, 5)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


def test_drawn_tokens_follow_the_request_seed_not_the_batch(tmp_path):
    from llmengine_b200.sampling import uniform
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 6, dtype="float32")
    mk = lambda: LLM(d, dtype="float32", page_size=8, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
                     prefill_chunk=48, device="cpu", ops=HostOps(), use_cuda_graphs=False)
    sp = SamplingParams(greedy=False, temperature=0.7, seed=123)
    p = random_ids(20, 1000, 1)
    alone = mk().generate(p, sp, max_tokens=6, eos_token_id=None)[0].token_ids
    mixed = mk().generate([random_ids(50, 1000, 2), p, random_ids(3, 1000, 3)], sp, max_tokens=6, eos_token_id=None)[1].token_ids
    assert alone == mixed
    plain = PlainQwen3(d)
    ids, want = list(p), []
    for i in range(6):
        t = plain_sample(plain.logits(ids)[-1], greedy=False, temperature=0.7, u=uniform(123, i))
        want.append(t), ids.append(t)
    assert alone == want


def test_eos_and_bad_ids(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 7, dtype="float32")
    llm = LLM(d, dtype="float32", max_cached_tokens=256, max_num_seqs=2, max_num_batched_tokens=64, device="cpu",
              ops=HostOps(), use_cuda_graphs=False)
    first = llm.generate([3, 4, 5], max_tokens=4, eos_token_id=None)[0].token_ids
    eos = first[1]
    out = llm.generate([3, 4, 5], max_tokens=4, eos_token_id=eos)[0]
    assert out.token_ids == first[:first.index(eos)] and out.finish_reason == "eos"
    with pytest.raises(ValueError, match="vocabulary"):
        llm.generate([3, 512], max_tokens=2)


def test_prompt_parsing():
    assert parse_prompts("5,17,3") == [[5, 17, 3]]
    assert parse_prompts("1 2 3; 4,5") == [[1, 2, 3], [4, 5]]
    with pytest.raises(ValueError):
        parse_prompts(" ; ")


def test_requests_that_end_on_eos_at_different_steps_with_pipelined_decoding(tmp_path):
    """4 live requests and 2 waiting; end tokens picked so that requests end at different steps, one of them
    before its first token.  Pipelined decoding learns of an end one step late: the wasted token must be
    dropped, the pages freed, the waiting requests admitted, and the tokens equal to the unpipelined run's."""
    from helpers import eos_scenario
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 15, dtype="float32", sharpen=2.0)
    mk = lambda pipelined: LLM(d, dtype="float32", page_size=8, max_cached_tokens=512, max_num_seqs=4,
                               max_num_batched_tokens=64, prefill_chunk=48, device="cpu", ops=HostOps(),
                               use_cuda_graphs=False, pipeline_decode=pipelined)
    prompts = [random_ids(n, 1000, 40 + i) for i, n in enumerate([9, 70, 3, 25, 1, 50])]
    expected, piped, plain_run, base = eos_scenario(mk, prompts)
    assert piped == expected and plain_run == expected
    assert len({len(t) for t, _ in expected}) >= 4, "the requests should end at different steps"
    plain = PlainQwen3(d)
    for p, toks in zip(prompts, base):
        assert toks == plain_generate(plain, p, len(toks))
