"""The scheduler's decisions on the host: lifecycle, admission, the token budget and portions,
finishing and freeing, and what happens when pages run out.  (The behaviours that the
reference's tests/test_continuous_batch_scheduler.cpp checks, plus the parts it leaves to its
caller.)"""
import pytest

from llmengine_b200.cache import CacheManager
from llmengine_b200.engine.scheduler import ContinuousBatchScheduler, SeqPhase, SequenceRequest
from llmengine_b200.parts.base import PagedKVSpec
from llmengine_b200.sampling import SamplingParams, uniform


def make(tokens=256, page=8, max_batch=4, budget=32, chunk=16, max_len=512, window=0):
    cache = CacheManager([(PagedKVSpec(2, 16, window), None)], page, tokens, 8, max_len)
    return ContinuousBatchScheduler(cache, max_batch, budget, chunk), cache


def run_step(s, sampled_token=7):
    """One scheduling round with a stand-in for the model: every sampling entry yields `sampled_token`."""
    s.admit_waiting()
    entries = s.schedule()
    for e in entries:                                   # what Engine.step does with the cache
        st = s.cache.requests[e.sequence_id]
        s.cache.reserve(e.sequence_id, st.length + len(e.tokens))
        s.cache.advance(e.sequence_id, st.length + len(e.tokens))
    s.process_outputs(entries, {e.sequence_id: sampled_token for e in entries if e.samples})
    s.evict_finished()
    return entries


def test_submit_checks_and_ids():
    s, _ = make()
    with pytest.raises(ValueError, match="at least one prompt token"):
        s.submit(SequenceRequest([], 4))
    with pytest.raises(ValueError, match="max_tokens"):
        s.submit(SequenceRequest([1], 0))
    assert s.submit(SequenceRequest([1, 2], 4)) == 0
    assert s.submit(SequenceRequest([1], 4, sequence_id=5)) == 5
    assert s.submit(SequenceRequest([1], 4)) == 6        # an explicit id moves the counter on
    with pytest.raises(ValueError, match="already in use"):
        s.submit(SequenceRequest([1], 4, sequence_id=5))
    assert s.waiting_ids() == [0, 5, 6] and s.waiting_count() == 3 and not s.has_active()


def test_lifecycle_and_portions_under_the_budget():
    s, cache = make(budget=20, chunk=16)
    a = s.submit(SequenceRequest(list(range(40)), 3))
    b = s.submit(SequenceRequest(list(range(5)), 2))
    e = run_step(s)
    assert s.state(a).phase is SeqPhase.Prefilling and s.state(b).phase is SeqPhase.Prefilling
    assert [(x.sequence_id, len(x.tokens), x.samples) for x in e] == [(a, 16, False), (b, 4, False)]   # 20 in all
    e = run_step(s)
    assert [(x.sequence_id, len(x.tokens), x.samples) for x in e] == [(a, 16, False), (b, 1, True)]
    assert s.state(b).phase is SeqPhase.Decoding and s.state(b).generated_tokens == [7]
    e = run_step(s)                                       # decode tokens come first, then the prompt's rest
    assert [(x.sequence_id, x.tokens, x.samples) for x in e] == [(b, [7], True), (a, list(range(32, 40)), True)]
    assert s.state(a).phase is SeqPhase.Decoding and s.state(a).prefilled_tokens == 40
    assert b not in s.active_ids()                        # b reached max_tokens = 2: finished, evicted, pages back
    outs = {o.sequence_id: o for o in s.collect_finished()}
    assert outs[b].generated_tokens == [7, 7] and outs[b].finish_reason == "length" and outs[b].finished
    assert not cache.has(b) and cache.has(a)
    run_step(s), run_step(s)
    assert s.all_done() and cache.free_pages() == cache.groups[0].pool.num_pages
    assert s.collect_finished()[0].generated_tokens == [7, 7, 7]


def test_eos_finishes_without_keeping_the_token():
    s, _ = make()
    a = s.submit(SequenceRequest([1, 2, 3], 10, eos_token_id=99))
    run_step(s, 5)
    run_step(s, 99)
    out = s.collect_finished()[0]
    assert out.sequence_id == a and out.generated_tokens == [5] and out.finish_reason == "eos"


def test_batch_limit_and_first_in_first_out():
    s, _ = make(max_batch=2)
    ids = [s.submit(SequenceRequest([1] * 4, 2)) for _ in range(4)]
    s.admit_waiting()
    assert s.active_ids() == ids[:2] and s.waiting_ids() == ids[2:]
    run_step(s), run_step(s)
    assert s.active_ids() == [] or set(s.active_ids()) <= set(ids)
    while not s.all_done():
        run_step(s)
    assert [o.sequence_id for o in s.collect_finished()] == ids


def test_when_pages_run_out():
    """Decided at admission: a request waits until the pages it can ever need can be promised; the
    queue keeps its order (the head blocks those behind it); nothing is preempted; an admitted request
    never lacks a page; a request that can never fit is refused at submit."""
    s, cache = make(tokens=64, page=8, max_batch=4, budget=64, chunk=64)      # 8 pages in all
    with pytest.raises(ValueError, match="more than"):
        s.submit(SequenceRequest([1] * 60, 8))                                # 68 tokens can never fit
    a = s.submit(SequenceRequest([1] * 30, 10))                               # 5 pages
    b = s.submit(SequenceRequest([1] * 20, 10))                               # 4 pages: does not fit beside a
    c = s.submit(SequenceRequest([1] * 4, 4))                                 # 1 page: would fit, but waits behind b
    s.admit_waiting()
    assert s.active_ids() == [a] and s.waiting_ids() == [b, c]
    assert not cache.has(b)                                                   # the failed admission left nothing behind
    steps = 0
    while s.state(a).phase is not SeqPhase.Finished and a in s.states:
        run_step(s)
        steps += 1
        cache.check_invariants()
        if a not in s.states or s.state(a).phase is SeqPhase.Finished:
            break
    run_step(s)
    assert b in s.active_ids() and c in s.active_ids()                        # both admitted once a gave its pages back
    while not s.all_done():
        run_step(s)
        cache.check_invariants()
    assert cache.groups[0].committed == 0 and cache.free_pages() == 8


def test_window_groups_commit_their_peak_only():
    s, cache = make(tokens=64, page=8, window=16, chunk=8, budget=16, max_len=4096)
    a = s.submit(SequenceRequest([1] * 300, 100))     # 400 tokens, but a window of 16 never holds more than 4 pages
    s.admit_waiting()
    assert s.active_ids() == [a] and cache.groups[0].committed == 4
    for _ in range(60):
        run_step(s)
        cache.check_invariants()
    assert cache.length(a) > 64                       # far more tokens went through than the pool holds


def test_constructor_checks():
    cache = CacheManager([(PagedKVSpec(2, 16, 0), None)], 8, 64, 8, 64)
    with pytest.raises(ValueError, match="max_batch_size"):
        ContinuousBatchScheduler(cache, 0)
    with pytest.raises(ValueError, match="max_num_batched_tokens"):
        ContinuousBatchScheduler(cache, 8, 4)


def test_sampling_params_and_uniform_numbers():
    p = SamplingParams()
    assert (p.greedy, p.top_k, p.top_p, p.temperature, p.repetition_penalty, p.seed) == (True, 0, 0.0, 1.0, 1.0, 42)
    for bad in (dict(top_k=-1), dict(top_p=1.5), dict(temperature=-0.1), dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    us = [uniform(42, i) for i in range(2000)]
    assert all(0.0 < u < 1.0 for u in us) and len(set(us)) > 1990
    assert abs(sum(us) / len(us) - 0.5) < 0.02
    assert uniform(42, 3) == uniform(42, 3) != uniform(43, 3)
