"""`Engine.step` on the host (a CPU stand-in replaces the kernels): every kind of refused batch leaves
block tables, free lists, state slots and lengths exactly as they were.  The reference tests the same
promise for its cache alone ("capacity error leaves state untouched", tests/test_paged_kv_cache.cpp:107-119)."""
import copy

import numpy as np
import pytest

from helpers import engine_for, make_model_dir, random_ids
from host_ops import HostOps
from llmengine_b200.engine.engine import StepEntry, StepError
from tiny_configs import TINY_A, TINY_C


def _snapshot(eng):
    c = eng.cache
    return {
        "tables": [t.copy() for t in c.tables],
        "free": [list(g.pool._free) for g in c.groups],
        "used": [list(g.pool._used) for g in c.groups],
        "committed": [g.committed for g in c.groups],
        "slots": list(c._free_slots),
        "requests": {r: (st.slot, st.length, copy.deepcopy(st.blocks)) for r, st in c.requests.items()},
        "steps": eng.steps,
    }


def _same(a, b):
    assert all(np.array_equal(x, y) for x, y in zip(a["tables"], b["tables"])), "a block table changed"
    for k in ("free", "used", "committed", "slots", "requests", "steps"):
        assert a[k] == b[k], f"{k} changed"


@pytest.fixture(params=["A", "C"])
def engine(request, tmp_path):
    cfg = {"A": TINY_A, "C": TINY_C}[request.param]          # C has two cache groups (one with a window)
    d = make_model_dir(str(tmp_path / "m"), cfg, 3, dtype="float32")
    eng = engine_for(d, "float32", 160, page_size=16, ops=HostOps(), device="cpu", max_requests=3, max_model_len=120)
    eng.vocab = cfg["vocab_size"]
    # two live requests, one of them at a page's edge
    eng.step([StepEntry("a", random_ids(32, eng.vocab, 1), [31]), StepEntry("b", random_ids(21, eng.vocab, 2), [])])
    return eng


def _refused(eng, entries, end=(), match=None):
    before = _snapshot(eng)
    with pytest.raises(StepError, match=match):
        eng.step(entries, end)
    _same(before, _snapshot(eng))
    eng.cache.check_invariants()


def test_a_request_twice_in_one_step(engine):
    _refused(engine, [StepEntry("a", [1], [0]), StepEntry("a", [2], [0])], match="twice")


def test_a_token_outside_the_vocabulary(engine):
    _refused(engine, [StepEntry("a", [1], [0]), StepEntry("b", [5, engine.vocab], [1])], match="vocabulary")
    _refused(engine, [StepEntry("c", [-1], [0])], match="vocabulary")
    _refused(engine, [StepEntry("c", [[1, 2]], [0])], match="flat list")


def test_over_the_token_budget(engine):
    _refused(engine, [StepEntry("a", [1] * 100, []), StepEntry("b", [1] * 61, [])], match="budget")


def test_over_the_model_length(engine):
    _refused(engine, [StepEntry("b", [1] * 100, [])], match="limit")


def test_a_wanted_place_outside_the_tokens_or_named_twice(engine):
    _refused(engine, [StepEntry("a", [1, 2], [2])], match="outside")
    _refused(engine, [StepEntry("a", [1, 2], [0, 0])], match="wanted twice")


def test_ending_a_request_that_is_not_live(engine):
    _refused(engine, [StepEntry("a", [1], [0])], end=["ghost"], match="not live")


def test_pages_run_out_after_some_entries_have_grown(engine):
    # 10 pages in the pool, "a" holds 2 and "b" 2 (group of all keys); a: +3 pages fits, then c: 5 more do not
    free0 = engine.cache.groups[0].pool.free_count
    assert free0 == 6
    _refused(engine, [StepEntry("a", [1] * 40, []), StepEntry("c", [1] * 70, [])], match="does not fit the cache")
    assert not engine.cache.has("c")


def test_more_requests_than_slots(engine):
    engine.step([StepEntry("c", [1], [0])])
    _refused(engine, [StepEntry("d", [1], [0])], match="does not fit the cache")
    _refused(engine, [StepEntry(f"n{i}", [1], [0]) for i in range(4)], match="limit")


def test_a_good_step_still_works_after_refusals(engine):
    _refused(engine, [StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    out = engine.step([StepEntry("a", [7], [0]), StepEntry("b", [8, 9], [1])], end=["a"])
    assert out.shape == (2, engine.vocab)
    assert not engine.cache.has("a") and engine.cache.length("b") == 23
    engine.cache.check_invariants()


@pytest.mark.parametrize("name", ["A", "C"])
def test_the_host_cheap_decode_path_does_what_the_general_one_does(tmp_path, name):
    """Steps of single tokens take a path that works on whole arrays; forced through the general path instead, the
    same requests give the same logits and leave the same tables, free lists and lengths, step after step: across
    page edges, and in C while the window of one cache group gives pages back."""
    cfg = {"A": TINY_A, "C": TINY_C}[name]
    d = make_model_dir(str(tmp_path / "m"), cfg, 4, dtype="float32")
    engines = [engine_for(d, "float32", 256, page_size=8, ops=HostOps(), device="cpu", max_requests=3) for _ in range(2)]
    engines[1]._decode_step = lambda entries, end, device_tokens=None: NotImplemented
    ids = {"a": random_ids(70, cfg["vocab_size"], 1), "b": random_ids(45, cfg["vocab_size"], 2)}
    outs = []
    for eng in engines:
        got = [eng.step([StepEntry("a", ids["a"][:20], [19])])]
        for i in range(45):
            entries = [StepEntry("a", ids["a"][20 + i:21 + i], [0]), StepEntry("b", ids["b"][i:i + 1], [0])]
            if i == 0:
                entries[1] = StepEntry("b", ids["b"][:1], [0])          # b's first token: a new request, the general path
            got.append(eng.step(entries, end=["b"] if i == 44 else []))
            eng.cache.check_invariants()
        outs.append(got)
    for x, y in zip(*outs):
        assert np.array_equal(x.numpy(), y.numpy())
    _same(_snapshot(engines[0]), _snapshot(engines[1]))
    if name == "C":
        assert any(p == -1 for p in engines[0].cache.requests["a"].blocks[1]), "the window gave no page back"
