"""Replay of the same requests under different ways of cutting them into steps, compared with
the plain implementation: whole; most of it in one step and the last 32 tokens one by one; in
portions of changing size down to two tokens; mixed, up to four live requests with so few
pages that they are used again.  In 32-bit and in bfloat16 on the GPU; the host logic alone
(batch metadata, cache bookkeeping) also runs without a GPU against a CPU stand-in for the
kernels."""
import os
import subprocess
import sys
import json

import numpy as np
import pytest
import torch

from helpers import (compare, engine_for, make_model_dir, max_live_tokens, random_ids, replay, trace_bulk_then_single,
                     trace_mixed, trace_portions, trace_whole)
from plain_model import PlainQwen3
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D, TINY_E

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Largest |logit difference| allowed against the plain implementation.  Logits of these models
# are of order 1.  32-bit: only the order of sums differs, 1e-4 at most.  bfloat16: the plain
# implementation rounds to bfloat16 at the same places as the engine, but the engine's kernels round a
# few values more (attention probabilities before the value product) and add in another order, and a value
# that falls on the other side of a rounding step is carried on and amplified by a model with sharp
# attention.  The yardstick is the model's own sensitivity to such rounding, measured on the plain
# implementation: the distance between its bfloat16-rounded run and its 32-bit run.  The engine's distance
# from the rounded plain run is the sum of the same kind of rounding steps: measured, it is 0.2 to 0.6 of
# that yardstick for every configuration and schedule (the tests print it), so the bound is three quarters
# of the yardstick (and 5e-3 at least).  The negative controls below show what the bound catches: one page
# exchanged with another's moves the logits to 20 to 30 times the bound (10,000 times in 32-bit).
TOL_F32 = 1e-4


def bf16_tolerance(ref16, ref32):
    inherent = max(float((ref16[r] - ref32[r]).abs().max()) for r in ref16)
    return max(5e-3, 0.75 * inherent)


CONFIGS = {
    "A": (TINY_A, 16, [70, 33, 100, 19, 45, 64, 7]),
    "B": (TINY_B, 8, [1, 5, 64, 130, 200, 48]),
    "C": (TINY_C, 16, [90, 37, 120, 64, 23]),
    "D": (TINY_D, 16, [300, 129, 40, 520, 128, 17]),
    "E": (TINY_E, 32, [2, 128, 200, 33, 127]),
}


def _setup(tmp_path, name, dtype, sharpen):
    cfg, page, lens = CONFIGS[name]
    d = make_model_dir(str(tmp_path / f"{name}_{dtype}"), cfg, seed=11, dtype="bfloat16", sharpen=sharpen)
    reqs = {f"r{i}": random_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(lens)}
    plain = PlainQwen3(d)
    ref = {r: plain.logits(ids) for r, ids in reqs.items()}
    tol = TOL_F32
    if dtype == "bfloat16":
        rounded = PlainQwen3(d, round_to=torch.bfloat16)
        ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
        tol, ref = bf16_tolerance(ref16, ref), ref16
    return d, page, reqs, ref, tol


def _traces(reqs):
    prompt = {r: max(1, len(ids) - 12) for r, ids in reqs.items()}
    return {
        "whole": trace_whole(reqs),
        "bulk_then_single": trace_bulk_then_single(reqs, 32),
        "portions": trace_portions(reqs),
        "mixed": trace_mixed(reqs, prompt, max_live=4, seed=3),
    }


def _run_all(tmp_path, name, dtype, sharpen, ops, device, page_size=None):
    d, page, reqs, ref, tol = _setup(tmp_path, name, dtype, sharpen)
    page = page_size or page
    worst = {}
    for what, steps in _traces(reqs).items():
        pool = max_live_tokens(steps, 64)
        eng = engine_for(d, dtype, pool, page_size=page, ops=ops, device=device)
        pages = {} if what == "mixed" else None
        got = replay(eng, steps, poison=True, page_log=pages)
        worst[what] = compare(got, ref, tol, f"{name}/{dtype}/{what}") / tol
        eng.cache.check_invariants()
        assert not eng.cache.requests, "every request was ended, nothing may be held"
        assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.groups)
        if pages is not None:
            owners = {}
            for r, held in pages.items():
                for p in held:
                    owners.setdefault(p, set()).add(r)
            assert any(len(o) > 1 for o in owners.values()), "no page was handed to a second request: the pool is too large"
    return worst


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_host_logic_replay_cpu(tmp_path, name):
    from host_ops import HostOps
    _run_all(tmp_path, name, "float32", 1.0, HostOps(), "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,sharpen", [("float32", 1.0), ("float32", 3.0), ("bfloat16", 1.0), ("bfloat16", 2.0)])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_gpu(tmp_path, name, dtype, sharpen):
    """`sharpen` scales the QK-norm gains: attention becomes peaked, so that a key that is skipped,
    read from a wrong page or seen through a wrong mask moves the logits by far more than the tolerance."""
    worst = _run_all(tmp_path, name, dtype, sharpen, None, "cuda:0")
    print(f"replay {name} {dtype} sharpen={sharpen}: distance as a share of the tolerance: "
          + ", ".join(f"{k} {v:.2f}" for k, v in worst.items()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_gpu_with_the_default_page_size(tmp_path, name, dtype):
    """The same traces with pages as large as the engine makes them when nobody says otherwise (the tests above
    use small pages, which put more page edges into a sequence)."""
    from llmengine_b200.config import EngineConfig
    _run_all(tmp_path, name, dtype, 2.0 if dtype == "bfloat16" else 3.0, None, "cuda:0", page_size=EngineConfig().page_size)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """The program itself, as a user calls it: JSON lines in, <step>.f32 files and `done` lines out."""
    d, page, reqs, ref, tol = _setup(tmp_path, "B", dtype, 2.0)
    steps = _traces(reqs)["mixed"]
    out = tmp_path / "out"
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in e], "end": end})
             for i, (e, end) in enumerate(steps)]
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_live_tokens(steps, 64))],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    rows = {}
    V = TINY_B["vocab_size"]
    for i, (e, _) in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V))
        k = 0
        for r, t, w in e:
            rows.setdefault(r, []).append(arr[k:k + len(w)])
            k += len(w)
        assert k == arr.shape[0]
    compare({r: torch.cat(v) for r, v in rows.items()}, ref, tol, f"trace_run/{dtype}")


# many heads of 32 and a long prompt: a step of more than a thousand tokens takes the kernels that only large
# steps take (QK norm + RoPE + cache write with a warp per token and run of heads; the tcgen05 product when its
# tiles fill the GPU, which a model this small never does, so the test switches it on)
LONG_PROMPT = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 64,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 32, "intermediate_size": 96,
    "vocab_size": 300, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 1600, "hidden_act": "silu",
}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("products", ["auto", "tcgen05"])
def test_long_prompt_in_one_step_gpu(tmp_path, dtype, products):
    d = make_model_dir(str(tmp_path / "m"), LONG_PROMPT, seed=21, dtype="bfloat16", sharpen=2.0)
    reqs = {"long": random_ids(1500, LONG_PROMPT["vocab_size"], 7), "short": random_ids(40, LONG_PROMPT["vocab_size"], 8)}
    plain = PlainQwen3(d)
    ref = {r: plain.logits(ids) for r, ids in reqs.items()}
    tol = TOL_F32
    if dtype == "bfloat16":
        rounded = PlainQwen3(d, round_to=torch.bfloat16)
        ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
        tol, ref = bf16_tolerance(ref16, ref), ref16
    # both requests in one step of 1,540 tokens; then the long one again in two steps (1,300 + 200)
    both = [([(r, ids, list(range(len(ids)))) for r, ids in reqs.items()], list(reqs))]
    ids = reqs["long"]
    cut = [([("long", ids[:1300], list(range(1300)))], []), ([("long", ids[1300:], list(range(200)))], ["long"])]
    for what, steps in (("one step", both), ("two steps", cut)):
        eng = engine_for(d, dtype, max_live_tokens(steps, 64), page_size=64)
        eng.ops.plain_gemm = products
        got = replay(eng, steps, poison=True)
        compare(got, {r: ref[r] for r in got}, tol, f"long prompt/{dtype}/{products}/{what}")
        eng.check_kernels()


# ----------------------------------------------------------------------------- negative controls
def _tamper_plan(steps, page):
    """A step of the mixed trace before which two live requests each hold at least one full page and both go on
    afterwards: (step index, request 1, request 2)."""
    held = {}
    future = [set() for _ in steps]
    seen = set()
    for i in range(len(steps) - 1, -1, -1):
        future[i] = set(seen)
        seen |= {r for r, _, _ in steps[i][0]}
    for i, (entries, end) in enumerate(steps):
        ready = [r for r, n in held.items() if n >= page and r in future[i] | {e[0] for e in entries}]
        ready = [r for r in ready if any(r == e[0] for j in range(i, len(steps)) for e in steps[j][0])]
        if len(ready) >= 2:
            return i, ready[0], ready[1]
        for r, t, _ in entries:
            held[r] = held.get(r, 0) + len(t)
        for r in end:
            held.pop(r, None)
    raise AssertionError("the trace never has two live requests with a full page each")


def _swap_page_contents(run):
    """Exchange what the first pages of two live requests hold, in one layer's cache tensor."""
    def tamper(eng, i, plan={}):
        if i != tamper.at:
            return
        a = eng.cache.requests[tamper.r1].blocks[0][0]
        b = eng.cache.requests[tamper.r2].blocks[0][0]
        kv = eng.cache.kv[eng.cache.groups[0].runs[run]]
        keep = kv[a].clone()
        kv[a] = kv[b]
        kv[b] = keep
    return tamper


def _swap_table_entries():
    """Exchange the first block-table entries of two live requests (host and device tables alike): from then on
    each reads, and owns, the other's first page in every layer of the group."""
    def tamper(eng, i):
        if i != tamper.at:
            return
        c = eng.cache
        s1, s2 = c.requests[tamper.r1], c.requests[tamper.r2]
        s1.blocks[0][0], s2.blocks[0][0] = s2.blocks[0][0], s1.blocks[0][0]
        c.tables[0][s1.slot, 0], c.tables[0][s2.slot, 0] = s1.blocks[0][0], s2.blocks[0][0]
        c._mark(0, s1.slot, 0, 1)
        c._mark(0, s2.slot, 0, 1)
    return tamper


@pytest.mark.gpu
@pytest.mark.parametrize("damage", ["page_contents", "table_entries"])
@pytest.mark.parametrize("dtype,sharpen", [("float32", 3.0), ("bfloat16", 2.0)])
@pytest.mark.parametrize("page_size", [None, 64])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_a_wrong_page_is_seen_at_the_tolerance_of_the_replay_tests(tmp_path, name, dtype, sharpen, page_size, damage):
    """The negative control of the tests above: the same mixed trace, the same tolerance, but before one step a
    page of one request is exchanged with a page of another (its contents in one layer, or the two block-table
    entries).  Nothing faults (all memory is valid and held); the comparison must fail."""
    d, page, reqs, ref, tol = _setup(tmp_path, name, dtype, sharpen)
    page = page_size or page
    steps = _traces(reqs)["mixed"]
    try:
        at, r1, r2 = _tamper_plan(steps, page)
    except AssertionError:
        pytest.skip("with pages this large no two requests of the trace hold a full page at the same time")
    tamper = _swap_page_contents(0) if damage == "page_contents" else _swap_table_entries()
    tamper.at, tamper.r1, tamper.r2 = at, r1, r2
    eng = engine_for(d, dtype, max_live_tokens(steps, 64) + 2 * page, page_size=page)
    got = replay(eng, steps, tamper=tamper)
    worst = max(float((got[r] - ref[r]).abs().max()) for r in ref)
    print(f"negative control {name} {dtype} page {page} {damage}: distance {worst / tol:.1f} x the tolerance")
    with pytest.raises(AssertionError, match="max .diff."):
        compare(got, ref, tol, "damaged")


# ----------------------------------------------------------------------------- captured decode steps
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("short_context", [8192, 48])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_logits_of_captured_decode_steps(tmp_path, monkeypatch, name, dtype, short_context):
    """Decode steps replayed from CUDA graphs give the plain implementation's logits: most of each request in one
    step and its last 32 tokens one by one, and a long run of single-token steps of two requests side by side.  With
    the small limit the requests grow past it while they decode, so both kinds of capture (launch shapes for short
    contexts, and for any context) are made and replayed.  Configuration C has two cache groups, one of them with a
    window whose pages go back while the requests decode, and a layer order that runs a layer twice."""
    from llmengine_b200.engine.engine import Engine
    monkeypatch.setattr(Engine, "SHORT_CONTEXT", short_context)
    d, page, reqs, ref, tol = _setup(tmp_path, name, dtype, 2.0)
    steps = trace_bulk_then_single(reqs, 32)
    ids = {r: reqs[r] for r in sorted(reqs, key=lambda r: -len(reqs[r]))[:2]}
    n = max(len(v) for v in ids.values())
    side = []
    for i in range(n):
        entries = [(r, v[i:i + 1], [0]) for r, v in ids.items() if i < len(v)]
        side.append((entries, [r for r, v in ids.items() if i == len(v) - 1]))
    pool = max(max_live_tokens(steps, 64), max_live_tokens(side, 64))
    eng = engine_for(d, dtype, pool, page_size=page, use_cuda_graphs=True)
    got = replay(eng, steps, poison=True)
    compare(got, ref, tol, f"graphs/{name}/{dtype}/bulk_then_single")
    assert eng._graphs, "no decode step was captured"
    assert {k[1] for k in eng._graphs} == ({True, False} if short_context == 48 else {False})
    # two requests side by side, one token a step from the first token on
    got = replay(eng, side, poison=True)
    compare(got, {r: ref[r] for r in ids}, tol, f"graphs/{name}/{dtype}/side by side")
    assert any(k[0] == 2 for k in eng._graphs)
    eng.cache.check_invariants()
    eng.check_kernels()


# ----------------------------------------------------------------------------- one kernel exchanged for another inside the model
@pytest.mark.gpu
@pytest.mark.parametrize("kernels", ["plain", {"attention.portion": "mma"}, {"attention.decode": "split"},
                                     {"attention": "plain"}, {"linear": "cublas"}, {"linear": "tcgen05"},
                                     {"linear.decode": "cublas"}, {"linear_swiglu": "unfused"}])
def test_single_kernels_exchanged_inside_the_model(tmp_path, kernels):
    """`EngineConfig.kernels` as a mapping operation -> variant: the whole model runs with one kernel exchanged for its
    twin (the mma.sync portion attention for the tcgen05 one, the unfused decode attention, the library product, ...)
    and still gives the plain implementation's logits.  This is the tool that narrows a wrong logit down to a kernel."""
    d, page, reqs, ref, tol = _setup(tmp_path, "D", "bfloat16", 2.0)
    steps = _traces(reqs)["mixed"]
    eng = engine_for(d, "bfloat16", max_live_tokens(steps, 64), page_size=page, kernels=kernels)
    if isinstance(kernels, dict):
        for op, variant in kernels.items():
            assert eng.ops.chosen(op) == variant
    else:
        assert eng.ops.chosen("attention") == "plain" and eng.ops.chosen("linear") == "plain"
    before = eng.ops.launches
    got = replay(eng, steps, poison=True)
    compare(got, ref, tol, f"kernels={kernels}")
    assert eng.ops.launches > before
    eng.check_kernels()


@pytest.mark.gpu
def test_an_unknown_operation_or_variant_is_refused():
    from llmengine_b200.kernels.ops import CudaOps, KernelError
    ops = CudaOps(torch.device("cuda:0"))
    with pytest.raises(KernelError, match="no operation 'softmax'"):
        ops.choose("softmax", "fast")
    with pytest.raises(KernelError, match="has no variant 'wgmma'"):
        ops.choose("linear", "wgmma")
    with pytest.raises(Exception, match="kernels must be"):
        from llmengine_b200.config import EngineConfig
        EngineConfig(kernels="fastest")
