"""Shared test equipment: tiny model folders, traces (ways of cutting requests into steps) and
the comparison of a replayed trace with the plain implementation."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from llmengine_b200.config import EngineConfig, config_from_dict
from llmengine_b200.weights import SafetensorsFile, write_random_model, write_safetensors


def make_model_dir(path: str, cfg: dict, seed: int, dtype: str = "bfloat16", sharpen: float = 1.0) -> str:
    """Random model folder.  `sharpen` > 1 scales the QK-norm gains so that attention is far from
    uniform: a key read from a wrong place, or not read, then changes the logits visibly."""
    write_random_model(config_from_dict(cfg), seed, path, dtype=dtype)
    if sharpen != 1.0:
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        tensors = {n: f.tensor(n).clone() for n in f.names()}
        for n in tensors:
            if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
                tensors[n] = (tensors[n].float() * sharpen).to(tensors[n].dtype)
        del f
        write_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# A trace is a list of steps; a step is (entries, end) with entries = [(request, tokens, want)].
Step = Tuple[List[Tuple[str, List[int], List[int]]], List[str]]


def trace_whole(reqs: Dict[str, List[int]]) -> List[Step]:
    """Each request alone, in one step, every position wanted."""
    return [([(r, ids, list(range(len(ids))))], [r]) for r, ids in reqs.items()]


def trace_bulk_then_single(reqs: Dict[str, List[int]], tail: int = 32) -> List[Step]:
    """All but the last `tail` tokens in one step, then one token a step."""
    steps: List[Step] = []
    for r, ids in reqs.items():
        n = len(ids)
        cut = max(n - tail, 0)
        if cut:
            steps.append(([(r, ids[:cut], list(range(cut)))], []))
        for i in range(cut, n):
            steps.append(([(r, ids[i:i + 1], [0])], [r] if i == n - 1 else []))
    return steps


def trace_portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (48, 7, 2, 16, 1, 33, 2, 5)) -> List[Step]:
    """Portions of changing size, down to two tokens (and one)."""
    steps: List[Step] = []
    for r, ids in reqs.items():
        pos, k = 0, 0
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            steps.append(([(r, ids[pos:pos + n], list(range(n)))], [r] if pos + n == len(ids) else []))
            pos += n
    return steps


def trace_mixed(reqs: Dict[str, List[int]], prompt_len: Dict[str, int], max_live: int = 4, seed: int = 0,
                sizes: Sequence[int] = (24, 3, 2, 9, 17, 5)) -> List[Step]:
    """Up to `max_live` requests at a time: portions of some prompts beside single decoded tokens of
    others in the same step, a request now and then left out of a step, new requests started as old
    ones end (so their pages are used again)."""
    rng = random.Random(seed)
    waiting = list(reqs)
    live: List[str] = []
    pos = {r: 0 for r in reqs}
    steps: List[Step] = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, end = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            ids = reqs[r]
            if pos[r] < prompt_len[r]:
                n = min(rng.choice(sizes), prompt_len[r] - pos[r])
            else:
                n = 1
            entries.append((r, ids[pos[r]:pos[r] + n], list(range(n))))
            pos[r] += n
            if pos[r] == len(ids):
                end.append(r)
                live.remove(r)
        if entries:
            steps.append((entries, end))
    return steps


def poison_free_pages(engine) -> None:
    """Fill every page that no request holds with NaN: whatever is read from a page that was given
    back, or from one never written, then shows in the logits."""
    for gi, g in enumerate(engine.cache.groups):
        free = torch.tensor(sorted(g.pool._free), dtype=torch.long, device=engine.device)
        if free.numel():
            for run in g.runs:
                engine.cache.kv[run][free] = float("nan")


def replay(engine, steps: List[Step], poison: bool = False, page_log: Optional[Dict[str, set]] = None,
           tamper=None) -> Dict[str, torch.Tensor]:
    """Run a trace through `engine.step`; returns request -> [positions, vocab] logits in position order.
    `page_log` collects, per request, every page of cache group 0 it ever held.  `tamper(engine, i)` is
    called before step i (the negative controls damage the cache there)."""
    from llmengine_b200.engine.engine import StepEntry

    rows: Dict[str, List[torch.Tensor]] = {}
    for i, (entries, end) in enumerate(steps):
        if tamper is not None:
            tamper(engine, i)
        if poison:
            poison_free_pages(engine)
        if page_log is not None:
            # what the step will hold: reserve as the step does, by looking after it (ended requests are gone
            # by then, so look at the tables before they are freed: run the step without `end`, then end them)
            out = engine.step([StepEntry(r, t, w) for r, t, w in entries], [])
            for r, _, _ in entries:
                page_log.setdefault(r, set()).update(p for p in engine.cache.requests[r].blocks[0] if p >= 0)
            for r in end:
                engine.free(r)
        else:
            out = engine.step([StepEntry(r, t, w) for r, t, w in entries], end)
        k = 0
        for r, t, w in entries:
            if w:
                assert list(w) == list(range(len(t))), "helper traces want every place"
                rows.setdefault(r, []).append(out[k:k + len(w)].float().cpu().clone())
                k += len(w)
    return {r: torch.cat(v) for r, v in rows.items()}


def max_live_tokens(steps: List[Step], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up to `round_to`."""
    held: Dict[str, int] = {}
    worst = 0
    for entries, end in steps:
        for r, t, _ in entries:
            held[r] = held.get(r, 0) + len(t)
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for r in end:
            held.pop(r, None)
    return worst


def first_bad(got: torch.Tensor, want: torch.Tensor, tol: float) -> Optional[int]:
    bad = ((got - want).abs().amax(-1) > tol).nonzero()
    return int(bad[0]) if bad.numel() else None


def compare(got: Dict[str, torch.Tensor], ref: Dict[str, torch.Tensor], tol: float, what: str) -> float:
    worst = 0.0
    for r, want in ref.items():
        g = got[r]
        assert g.shape == want.shape, f"{what}: request {r}: {tuple(g.shape)} vs {tuple(want.shape)}"
        assert torch.isfinite(g).all(), f"{what}: request {r}: non-finite logits"
        d = float((g - want).abs().max())
        worst = max(worst, d)
        if d > tol:
            p = first_bad(g, want, tol)
            raise AssertionError(
                f"{what}: request {r}: max |diff| {d:.3e} > {tol:.1e}; first wrong position {p} of {len(want)} "
                f"(diff there {float((g[p] - want[p]).abs().max()):.3e})")
    return worst


def engine_for(model_dir: str, dtype: str, pool_tokens: int, page_size: int = 16, ops=None, device: str = "cuda:0",
               kernels: str = "fast", max_requests: int = 8, use_cuda_graphs: bool = False, **more) -> "Engine":
    from llmengine_b200.engine.engine import Engine

    pool = -(-pool_tokens // page_size) * page_size
    ec = EngineConfig(dtype=dtype, page_size=page_size, max_cached_tokens=pool, max_num_seqs=max_requests,
                      max_num_batched_tokens=pool, prefill_chunk=pool, device=device, kernels=kernels,
                      use_cuda_graphs=use_cuda_graphs, **more)
    return Engine(model_dir, engine_config=ec, ops=ops)


def eos_scenario(make_llm, prompts: List[List[int]], max_tokens: int = 12):
    """Requests that end on an end-of-sequence token at different steps while others go on and some wait for
    admission.  A first greedy run without any end token gives each request's tokens; request i then gets as its
    end token the one it generated at place `cut[i]` (place 0: it ends before it has generated anything; None: it
    runs to max_tokens), so the expected output is its tokens up to the first occurrence of that token.  Returns
    (expected, with pipelined decoding, without) as lists of (tokens, finish_reason), and the last engine used."""
    free_run = make_llm(True)
    base = [o.token_ids for o in free_run.generate(prompts, None, max_tokens=max_tokens, eos_token_id=None)]
    cuts = [2, 5, 0, 9, None, 3, 7, 1]
    expected, eos = [], []
    for i, toks in enumerate(base):
        cut = cuts[i % len(cuts)]
        if cut is None:
            eos.append(None)
            expected.append((toks, "length"))
        else:
            e = toks[cut]
            eos.append(e)
            expected.append((toks[:toks.index(e)], "eos"))
    runs = []
    for pipelined in (True, False):
        llm = make_llm(pipelined)
        ids = [llm.add_request(p, None, max_tokens=max_tokens, eos_token_id=e) for p, e in zip(prompts, eos)]
        done = {}
        for _ in range(10000):
            for out in llm.step():
                done[out.sequence_id] = out
            if len(done) == len(ids) and llm._inflight is None:
                break
        assert len(done) == len(ids), "some request never finished"
        llm.step()                                            # nothing left: must be harmless
        runs.append([(done[i].generated_tokens, done[i].finish_reason) for i in ids])
        llm.engine.cache.check_invariants()
        assert not llm.engine.cache.requests and llm.scheduler.all_done()
        assert all(g.pool.free_count == g.pool.num_pages and g.committed == 0 for g in llm.engine.cache.groups)
        assert llm.engine.cache.free_slots == llm.engine.cache.max_requests
    return expected, runs[0], runs[1], base
