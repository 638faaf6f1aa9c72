"""Time of each operation of one layer (`python bench.py --breakdown`).

The model's own plan is timed record by record: record j of every layer in turn (each layer has weights of its own,
so nothing is served from L2 that a real step would read from HBM), averaged over the layers.  The records run
inside a CUDA graph, CUDA events around its replays: the kernels, their choice and their
arguments are exactly those of a step."""
from __future__ import annotations


def breakdown(args, model_cfg, CACHED, CONTEXT, PREFILL_TOKENS, pk) -> int:
    import torch

    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import Engine, StepEntry

    cfg = dict(model_cfg)
    cfg["num_hidden_layers"] = min(args.layers or 12, 12)
    B, T = args.batch, PREFILL_TOKENS
    behind = max(0, int(getattr(args, "behind", 0) or 0))          # tokens the prompt's request already holds
    ec = EngineConfig(dtype="bfloat16", page_size=args.page_size, max_cached_tokens=B * CONTEXT + T + behind, max_num_seqs=B + 1,
                      max_num_batched_tokens=T, max_model_len=max(CONTEXT, behind + T), use_cuda_graphs=False)
    eng = Engine(config=cfg, random_seed=0, engine_config=ec)
    gen = torch.Generator().manual_seed(0)
    names = [f"r{i}" for i in range(B)]
    for n in names:
        eng.step([StepEntry(n, torch.randint(0, 1000, (CACHED,), generator=gen).tolist(), [])])
        eng.cache.reserve(n, CACHED + 1)
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qs, kvs = nh * hd, nkv * hd

    plan = eng.model.plan(eng._caches)
    compiled = eng.ops.compile(plan)
    # the plan: one embedding record, then the same records for every layer, then the final norm and the head
    per_layer = (len(plan.ops) - 3) // L
    assert 1 + per_layer * L + 2 == len(plan.ops), "the layers of this model do not emit the same records"
    weights = {"linear": lambda a: a["w"].numel(), "linear_swiglu": lambda a: a["w_gate_up"].numel()}
    labels = {0: "rmsnorm + residual add (attention)", 1: "q|k|v product", 2: "qk norm + rope + cache write + attention",
              3: "output product", 4: "rmsnorm + residual add (feed-forward)", 5: "gate|up product + swiglu", 6: "down product"}

    def measure(j, batch, graph, reps=10):
        eng.rt.batch = batch

        def every_layer():
            for l in range(L):
                compiled.run(batch, 1 + l * per_layer + j, 1)
        every_layer()
        torch.cuda.synchronize()
        run = every_layer
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                every_layer()
            run = g.replay
        run()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            run()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps / L * 1000.0

    def table(batch, graph):
        rows, total = [], 0.0
        for j in range(per_layer):
            op = plan.ops[1 + j]
            us = measure(j, batch, graph)
            total += us
            w = weights.get(op.kind, lambda a: 0)(op.a)
            rows.append((labels.get(j, op.kind) if per_layer == 7 else op.kind, us, w))
        return rows, total

    print(f"# Time per operation of one layer, Qwen3 layer sizes {H}/{I}, {nh}/{nkv} heads of {hd}, bfloat16 ({L} layers "
          f"averaged, pages of {args.page_size})\n")
    print("Made by `python bench.py --breakdown`; CUDA events, warm; peaks: %s (%.0f GB/s, %.0f TFLOP/s).\n"
          % (pk["source"], pk["hbm_gbs"], pk["bf16_tflops"]))
    dec = eng._build_batch([StepEntry(n, [5], [0]) for n in names], [CACHED] * B)
    eng.cache.flush()
    rows, total = table(dec, True)
    print(f"## Decode step, batch {B}, {CACHED} cached tokens per request (inside a CUDA graph)\n")
    print("| operation | us per layer | weight bytes / time (GB/s) | share |\n|---|---|---|---|")
    for name, us, w in rows:
        print(f"| {name} | {us:.2f} | {('%.0f' % (2 * w / us / 1e3)) if w else ''} | {100 * us / total:.0f}% |")
    kv = B * CACHED * 2 * kvs * 2
    layer_weights = 2 * ((qs + 2 * kvs) * H + H * qs + 3 * H * I)
    print(f"| **sum** | **{total:.1f}** | | |\n\nAttention reads {kv / 1e6:.1f} MB of cache per layer; "
          f"the layer's weights are {layer_weights / 1e6:.0f} MB: at the peak "
          f"bandwidth the layer would take {(layer_weights + kv) / pk['hbm_gbs'] / 1e3:.1f} us.\n")
    if behind:
        ids = torch.randint(0, 1000, (behind,), generator=gen).tolist()
        for a in range(0, behind, T):
            eng.step([StepEntry("prefill", ids[a:a + T], [])])
    else:
        eng.cache.add_request("prefill")
    eng.cache.reserve("prefill", behind + T)
    pre = eng._build_batch([StepEntry("prefill", torch.randint(0, 1000, (T,), generator=gen).tolist(), [T - 1])], [behind])
    eng.cache.flush()
    rows, total = table(pre, True)
    print(f"## Prefill of one {T}-token prompt\n" if not behind else
          f"## A {T}-token portion of a prompt behind {behind} cached tokens\n")
    print("| operation | us per layer | TFLOP/s | share |\n|---|---|---|---|")
    for name, us, w in rows:
        fl = 2.0 * T * w if w else (4.0 * nh * hd * (T * behind + T * (T + 1) / 2) if "attention" in name and "rmsnorm" not in name else 0)
        print(f"| {name} | {us:.1f} | {('%.0f' % (fl / us / 1e6)) if fl else ''} | {100 * us / total:.0f}% |")
    print(f"| **sum** | **{total:.0f}** | | |")
    eng.check_kernels()
    return 0
