"""Time of each operation of one layer (`python bench.py --breakdown`): decode operations inside a CUDA graph
that launches the operation once per layer, prefill operations as eager launches, CUDA events around both."""
from __future__ import annotations


def breakdown(args, model_cfg, CACHED, CONTEXT, PREFILL_TOKENS, pk) -> int:
    """Time of each operation of one layer, averaged over the layers (each layer has weights of its own, so
    nothing is served from L2 that a real step would read from HBM).  Decode operations are timed as a
    CUDA graph that launches the operation once per layer; prefill operations as eager launches."""
    import torch

    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import Engine, StepEntry

    cfg = dict(model_cfg)
    cfg["num_hidden_layers"] = min(args.layers or 12, 12)
    PAGE_SIZE = args.page_size
    B, T = args.batch, PREFILL_TOKENS
    ec = EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE, max_cached_tokens=B * CONTEXT + T, max_num_seqs=B + 1,
                      max_num_batched_tokens=T, max_model_len=CONTEXT, use_cuda_graphs=False)
    eng = Engine(config=cfg, random_seed=0, engine_config=ec)
    ops, blocks = eng.ops, eng.model.blocks
    gen = torch.Generator().manual_seed(0)
    names = [f"r{i}" for i in range(B)]
    for n in names:
        eng.step([StepEntry(n, torch.randint(0, 1000, (CACHED,), generator=gen).tolist(), [])])
        eng.cache.reserve(n, CACHED + 1)
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qs, kvs = nh * hd, nkv * hd

    def measure(fn, graph, reps=10):
        for l in range(len(blocks)):
            fn(l)
        torch.cuda.synchronize()
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for l in range(len(blocks)):
                    fn(l)
            run = g.replay
        else:
            def run():
                for l in range(len(blocks)):
                    fn(l)
        run()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            run()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps / len(blocks) * 1000.0

    def layer_ops(batch, rows, graph):
        x = torch.randn(rows, H, device="cuda")
        delta = torch.randn(rows, H, device="cuda")
        h = torch.randn(rows, H, device="cuda").bfloat16()
        qkv = torch.empty(rows, qs + 2 * kvs, device="cuda", dtype=torch.bfloat16)
        q = torch.empty(rows, qs, device="cuda", dtype=torch.bfloat16)
        ao = torch.empty(rows, qs, device="cuda", dtype=torch.bfloat16)
        mo = torch.empty(rows, H, device="cuda")
        act = torch.empty(rows, I, device="cuda", dtype=torch.bfloat16)
        grp = batch.groups[0]

        def post(l):
            m = blocks[l].mixer
            ops.qkv_post(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs], v_in=qkv[:, qs + kvs:], num_heads=nh,
                         num_kv_heads=nkv, head_dim=hd, q_gain=m.q_gain, k_gain=m.k_gain, eps=m.eps,
                         cos_sin=m.position.rotary_table(), positions=batch.positions, q_out=q,
                         cache=eng._caches[l].kv, slot_mapping=grp.slot_mapping, page_size=grp.page_size)

        def fused_attention(l):
            m = blocks[l].mixer
            n_dec = batch.decode_rows.numel()
            splits = m.decode_splits(n_dec, batch.max_decode_ctx)
            scratch = None
            if splits > 1:
                need = ops.attention_decode_scratch_floats(hd, n_dec, nh, splits)
                scratch = eng.rt.buffer("attention_scratch", 1, need, torch.float32, exact=True, zero=True)
            ops.attention_decode_fused(qkv=qkv, q_gain=m.q_gain, k_gain=m.k_gain, eps=m.eps, cos_sin=m.position.rotary_table(),
                                       write_kv=True, cache=eng._caches[l].kv, out=ao, rows=batch.decode_rows,
                                       cu_q_lens=batch.cu_q_lens, ctx_lens=batch.ctx_lens, table_rows=batch.state_slots,
                                       block_tables=grp.block_tables, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                       page_size=grp.page_size, window=0, scale=m.scale, splits=splits, scratch=scratch)

        table = [
            ("rmsnorm + residual add (attention)", lambda l: blocks[l].mixer_norm.forward(x, delta=delta), 0),
            ("q|k|v product", lambda l: ops.linear(h, blocks[l].mixer.w_qkv, qkv), (qs + 2 * kvs) * H),
        ]
        if graph:       # a decode step: norm, rotation and cache write happen inside the attention kernel
            table.append(("qk norm + rope + cache write + attention", fused_attention, 0))
        else:
            table.append(("qk norm + rope + cache write", post, 0))
            table.append(("attention", lambda l: blocks[l].mixer.attend(q, eng._caches[l].kv, ao, batch, grp), 0))
        table += [
            ("output product", lambda l: ops.linear(ao, blocks[l].mixer.w_o, mo), H * qs),
            ("rmsnorm + residual add (feed-forward)", lambda l: blocks[l].ffn_norm.forward(x, delta=mo), 0),
        ]
        if ops.linear_swiglu_supports(h, blocks[0].ffn.w_gate_up, act):
            table.append(("gate|up product + swiglu", lambda l: ops.linear_swiglu(h, blocks[l].ffn.w_gate_up, act), 2 * I * H))
        else:                                  # where no fused kernel is taken: the library product, then the activation
            gu = torch.empty(rows, 2 * I, device="cuda", dtype=torch.bfloat16)
            table.append(("gate|up product", lambda l: ops.linear(h, blocks[l].ffn.w_gate_up, gu), 2 * I * H))
            table.append(("swiglu", lambda l: ops.swiglu(gu, act), 0))
        table += [
            ("down product", lambda l: ops.linear(act, blocks[l].ffn.w_down, mo), H * I),
        ]
        out, total = [], 0.0
        for name, fn, weights in table:
            us = measure(fn, graph)
            total += us
            out.append((name, us, weights))
        return out, total

    print(f"# Time per operation of one layer, Qwen3-8B layer sizes, bfloat16 ({len(blocks)} layers averaged)\n")
    print("Made by `python bench.py --breakdown`; CUDA events, warm; peaks: %s (%.0f GB/s, %.0f TFLOP/s).\n"
          % (pk["source"], pk["hbm_gbs"], pk["bf16_tflops"]))
    dec = eng._build_batch([StepEntry(n, [5], [0]) for n in names], [CACHED] * B)
    eng.cache.flush()
    rows, total = layer_ops(dec, B, True)
    print(f"## Decode step, batch {B}, {CACHED} cached tokens per request (inside a CUDA graph)\n")
    print("| operation | us per layer | weight bytes / time (GB/s) | share |\n|---|---|---|---|")
    for name, us, w in rows:
        print(f"| {name} | {us:.2f} | {('%.0f' % (2 * w / us / 1e3)) if w else ''} | {100 * us / total:.0f}% |")
    kv = B * CACHED * 2 * kvs * 2
    print(f"| **sum** | **{total:.1f}** | | |\n\nAttention reads {kv / 1e6:.1f} MB of cache per layer; "
          f"the layer's weights are {2 * ((qs + 2 * kvs) * H + H * qs + 3 * H * I) / 1e6:.0f} MB: at the peak "
          f"bandwidth the layer would take {(2 * ((qs + 2 * kvs) * H + H * qs + 3 * H * I) + kv) / pk['hbm_gbs'] / 1e3:.1f} us.\n")
    eng.cache.add_request("prefill")
    eng.cache.reserve("prefill", T)
    pre = eng._build_batch([StepEntry("prefill", torch.randint(0, 1000, (T,), generator=gen).tolist(), [T - 1])], [0])
    eng.cache.flush()
    rows, total = layer_ops(pre, T, False)
    print(f"## Prefill of one {T}-token prompt\n")
    print("| operation | us per layer | TFLOP/s | share |\n|---|---|---|---|")
    for name, us, w in rows:
        fl = 2.0 * T * w if w else (4.0 * nh * hd * T * (T + 1) / 2 if name == "attention" else 0)
        print(f"| {name} | {us:.1f} | {('%.0f' % (fl / us / 1e6)) if fl else ''} | {100 * us / total:.0f}% |")
    print(f"| **sum** | **{total:.0f}** | | |")
    eng.check_kernels()
    return 0


