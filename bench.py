#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one GPU, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the third configuration of BASELINE.json): Qwen3-8B layer sizes, random weights,
bfloat16; a decode step for a batch of 8 requests that each hold 2,048 cached tokens (context
length 4,096: they could go on to 4,096), plus decode at batch 1 and 64 and one prefill of a
2,048-token prompt.  Token ids are synthetic, uniform over the vocabulary.

`value` is decoded tokens per second timed on the device with CUDA events around exactly K
steps (after W warm-up steps).  `e2e` is the same through the Python entry point (`LLM.step`),
host token ids in and host token ids out every step, timed on the host clock around
synchronised steps.  Every decode step reads all weights (15 GB) and the live cache, far more
than the L2 holds, so no explicit L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_8B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960, "hidden_act": "silu",
}
CONTEXT = 4096          # benchmark context length
CACHED = 2048           # tokens each request holds when decoding is timed
PAGE_SIZE = 64          # tokens per cache page (--page-size)
PREFILL_TOKENS = 2048


def peaks():
    """Measured peaks of this pool if the driver wrote them, else the fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(path) as f:
            d = json.load(f)
        if "hbm_gbs" in d:
            out["hbm_gbs"] = float(d["hbm_gbs"])
        if "bf16_tflops" in d:
            out["bf16_tflops"] = float(d["bf16_tflops"])
        if "bf16_tflops_sustained" in d:                 # the same product looped for seconds under the power cap
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", "0", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0, t1):
        sm, mx, reasons = [], [], set()
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    # The reference is a CMake/C++ project without any Python packaging (no setup.py, no pyproject.toml),
    # so an offline `pip install --target baseline/_ref <the reference's source tree>` has nothing to build; its
    # generate_cuda example also needs a GGUF file with tokenizer metadata and runs one sequence at a
    # time, so the batch-8 metric on random Qwen3-8B weights cannot be produced through its stock path.
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a CMake C++ project with no Python package to pip-install offline, and its "
                      "stock generate path needs a GGUF model file with tokenizer and decodes one sequence at a time"}))
    return 0


def breakdown(args) -> int:
    """Time of each operation of one layer, averaged over the layers (each layer has weights of its own, so
    nothing is served from L2 that a real step would read from HBM).  Decode operations are timed as a
    CUDA graph that launches the operation once per layer; prefill operations as eager launches."""
    import torch

    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import Engine, StepEntry

    cfg = dict(MODEL_8B)
    cfg["num_hidden_layers"] = min(args.layers, 12)
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

    pk = peaks()
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


def main() -> int:
    global PAGE_SIZE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL_8B["num_hidden_layers"],
                    help="fewer layers than the model has (the record then names both numbers)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-graphs", action="store_true", help="do not capture decode steps in CUDA graphs")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 / 64 and the end-to-end run")
    ap.add_argument("--breakdown", action="store_true",
                    help="instead of the bench line, print the time of every operation of a layer (decode at --batch "
                         "inside a CUDA graph, and a 2,048-token prefill), timed with CUDA events")
    args = ap.parse_args()
    PAGE_SIZE = args.page_size
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.breakdown:
        return breakdown(args)

    import torch

    from llmengine_b200 import LLM, SamplingParams
    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import StepEntry

    cfg = dict(MODEL_8B)
    cfg["num_hidden_layers"] = args.layers
    max_batch = 64 if not args.skip_points else args.batch
    ec = EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE, max_cached_tokens=max_batch * CONTEXT, max_num_seqs=max_batch,
                      max_num_batched_tokens=max(PREFILL_TOKENS, max_batch), prefill_chunk=PREFILL_TOKENS,
                      max_model_len=CONTEXT, use_cuda_graphs=not args.no_graphs)
    llm = LLM(config=cfg, random_seed=0, engine_config=ec)
    eng = llm.engine
    ops = eng.ops
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    def tokens(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ops.launches
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps, ops.launches - l0

    clocks = ClockSampler()
    clocks.start()

    # ---- prefill: one 2,048-token prompt per step (each leaves a request with 2,048 cached tokens)
    prompt = tokens(PREFILL_TOKENS)
    counter = [0]

    def prefill_once():
        name = f"p{counter[0]}"
        counter[0] += 1
        eng.step([StepEntry(name, prompt, [PREFILL_TOKENS - 1])], end=[name])

    prefill_ms, _ = timed(prefill_once, 5, 3)

    # ---- decode at a given batch: requests that hold CACHED tokens, one new token each per step
    sp = SamplingParams(greedy=True)

    def decode_bench(batch, steps, warmup):
        names = [f"d{batch}_{i}" for i in range(batch)]
        for n in names:
            eng.step([StepEntry(n, tokens(CACHED), [])])
        feed = [tokens(1) for _ in range(batch)]

        def one():
            logits = eng.step([StepEntry(n, t, [0]) for n, t in zip(names, feed)])
            llm.sampler.sample(logits, [sp] * batch, [0] * batch)

        t0 = clocks.mark()
        ms, launches = timed(one, steps, warmup)
        t1 = clocks.mark()
        ctx = CACHED + warmup + steps // 2          # mean cached length over the timed steps
        for n in names:
            eng.free(n)
        return ms, launches, ctx, (t0, t1)

    ms, launches, ctx, window = decode_bench(args.batch, args.steps, args.warmup)
    points = {}
    e2e = None
    if not args.skip_points:
        for b in (1, 64):
            m, _, _, _ = decode_bench(b, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / m, 1)

        # ---- end to end through the Python entry point: host tokens in, host tokens out, every step
        # (a request decodes while the prompts behind it are still being read: room for those tokens too, so that
        # none ends inside the timed steps)
        ids = [llm.add_request(tokens(CACHED), sp, max_tokens=args.warmup + args.steps + 2 * args.batch + 8, eos_token_id=None)
               for _ in range(args.batch)]
        while any(llm.scheduler.state(i).phase.value != "decoding" for i in ids):
            llm.step()
        for _ in range(args.warmup):
            llm.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            llm.step()                               # ends with the device-to-host read of the sampled tokens
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        e2e = {"value": round(args.batch * args.steps / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(eng._meta_len * 4 + llm.sampler._hosts[0].numel() * 4),
               "d2h_bytes_per_step": int(args.batch * 4)}
    clocks.stop()

    # ---- roofline of the decode step: every weight it uses once + the cache of the live requests
    L, H, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * H * I + 2 * H + 2 * hd
    weight_bytes = 2 * (L * per_layer + V * H + H) + 2 * args.batch * H       # + the embedding rows that are read
    kv_bytes = args.batch * ctx * L * 2 * nkv * hd * 2
    pk = peaks()
    achieved = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * L * per_layer + 2 * V * H + L * 4 * nh * hd * T * (T + 1) / 2
    prefill = {"value": round(T * 1000.0 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    if "bf16_tflops_sustained" in pk:
        prefill["frac_sustained"] = round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    value = args.batch * 1000.0 / ms
    rec = {
        "metric": "decode tokens/s, Qwen3-8B shape bf16, batch 8, 2048 cached tokens per request",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random weights",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_of_model": MODEL_8B["num_hidden_layers"],
            "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
            "global_batch": args.batch, "seq_len": CONTEXT, "cached_tokens": CACHED, "page_size": PAGE_SIZE,
            "parallelism": "single GPU", "cuda_graphs": bool(getattr(eng, "graphs_enabled", False)),
            "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": pk["source"],
        },
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "clocks": clocks.summary(*window),
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
