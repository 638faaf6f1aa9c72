#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one GPU, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 8b|14b|32b] [--mode decode|prefill|serve|sweep] [--no-extra] [--breakdown]

Headline (no --shape/--mode): Qwen3-8B layer sizes, random weights, bfloat16, cache pages of 16 tokens; a decode
step for a batch of 8 requests that each hold 2,048 cached tokens (context length 4,096: they could go on to
4,096), plus decode at batch 1 and 64 and a prefill of one 2,048-token prompt (median of 20 steps).  Token ids
are synthetic, uniform over the vocabulary; weights come from the engine's counter-based generator (the values
`python -m llmengine_b200.make_random_model` would write for seed 0).

`value` is decoded tokens per second timed on the device with CUDA events around exactly K steps (after W
warm-up steps).  `e2e` is the same through the Python entry point (`LLM.step`), host token ids in and host token
ids out every step, timed on the host clock around synchronised steps.  Every decode step reads all weights
(15 GB) and the live cache, far more than the L2 holds, so no explicit L2 flush is needed between steps.

Beside the headline the same line carries (`points`, `shapes`; skipped with --no-extra): the headline with the
engine's default pages of 64 tokens; a step that mixes a 121-token prompt portion with 7 decoded tokens, with
its host and device time; a read-only memory stream as a second bandwidth figure; continuous batching of 32
requests on the Qwen3-14B shape (prompts of 128 to 2,048 tokens, 256 new tokens each, portions of 512, through
`LLM.step`) with host and device time per step; and decode at batch 1/8/64 over 4,096-token contexts and a
2,048-token prefill on the Qwen3-32B shape.  `--shape`/`--mode` run one of these alone.

`--impl reference` times the unmodified reference project (built by baseline/build_reference.py) on the same
layer sizes through its own graph builder, CUDA executor and cache: see baseline/reference_bench.cpp.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _shape(layers, hidden, heads, inter):
    return {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
            "num_attention_heads": heads, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": inter,
            "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
            "max_position_embeddings": 40960, "hidden_act": "silu"}


SHAPES = {"8b": _shape(36, 4096, 32, 12288), "14b": _shape(40, 5120, 40, 17408), "32b": _shape(64, 5120, 64, 25600)}
MODEL_8B = SHAPES["8b"]
CONTEXT = 4096          # benchmark context length of the headline
CACHED = 2048           # tokens each request holds when the headline's decoding is timed
PAGE_SIZE = 16          # tokens per cache page of the headline (--page-size)
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


# ----------------------------------------------------------------------------- the reference arm
def reference_arm(args) -> int:
    """The unmodified reference on the headline's layer sizes: 8 sequences with 2,048 cached tokens each (put there
    by its own prefill), one new token for each per step, through its CudaExecutor."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import build_reference

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
        return 0

    binary = build_reference.BINARY
    if not os.path.exists(binary):
        try:
            binary = build_reference.build()
        except Exception as e:                                   # no sources, no cmake, or a compiler error: say which
            return unavailable(f"the reference could not be built here: {e}")
    cfg = SHAPES[args.shape or "8b"]
    clocks = ClockSampler()
    clocks.start()
    t0 = clocks.mark()
    cmd = [binary] + [str(cfg[k]) for k in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                                            "head_dim", "intermediate_size", "vocab_size")]
    cmd += [str(args.batch), str(CACHED), str(PREFILL_TOKENS), str(args.steps), str(max(args.warmup, 3))]
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    except (OSError, subprocess.TimeoutExpired) as e:
        clocks.stop()
        return unavailable(f"the reference's driver did not finish: {e}")
    t1 = clocks.mark()
    clocks.stop()
    line = (p.stdout.strip().splitlines() or [""])[-1]
    try:
        r = json.loads(line)
    except ValueError:
        return unavailable(f"the reference's driver exited with {p.returncode}: {(p.stderr or p.stdout)[-400:]}")
    if "error" in r:
        return unavailable(f"the reference's own code refused the workload: {r['error']}")
    ms = r["decode_ms_per_step"]
    rec = {
        "impl": "reference",
        "metric": "decode tokens/s, Qwen3-8B shape bf16, batch 8, 2048 cached tokens per request",
        "value": round(args.batch * 1000.0 / ms, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp32 (the reference computes in 32-bit; 32-bit weights take its library product, bfloat16 weights "
                 "would take its plain 16x16 kernel)",
        "data": "synthetic token ids, random weights",
        "config": {"model": "Qwen3-8B shape", "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": 8, "head_dim": 128,
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "cached_tokens": CACHED, "parallelism": "single GPU",
                   "batching": "one sequence per run, the batch decoded round-robin",
                   "l2": "inputs larger than L2 (33 GB of weights per token)"},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / r["prefill_ms"], 1), "tokens": PREFILL_TOKENS,
                    "ms": r["prefill_ms"]},
        "e2e": {"value": round(args.batch * 1000.0 / r["e2e_ms_per_step"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
        "gpu_launches": 0,
        "clocks": clocks.summary(t0, t1),
    }
    print(json.dumps(rec))
    return 0


# ----------------------------------------------------------------------------- sizes
def layer_params(cfg) -> int:
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * H * I + 2 * H + 2 * hd


def decode_bytes(cfg, batch: int, ctx: float) -> float:
    """What a decode step has to read: every weight it uses once (the embedding rows of its tokens included)
    and the cache of the live requests."""
    L, H, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["vocab_size"]
    weights = 2 * (L * layer_params(cfg) + V * H + H) + 2 * batch * H
    return weights + batch * ctx * L * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, T: int) -> float:
    L, H, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["vocab_size"]
    return 2.0 * T * L * layer_params(cfg) + 2.0 * V * H + L * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * T * (T + 1) / 2


# ----------------------------------------------------------------------------- measuring
class Bench:
    """One engine of one shape, and the measurements that run on it."""

    def __init__(self, cfg, page_size: int, max_batch: int, context: int, budget: int, chunk: int, graphs: bool = True,
                 max_cached_tokens: int = 0):
        import torch

        from llmengine_b200 import LLM, SamplingParams
        from llmengine_b200.config import EngineConfig

        self.torch, self.cfg = torch, cfg
        ec = EngineConfig(dtype="bfloat16", page_size=page_size, max_cached_tokens=max_cached_tokens or max_batch * context,
                          max_num_seqs=max_batch, max_num_batched_tokens=max(budget, max_batch), prefill_chunk=chunk,
                          max_model_len=context, use_cuda_graphs=graphs)
        self.llm = LLM(config=cfg, random_seed=0, engine_config=ec)
        self.eng, self.ops = self.llm.engine, self.llm.engine.ops
        self.gen = torch.Generator().manual_seed(0)
        self.greedy = SamplingParams(greedy=True)
        self.counter = 0

    def close(self):
        self.llm = self.eng = self.ops = None
        gc.collect()
        self.torch.cuda.empty_cache()

    def tokens(self, n):
        return self.torch.randint(0, self.cfg["vocab_size"], (n,), generator=self.gen).tolist()

    def timed(self, fn, steps, warmup):
        """Mean milliseconds per call over `steps` calls, CUDA events on the launching stream, after `warmup` calls."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = self.ops.launches
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps, self.ops.launches - l0

    def prefill(self, tokens: int, reps: int = 20, warmup: int = 3) -> float:
        """Median milliseconds of a step that runs one prompt of `tokens` tokens (each step timed by itself)."""
        from llmengine_b200.engine.engine import StepEntry
        torch = self.torch
        prompt = self.tokens(tokens)
        times = []
        for i in range(warmup + reps):
            name = f"p{self.counter}"
            self.counter += 1
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self.eng.step([StepEntry(name, prompt, [tokens - 1])], end=[name])
            b.record()
            torch.cuda.synchronize()
            if i >= warmup:
                times.append(a.elapsed_time(b))
        return statistics.median(times)

    def fill(self, names, cached: int) -> None:
        """Requests that hold `cached` tokens each, put there by real prompt steps."""
        from llmengine_b200.engine.engine import StepEntry
        cut = self.eng.ec.max_num_batched_tokens
        for n in names:
            ids = self.tokens(cached)
            for a in range(0, cached, cut):
                self.eng.step([StepEntry(n, ids[a:a + cut], [])])

    def decode(self, batch: int, cached: int, steps: int, warmup: int, clocks=None):
        from llmengine_b200.engine.engine import StepEntry
        names = [f"d{self.counter}_{i}" for i in range(batch)]
        self.counter += 1
        self.fill(names, cached)
        feed = [self.tokens(1) for _ in range(batch)]

        def one():
            logits = self.eng.step([StepEntry(n, t, [0]) for n, t in zip(names, feed)])
            self.llm.sampler.sample(logits, [self.greedy] * batch, [0] * batch)

        t0 = clocks.mark() if clocks else 0
        ms, launches = self.timed(one, steps, warmup)
        t1 = clocks.mark() if clocks else 0
        ctx = cached + warmup + steps // 2              # mean cached length over the timed steps
        for n in names:
            self.eng.free(n)
        return ms, launches, ctx, (t0, t1)

    def end_to_end(self, batch: int, cached: int, steps: int, warmup: int):
        """Decoded tokens per second through `LLM.step`: host token ids in, host token ids out, every step."""
        llm, torch = self.llm, self.torch
        # a request decodes while the prompts behind it are still being read: room for those tokens too, so that
        # none ends inside the timed steps
        ids = [llm.add_request(self.tokens(cached), self.greedy, max_tokens=warmup + steps + 2 * batch + 8, eos_token_id=None)
               for _ in range(batch)]
        while any(llm.scheduler.state(i).phase.value != "decoding" for i in ids):
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()                               # ends with the device-to-host read of the sampled tokens
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        out = {"value": round(batch * steps / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(self.eng._meta_len * 4 + llm.sampler._hosts[0].numel() * 4),
               "d2h_bytes_per_step": int(batch * 4)}
        while not llm.scheduler.all_done() or llm._inflight is not None:
            llm.step()
        return out

    def mixed_step(self, decoders: int, portion: int, cached: int, reps: int = 20):
        """A step of `decoders` single tokens beside one prompt portion of `portion` tokens: host milliseconds (the
        time `Engine.step` takes to return) and device milliseconds (CUDA events around it), medians."""
        from llmengine_b200.engine.engine import StepEntry
        torch = self.torch
        names = [f"m{self.counter}_{i}" for i in range(decoders)]
        self.counter += 1
        self.fill(names, cached)
        host, dev = [], []
        prompt = self.tokens(portion)
        for i in range(reps + 3):
            p = f"mp{self.counter}"
            self.counter += 1
            entries = [StepEntry(n, self.tokens(1), [0]) for n in names] + [StepEntry(p, prompt, [portion - 1])]
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            a.record()
            self.eng.step(entries, end=[p])
            b.record()
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            if i >= 3:
                host.append((t1 - t0) * 1e3)
                dev.append(a.elapsed_time(b))
        for n in names:
            self.eng.free(n)
        return {"tokens": decoders + portion, "host_ms": round(statistics.median(host), 3),
                "gpu_ms": round(statistics.median(dev), 3)}

    def serve(self, n_requests: int, lo: int, hi: int, new_tokens: int):
        """Continuous batching through `LLM.step`: all requests submitted at once, run until all are done."""
        llm, torch = self.llm, self.torch
        lens = torch.randint(lo, hi + 1, (n_requests,), generator=self.gen).tolist()
        for n in lens:
            llm.add_request(self.tokens(n), self.greedy, max_tokens=new_tokens, eos_token_id=None)
        torch.cuda.synchronize()
        events, host_ms, mix = [], [], []
        done = 0
        t0 = time.perf_counter()
        while done < n_requests:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before = self.eng.steps
            h0 = time.perf_counter()
            a.record()
            done += len(llm.step())
            b.record()
            host_ms.append((time.perf_counter() - h0) * 1e3)
            events.append((a, b))
            mix.append(self.eng.steps - before)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        gpu_ms = [a.elapsed_time(b) for a, b in events]
        generated = n_requests * new_tokens
        steps = len(host_ms)
        return {"requests": n_requests, "prompt_tokens": int(sum(lens)), "generated_tokens": generated,
                "seconds": round(wall, 3), "generated_tokens_per_s": round(generated / wall, 1),
                "total_tokens_per_s": round((generated + sum(lens)) / wall, 1), "steps": steps,
                "tokens_per_step": round((generated + sum(lens)) / max(1, self.eng.steps), 1),
                "host_ms_per_step": round(statistics.mean(host_ms), 3), "gpu_ms_per_step": round(statistics.mean(gpu_ms), 3),
                "host_ms_median": round(statistics.median(host_ms), 3), "gpu_ms_median": round(statistics.median(gpu_ms), 3)}

    def read_peak(self, gigabytes: float = 4.0, reps: int = 10) -> float:
        """GB/s of a kernel that only reads: this package's read_stream over a buffer far larger than the L2."""
        torch = self.torch
        buf = torch.empty(int(gigabytes * (1 << 30)) // 4, dtype=torch.int32, device="cuda").fill_(1)
        sink = torch.zeros(1, dtype=torch.int32, device="cuda")
        best = 0.0
        for _ in range(3):
            self.ops.read_stream(buf, sink)
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self.ops.read_stream(buf, sink)
            b.record()
            torch.cuda.synchronize()
            best = max(best, buf.numel() * 4 / (a.elapsed_time(b) * 1e-3) / 1e9)
        del buf
        return best


def shape_record(cfg, layers):
    return {"layers": layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"]}


def run_decode_prefill(name, cfg, batches, cached, context, page, steps, warmup, pk, do_prefill=True, do_decode=True):
    """Decode at the given batch sizes over `cached`-token contexts and one prefill, on a fresh engine."""
    b = Bench(cfg, page, max(batches) if do_decode else 1, context, max(PREFILL_TOKENS, 2048), PREFILL_TOKENS)
    out = dict(shape_record(cfg, cfg["num_hidden_layers"]), page_size=page, cached_tokens=cached)
    if do_prefill:
        ms = b.prefill(PREFILL_TOKENS, reps=20 if name != "32b" else 10)
        fl = prefill_flops(cfg, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1000.0 / ms, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                          "frac": round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    if do_decode:
        for batch in batches:
            ms, _, ctx, _ = b.decode(batch, cached, steps if batch <= 8 else max(10, steps // 2), warmup)
            ach = decode_bytes(cfg, batch, ctx) / (ms * 1e-3) / 1e9
            out[f"decode_b{batch}"] = {"value": round(batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
                                       "hbm_gbs": round(ach, 1), "frac": round(ach / pk["hbm_gbs"], 4)}
    b.eng.check_kernels()
    b.close()
    return out


def long_prompt_flops(cfg, T: int) -> float:
    """A prompt of T tokens whose logits are wanted at its last place only."""
    return prefill_flops(cfg, T)


def run_sweep(cfg, page, steps, warmup, pk):
    """Further sizes: decode at batch 1 / 8 / 32 over 512 to 32,768 cached tokens, and whole prompts of 256 to 32,768
    tokens run in portions of 2,048; each as a fraction of its roofline (bytes of weights and live cache / time / copy
    bandwidth; flops / time / burst peak)."""
    from llmengine_b200.engine.engine import StepEntry
    contexts, batches, prompts = [512, 2048, 8192, 32768], [1, 8, 32], [256, 1024, 2048, 8192, 32768]
    longest = max(contexts) + 256
    b = Bench(cfg, page, max(batches), longest, 2048, 2048)
    torch = b.torch
    out = dict(shape_record(cfg, cfg["num_hidden_layers"]), page_size=page, decode={}, prefill={})
    for cached in contexts:
        for batch in batches:
            ms, _, ctx, _ = b.decode(batch, cached, steps, warmup)
            ach = decode_bytes(cfg, batch, ctx) / (ms * 1e-3) / 1e9
            out["decode"][f"ctx{cached}_b{batch}"] = {"ms": round(ms, 4), "frac": round(ach / pk["hbm_gbs"], 3)}
    for T in prompts:
        ids, times = b.tokens(T), []
        for i in range(2 + 5):
            name = f"s{b.counter}"
            b.counter += 1
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for a in range(0, T, 2048):
                part = ids[a:a + 2048]
                last = a + 2048 >= T
                b.eng.step([StepEntry(name, part, [len(part) - 1] if last else [])], end=[name] if last else [])
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        out["prefill"][f"t{T}"] = {"ms": round(ms, 3), "tokens_per_s": round(T * 1000.0 / ms, 1),
                                   "frac": round(long_prompt_flops(cfg, T) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3)}
    b.eng.check_kernels()
    b.close()
    return out


def run_serve(cfg, page, pk):
    b = Bench(cfg, page, 32, 2048 + 256 + 64, 1024, 512, max_cached_tokens=32 * (2048 + 256 + 64))
    b.serve(4, 128, 512, 16)                      # warm-up: compiles, captures, allocates
    out = dict(shape_record(cfg, cfg["num_hidden_layers"]), page_size=page, prefill_chunk=512, token_budget=1024)
    out.update(b.serve(32, 128, 2048, 256))
    b.eng.check_kernels()
    b.close()
    return out


def main() -> int:
    global PAGE_SIZE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default=None, choices=sorted(SHAPES), help="run one shape alone (with --mode)")
    ap.add_argument("--mode", default=None, choices=["decode", "prefill", "serve", "sweep"],
                    help="sweep: decode over 512 to 32,768 cached tokens at batch 1 / 8 / 32 and prompts of 256 to 32,768 "
                         "tokens (give --layers 4: the full depth does not leave room for the longest contexts' cache)")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the shape has (the record then names both numbers)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-graphs", action="store_true", help="do not capture decode steps in CUDA graphs")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--no-extra", "--skip-points", dest="no_extra", action="store_true",
                    help="the headline only: no further page size, shapes or probes")
    ap.add_argument("--behind", type=int, default=0,
                    help="with --breakdown: the timed prompt portion lies behind this many cached tokens of its request")
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
        from llmengine_b200.breakdown import breakdown
        return breakdown(args, SHAPES[args.shape or "8b"], CACHED, CONTEXT, PREFILL_TOKENS, peaks())
    pk = peaks()

    # ---- one shape and mode alone
    if args.shape or args.mode:
        name = args.shape or "8b"
        cfg = dict(SHAPES[name])
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        mode = args.mode or "decode"
        if mode == "sweep":
            rec = {"metric": f"roofline fractions at further sizes, Qwen3-{name.upper()} shape bf16",
                   "sweep": run_sweep(cfg, PAGE_SIZE, min(args.steps, 32), args.warmup, pk)}
            rec["value"], rec["unit"] = rec["sweep"]["decode"]["ctx2048_b8"]["frac"], "fraction of the copy bandwidth"
        elif mode == "serve":
            rec = {"metric": f"continuous batching, Qwen3-{name.upper()} shape bf16: 32 requests, prompts 128-2048, 256 new tokens",
                   "serve": run_serve(cfg, PAGE_SIZE, pk)}
            rec["value"], rec["unit"] = rec["serve"]["generated_tokens_per_s"], "tokens/s"
        else:
            cached = 4096 if name == "32b" else CACHED
            r = run_decode_prefill(name, cfg, [1, 8, 64], cached, 2 * cached if name != "32b" else 4096 + 256, PAGE_SIZE,
                                   args.steps, args.warmup, pk, do_prefill=mode == "prefill", do_decode=mode == "decode")
            rec = {"metric": f"{mode} tokens/s, Qwen3-{name.upper()} shape bf16", mode: r}
            rec["value"] = r["prefill"]["value"] if mode == "prefill" else r["decode_b8"]["value"]
            rec["unit"] = "tokens/s"
        rec.update({"n_gpus": 1, "dtype": "bf16", "data": "synthetic token ids, random weights", "peaks": pk["source"],
                    "layers_of_model": SHAPES[name]["num_hidden_layers"]})
        print(json.dumps(rec))
        return 0

    # ---- the headline
    cfg = dict(MODEL_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    max_batch = 64 if not args.no_extra else args.batch
    clocks = ClockSampler()
    clocks.start()
    b = Bench(cfg, PAGE_SIZE, max_batch, CONTEXT, PREFILL_TOKENS, PREFILL_TOKENS, graphs=not args.no_graphs)
    prefill_ms = b.prefill(PREFILL_TOKENS, reps=20)
    ms, launches, ctx, window = b.decode(args.batch, CACHED, args.steps, args.warmup, clocks)
    points, shapes, e2e = {}, {}, None
    if not args.no_extra:
        for n in (1, 64):
            m, _, _, _ = b.decode(n, CACHED, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{n}"] = round(n * 1000.0 / m, 1)
    e2e = b.end_to_end(args.batch, CACHED, args.steps, args.warmup)
    graphs_on = bool(getattr(b.eng, "graphs_enabled", False))
    if not args.no_extra:
        mixed = b.mixed_step(7, 121, CACHED)
        points["mixed128_host_ms"], points["mixed128_gpu_ms"] = mixed["host_ms"], mixed["gpu_ms"]
        points["hbm_read_gbs"] = round(b.read_peak(), 1)
    b.eng.check_kernels()
    b.close()
    clocks.stop()

    achieved = decode_bytes(cfg, args.batch, ctx) / (ms * 1e-3) / 1e9
    T = PREFILL_TOKENS
    flops = prefill_flops(cfg, T)
    prefill = {"value": round(T * 1000.0 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    if "bf16_tflops_sustained" in pk:
        prefill["frac_sustained"] = round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    if not args.no_extra:
        other = 64 if PAGE_SIZE != 64 else 16
        r = run_decode_prefill("8b", cfg, [args.batch], CACHED, CONTEXT, other, args.steps, args.warmup, pk, do_prefill=True)
        points[f"decode_b{args.batch}_page{other}"] = r[f"decode_b{args.batch}"]["value"]
        points[f"prefill_page{other}"] = r["prefill"]["value"]
        if not args.layers:
            shapes["14b_serve"] = run_serve(SHAPES["14b"], PAGE_SIZE, pk)
            points["serve_14b_generated_tok_s"] = shapes["14b_serve"]["generated_tokens_per_s"]
            shapes["32b"] = run_decode_prefill("32b", SHAPES["32b"], [1, 8, 64], 4096, 4096 + 256, PAGE_SIZE,
                                               max(16, args.steps // 2), args.warmup, pk)
            for n in (1, 8, 64):
                points[f"decode32b_b{n}"] = shapes["32b"][f"decode_b{n}"]["value"]
            points["prefill32b"] = shapes["32b"]["prefill"]["value"]

    value = args.batch * 1000.0 / ms
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    rec = {
        "metric": "decode tokens/s, Qwen3-8B shape bf16, batch 8, 2048 cached tokens per request",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random weights from the engine's counter-based generator (seed 0)",
        "config": {
            "model": "Qwen3-8B shape", "layers": cfg["num_hidden_layers"], "layers_of_model": MODEL_8B["num_hidden_layers"],
            "hidden": H, "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": I, "vocab": V,
            "global_batch": args.batch, "seq_len": CONTEXT, "cached_tokens": CACHED, "page_size": PAGE_SIZE,
            "parallelism": "single GPU", "cuda_graphs": graphs_on,
            "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": pk["source"],
        },
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "shapes": shapes,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "clocks": clocks.summary(*window),
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
