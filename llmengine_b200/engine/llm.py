"""The Python entry point: a model folder in, generated tokens out.

`LLM.generate` is the loop that the reference's examples spell out by hand (prefill, take the
logits of the last prompt token, sample, then one token a step until EOS or max_tokens:
examples/generate.cpp:236-347), run for many requests at once through the scheduler and the
step function.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config import EngineConfig
from ..sampling import Sampler, SamplingParams
from .engine import Engine, StepEntry
from .scheduler import ContinuousBatchScheduler, SequenceOutput, SequenceRequest


@dataclass
class GenerationOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]


class LLM:
    def __init__(self, model: Optional[str] = None, *, dtype: str = "bfloat16", config=None,
                 random_seed: Optional[int] = None, engine_config: Optional[EngineConfig] = None, ops=None,
                 pipeline_decode: bool = True, **engine_options):
        """`model`: a folder with config.json and model.safetensors (or `config` + `random_seed` for
        random weights).  Further keyword arguments are fields of `EngineConfig`."""
        ec = engine_config or EngineConfig(dtype=dtype, **engine_options)
        self.engine = Engine(model, config=config, random_seed=random_seed, engine_config=ec, ops=ops)
        self.scheduler = ContinuousBatchScheduler(self.engine.cache, ec.max_num_seqs, ec.max_num_batched_tokens,
                                                  ec.prefill_chunk)
        self.sampler = Sampler(self.engine.ops, self.engine.device, ec.max_num_seqs)
        self.eos_token_id = getattr(self.engine.config, "eos_token_id", None)
        self.default_seed = ec.seed
        self.pipeline_decode = pipeline_decode
        self._inflight = None
        pin = self.engine.device.type == "cuda"
        self._token_ring = [torch.zeros(ec.max_num_seqs, dtype=torch.int32, pin_memory=pin) for _ in range(4)]
        self._token_turn = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None,
                    max_tokens: int = 64, request_id: int = -1, eos_token_id: Union[int, None, str] = "model") -> int:
        sp = sampling_params or SamplingParams(seed=self.default_seed)
        eos = self.eos_token_id if eos_token_id == "model" else eos_token_id
        for t in prompt_token_ids:
            if not 0 <= int(t) < self.engine.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary [0, {self.engine.vocab_size})")
        return self.scheduler.submit(SequenceRequest(list(prompt_token_ids), max_tokens, request_id, sp, eos))

    def step(self) -> List[SequenceOutput]:
        """Admit, run one batch, sample, finish.  Returns the requests that are known to have finished.

        With `pipeline_decode` (the default) a step whose batch can be foreseen is launched before the
        host has read the tokens of the step before it: its input tokens are taken on the device from
        that step's sampler output.  The host then reads the earlier step's tokens while the GPU already
        works on the next one, so a request's tokens (and its finishing) become known one step late, and
        a request that ends on an end-of-sequence token costs one wasted token of compute."""
        sch = self.scheduler
        prev = self._inflight
        if prev is not None:
            self._inflight = self._launch_successor(prev) if self.pipeline_decode else None
            self._resolve(prev)
            return sch.collect_finished()
        sch.admit_waiting()
        entries = sch.schedule()
        if not entries:
            return sch.collect_finished()
        rec = self._launch(entries, None)
        if self.pipeline_decode:
            self._inflight = rec
        else:
            self._resolve(rec)
        return sch.collect_finished()

    # ------------------------------------------------------------------ launching and resolving steps
    def _launch(self, entries, device_tokens):
        """Queue one step and its sampling on the device; returns the record needed to read its tokens."""
        sch = self.scheduler
        batch = [StepEntry(e.sequence_id, e.tokens, [len(e.tokens) - 1] if e.samples else []) for e in entries]
        logits = self.engine.step(batch, device_tokens=device_tokens)
        rows = [e for e in entries if e.samples]
        rec = {"entries": entries, "rows": rows, "tokens": None, "host": None, "event": None}
        if rows:
            states = [sch.state(e.sequence_id) for e in rows]
            pending = 1 if device_tokens is not None else 0     # a token of the step before is not yet in the lists
            tokens = self.sampler.sample(logits, [s.sampling for s in states],
                                         [len(s.generated_tokens) + pending for s in states],
                                         [s.token_counts for s in states])
            rec["tokens"] = tokens
            if self.engine.device.type == "cuda":
                host = self._token_ring[self._token_turn]
                self._token_turn = (self._token_turn + 1) % len(self._token_ring)
                host[:len(rows)].copy_(tokens, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                rec["host"], rec["event"] = host, ev
        return rec

    def _resolve(self, rec) -> None:
        """Read a step's tokens and let the scheduler act on them."""
        sch = self.scheduler
        sampled: Dict[int, int] = {}
        if rec["rows"]:
            if rec["event"] is not None:
                rec["event"].synchronize()
                values = rec["host"][:len(rec["rows"])].tolist()
            else:
                values = rec["tokens"].tolist()
            sampled = dict(zip((e.sequence_id for e in rec["rows"]), values))
        live = [e for e in rec["entries"] if e.sequence_id in sch.states and e.sequence_id in sch.active]
        sch.process_outputs(live, sampled)        # rows of requests that ended meanwhile are dropped
        sch.evict_finished()

    def _launch_successor(self, prev):
        """If the step after `prev` is foreseeable without its tokens, launch it: every active request is
        decoding and was in `prev`, nothing waits for admission, and no request uses a repetition penalty
        (which needs the token on the host).  Requests that `prev` brings to max_tokens are left out."""
        sch = self.scheduler
        if (not self.engine.takes_device_tokens or sch.waiting_queue or len(prev["rows"]) != len(prev["entries"])
                or len(prev["rows"]) != len(sch.active)):
            return None
        from .scheduler import ScheduledEntry, SeqPhase
        entries, src = [], []
        for i, e in enumerate(prev["rows"]):
            st = sch.states.get(e.sequence_id)
            if st is None or e.sequence_id not in sch.active or st.sampling.repetition_penalty != 1.0:
                return None
            done_prompt = st.phase is SeqPhase.Decoding or st.prefilled_tokens + len(e.tokens) >= len(st.prompt_tokens)
            if not done_prompt:
                return None
            if len(st.generated_tokens) + 1 >= st.max_tokens:
                continue                                   # prev's token is its last one
            entries.append(ScheduledEntry(e.sequence_id, [0], True))
            src.append(i)
        if not entries:
            return None
        return self._launch(entries, (prev["tokens"], src))

    def generate(self, prompt_token_ids: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling_params: Union[None, SamplingParams, Sequence[SamplingParams]] = None,
                 max_tokens: int = 64, eos_token_id: Union[int, None, str] = "model") -> List[GenerationOutput]:
        """Generate for one prompt (a list of token ids) or several (a list of such lists).
        Outputs come back in the order of the prompts."""
        prompts = list(prompt_token_ids)
        if prompts and not isinstance(prompts[0], (list, tuple)):
            prompts = [prompts]
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            sampling_params = [sampling_params] * len(prompts)
        ids = [self.add_request(p, sp, max_tokens, eos_token_id=eos_token_id) for p, sp in zip(prompts, sampling_params)]
        done: Dict[int, SequenceOutput] = {}
        while len(done) < len(ids):
            for out in self.step():
                done[out.sequence_id] = out
            if self.scheduler.all_done() and self._inflight is None and len(done) < len(ids):
                for out in self.scheduler.collect_finished():
                    done[out.sequence_id] = out
                break
        # a kernel whose bounded wait gave up has produced invalid results: never hand those out silently
        self.engine.check_kernels()
        return [GenerationOutput(i, done[i].prompt_tokens, done[i].generated_tokens, done[i].finish_reason) for i in ids]
