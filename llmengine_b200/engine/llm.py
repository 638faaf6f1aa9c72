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
                 **engine_options):
        """`model`: a folder with config.json and model.safetensors (or `config` + `random_seed` for
        random weights).  Further keyword arguments are fields of `EngineConfig`."""
        ec = engine_config or EngineConfig(dtype=dtype, **engine_options)
        self.engine = Engine(model, config=config, random_seed=random_seed, engine_config=ec, ops=ops)
        self.scheduler = ContinuousBatchScheduler(self.engine.cache, ec.max_num_seqs, ec.max_num_batched_tokens,
                                                  ec.prefill_chunk)
        self.sampler = Sampler(self.engine.ops, self.engine.device, ec.max_num_seqs)
        self.eos_token_id = getattr(self.engine.config, "eos_token_id", None)
        self.default_seed = ec.seed

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
        """Admit, run one batch, sample, finish.  Returns the requests that finished in this step."""
        sch = self.scheduler
        sch.admit_waiting()
        entries = sch.schedule()
        if not entries:
            return sch.collect_finished()
        batch = [StepEntry(e.sequence_id, e.tokens, [len(e.tokens) - 1] if e.samples else []) for e in entries]
        logits = self.engine.step(batch)
        sampled: Dict[int, int] = {}
        rows = [e for e in entries if e.samples]
        if rows:
            states = [sch.state(e.sequence_id) for e in rows]
            tokens = self.sampler.sample(logits, [s.sampling for s in states],
                                         [len(s.generated_tokens) for s in states],
                                         [s.token_counts for s in states])
            sampled = dict(zip((e.sequence_id for e in rows), tokens.tolist()))
        sch.process_outputs(entries, sampled)
        sch.evict_finished()
        return sch.collect_finished()

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
            if self.scheduler.all_done() and len(done) < len(ids):
                for out in self.scheduler.collect_finished():
                    done[out.sequence_id] = out
                break
        return [GenerationOutput(i, done[i].prompt_tokens, done[i].generated_tokens, done[i].finish_reason) for i in ids]
