"""Continuous batching: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

The life of a request and the method names follow the reference's ContinuousBatchScheduler
(include/minillm/runtime/continuous_batch_scheduler.h:12-83,
src/runtime/continuous_batch_scheduler.cpp:19-125): Waiting -> Prefilling -> Decoding ->
Finished; `submit` refuses an empty prompt, a non-positive max_tokens and an id that is in
use; admission is first-in-first-out and stops at the first request that does not fit.
The reference leaves the token budget, the portions and the decode loop to its caller (it is
never connected to a model there); `schedule` and `process_outputs` add them.

What happens when pages run out is decided at admission: a request is admitted only if the
pages it can ever need (prompt + max_tokens, in every cache group, at that group's peak) can
be promised to it.  An admitted request therefore never lacks a page in mid-flight, nothing
is preempted, and a request that could never fit is refused at `submit` instead of waiting
forever (which the reference's would: src/runtime/continuous_batch_scheduler.cpp:68-70).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..cache import CacheManager
from ..sampling import SamplingParams


class SeqPhase(enum.Enum):
    Waiting = "waiting"
    Prefilling = "prefilling"
    Decoding = "decoding"
    Finished = "finished"


@dataclass
class SequenceRequest:
    prompt_tokens: Sequence[int]
    max_tokens: int = 64
    sequence_id: int = -1                      # -1 = assign the next free id
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_token_id: Optional[int] = None


@dataclass
class SeqState:
    sequence_id: int
    prompt_tokens: List[int]
    max_tokens: int
    sampling: SamplingParams
    eos_token_id: Optional[int]
    phase: SeqPhase = SeqPhase.Waiting
    generated_tokens: List[int] = field(default_factory=list)
    prefilled_tokens: int = 0
    finish_reason: Optional[str] = None
    token_counts: Dict[int, int] = field(default_factory=dict)     # prompt + generated, for the repetition penalty


@dataclass
class SequenceOutput:
    sequence_id: int
    prompt_tokens: List[int]
    generated_tokens: List[int]
    finished: bool
    finish_reason: Optional[str] = None


@dataclass
class ScheduledEntry:
    sequence_id: int
    tokens: List[int]
    samples: bool          # the step's last token of this entry yields the request's next token


class ContinuousBatchScheduler:
    def __init__(self, cache: CacheManager, max_batch_size: int = 4, max_num_batched_tokens: int = 2048,
                 prefill_chunk: int = 2048):
        if max_batch_size <= 0:
            raise ValueError("ContinuousBatchScheduler max_batch_size must be positive")
        if max_num_batched_tokens < max_batch_size:
            raise ValueError("max_num_batched_tokens must be at least max_batch_size: every decoding request needs one token a step")
        if prefill_chunk <= 0:
            raise ValueError("prefill_chunk must be positive")
        self.cache = cache
        self.max_batch_size = min(max_batch_size, cache.max_requests)
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk = min(prefill_chunk, max_num_batched_tokens)
        self.states: Dict[int, SeqState] = {}
        self.waiting_queue: List[int] = []
        self.active: List[int] = []
        self._next_id = 0

    # ------------------------------------------------------------------ submit / admit
    def submit(self, request: SequenceRequest) -> int:
        prompt = [int(t) for t in request.prompt_tokens]
        if not prompt:
            raise ValueError("SequenceRequest must have at least one prompt token")
        if request.max_tokens <= 0:
            raise ValueError("SequenceRequest max_tokens must be positive")
        total = len(prompt) + request.max_tokens
        if not self.cache.fits_at_all(total, self.prefill_chunk):
            raise ValueError(
                f"SequenceRequest needs {total} tokens (prompt {len(prompt)} + max_tokens {request.max_tokens}): "
                f"more than the model's length limit {self.cache.max_request_len} or than the whole cache holds")
        if request.sequence_id >= 0:
            sid = request.sequence_id
            if sid in self.states:
                raise ValueError(f"SequenceRequest sequence_id is already in use: {sid}")
            self._next_id = max(self._next_id, sid + 1)
        else:
            sid = self._next_id
            self._next_id += 1
        st = SeqState(sid, prompt, request.max_tokens, request.sampling, request.eos_token_id)
        for t in prompt:
            st.token_counts[t] = st.token_counts.get(t, 0) + 1
        self.states[sid] = st
        self.waiting_queue.append(sid)
        return sid

    def admit_waiting(self) -> List[int]:
        """Admit from the head of the queue while a batch place and the pages can be promised."""
        admitted = []
        while self.waiting_queue and len(self.active) < self.max_batch_size:
            sid = self.waiting_queue[0]
            st = self.states[sid]
            self.cache.add_request(sid)
            if not self.cache.try_commit(sid, len(st.prompt_tokens) + st.max_tokens, self.prefill_chunk):
                self.cache.free_request(sid)
                break                                       # head-of-line blocking, as in the reference
            st.phase = SeqPhase.Prefilling
            self.active.append(sid)
            self.waiting_queue.pop(0)
            admitted.append(sid)
        return admitted

    # ------------------------------------------------------------------ one step
    def schedule(self) -> List[ScheduledEntry]:
        """The next step's batch: one token for every decoding request, then prompt portions in
        admission order until the token budget is spent."""
        budget = self.max_num_batched_tokens
        out: List[ScheduledEntry] = []
        for sid in self.active:
            st = self.states[sid]
            if st.phase is SeqPhase.Decoding:
                out.append(ScheduledEntry(sid, [st.generated_tokens[-1]], True))
                budget -= 1
        for sid in self.active:
            st = self.states[sid]
            if st.phase is not SeqPhase.Prefilling or budget <= 0:
                continue
            left = len(st.prompt_tokens) - st.prefilled_tokens
            n = min(left, self.prefill_chunk, budget)
            tokens = st.prompt_tokens[st.prefilled_tokens:st.prefilled_tokens + n]
            out.append(ScheduledEntry(sid, tokens, n == left))
            budget -= n
        return out

    def process_outputs(self, entries: Sequence[ScheduledEntry], sampled: Dict[int, int]) -> None:
        """After the step ran: prompts move on, sampled tokens are appended, requests finish."""
        for e in entries:
            st = self.states[e.sequence_id]
            if st.phase is SeqPhase.Prefilling:
                self.mark_prefill_progress(e.sequence_id, st.prefilled_tokens + len(e.tokens))
            if e.samples:
                tok = int(sampled[e.sequence_id])
                if st.eos_token_id is not None and tok == st.eos_token_id:
                    # the reference's generate loop stops at EOS without keeping it (examples/generate.cpp:334)
                    st.finish_reason = "eos"
                    self.mark_finished(e.sequence_id)
                else:
                    self.mark_token_generated(e.sequence_id, tok)

    def mark_prefill_progress(self, sequence_id: int, tokens_prefilled: int) -> None:
        st = self.states[sequence_id]
        st.prefilled_tokens = tokens_prefilled
        if st.prefilled_tokens >= len(st.prompt_tokens):
            st.phase = SeqPhase.Decoding

    def mark_token_generated(self, sequence_id: int, token: int) -> None:
        st = self.states[sequence_id]
        st.generated_tokens.append(token)
        st.token_counts[token] = st.token_counts.get(token, 0) + 1
        if len(st.generated_tokens) >= st.max_tokens:
            st.finish_reason = st.finish_reason or "length"
            st.phase = SeqPhase.Finished

    def mark_finished(self, sequence_id: int) -> None:
        st = self.states[sequence_id]
        st.finish_reason = st.finish_reason or "stopped"
        st.phase = SeqPhase.Finished

    def evict_finished(self) -> List[int]:
        """Finished requests leave the batch and give back their pages and their slot at once."""
        gone = [sid for sid in self.active if self.states[sid].phase is SeqPhase.Finished]
        for sid in gone:
            self.cache.free_request(sid)
            self.active.remove(sid)
        return gone

    def collect_finished(self) -> List[SequenceOutput]:
        out = []
        for sid in [s for s, st in self.states.items() if st.phase is SeqPhase.Finished and s not in self.active]:
            st = self.states.pop(sid)
            out.append(SequenceOutput(sid, st.prompt_tokens, st.generated_tokens, True, st.finish_reason))
        return out

    # ------------------------------------------------------------------ queries (names of the reference)
    def state(self, sequence_id: int) -> SeqState:
        return self.states[sequence_id]

    def active_ids(self) -> List[int]:
        return list(self.active)

    def waiting_ids(self) -> List[int]:
        return list(self.waiting_queue)

    def has_active(self) -> bool:
        return bool(self.active)

    def has_waiting(self) -> bool:
        return bool(self.waiting_queue)

    def all_done(self) -> bool:
        return not self.active and not self.waiting_queue

    def active_count(self) -> int:
        return len(self.active)

    def waiting_count(self) -> int:
        return len(self.waiting_queue)
