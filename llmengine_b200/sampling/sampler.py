"""Sampling: options with the names, defaults and order of application of the reference's
SamplingConfig / Sampler (include/minillm/runtime/sampler.h:9-20, src/runtime/sampler.cpp:11-141),
computed on the device by this package's kernel.

Differences from the reference, both deliberate: the uniform number of a draw comes from a
counter-based generator keyed by (seed, draw index) instead of one Mersenne twister shared by
all requests, so a request's tokens do not depend on what else is running; and the draw
walks the candidates in vocabulary order instead of sorted order (no sort of the vocabulary).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class SamplingParams:
    greedy: bool = True                 # argmax; the other options then only matter through the penalty
    top_k: int = 0                      # keep the k most probable tokens (0 = off)
    top_p: float = 0.0                  # keep the smallest set with cumulative probability >= top_p (0 = off)
    temperature: float = 1.0            # logits are divided by it when it is positive and not 1
    repetition_penalty: float = 1.0     # applied once per occurrence of a token in the request so far
    seed: int = 42                      # the reference constructs Sampler(42)

    def __post_init__(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must be in [0, 1]")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")


_MASK = (1 << 64) - 1


def uniform(seed: int, draw: int) -> float:
    """The uniform number in (0,1) of draw number `draw` of a request with `seed`: a 64-bit mix of
    the two (splitmix64 finaliser), top 24 bits, centred in its cell so it is never 0 or 1."""
    z = (seed * 0x9E3779B97F4A7C15 + (draw + 1) * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return ((z >> 40) + 0.5) / float(1 << 24)


class Sampler:
    """Turns rows of logits into tokens on the device."""

    def __init__(self, ops, device: torch.device, max_rows: int):
        self.ops, self.device, self.max_rows = ops, device, max_rows
        pin = device.type == "cuda"
        # row-wise options, packed so that one copy brings them to the device
        # the options travel through pinned buffers used in turn; an event tells when a buffer's copy has run,
        # so that a later call (steps may be queued without waiting for each other) never overwrites it early
        self._hosts = [torch.zeros(6, max_rows, dtype=torch.float32, pin_memory=pin) for _ in range(4)]
        self._host_events = [None] * 4
        self._host_turn = 0
        self._dev = torch.zeros(6, max_rows, dtype=torch.float32, device=device)
        self._dev_int = self._dev.view(torch.int32)          # rows 4 and 5 hold integers
        # two output buffers used in turn: the tokens of one step stay readable while the next step samples
        self._outs = [torch.zeros(max_rows, dtype=torch.int32, device=device) for _ in range(2)]
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], draws: Sequence[int],
               histories: Optional[Sequence[Dict[int, int]]] = None) -> torch.Tensor:
        """`logits` [R, vocab] (modified in place when a repetition penalty applies); `draws[r]` is how
        many tokens request r has drawn before; `histories[r]` maps token -> occurrences so far.
        Returns int32 [R] on the device."""
        R = logits.shape[0]
        assert R == len(params) == len(draws) and R <= self.max_rows
        k = self._host_turn
        self._host_turn = (k + 1) % len(self._hosts)
        if self._host_events[k] is not None:
            self._host_events[k].synchronize()
        host = self._hosts[k]
        h = host.numpy()
        for r, (p, d) in enumerate(zip(params, draws)):
            h[0, r] = p.temperature
            h[1, r] = p.top_p
            h[2, r] = 0.5 if p.greedy else uniform(p.seed, d)
            h[3, r] = p.repetition_penalty
        hi = host.view(torch.int32).numpy()
        for r, p in enumerate(params):
            hi[4, r] = 1 if p.greedy else 0
            hi[5, r] = p.top_k
        self._dev.copy_(host, non_blocking=True)
        if self.device.type == "cuda":
            self._host_events[k] = torch.cuda.Event()
            self._host_events[k].record()
        dev = self._dev
        greedy = self._dev_int[4, :R]
        top_k = self._dev_int[5, :R]
        if histories is not None and any(p.repetition_penalty != 1.0 for p in params):
            rows, toks, counts = [], [], []
            for r, (p, hist) in enumerate(zip(params, histories)):
                if p.repetition_penalty != 1.0:
                    for t, c in hist.items():
                        rows.append(r), toks.append(t), counts.append(c)
            if rows:
                pairs = torch.tensor([rows, toks, counts], dtype=torch.int32).to(self.device)
                self.ops.repetition_penalty(logits, pairs[0], pairs[1], pairs[2], dev[3, :R].contiguous())
        self._turn ^= 1
        out = self._outs[self._turn][:R]
        self.ops.sample(logits, greedy=greedy, temperature=dev[0, :R], top_k=top_k,
                        top_p=dev[1, :R], u=dev[2, :R], out=out)
        return out

    def get_top_tokens(self, logits_row: torch.Tensor, params: SamplingParams, top_n: int):
        """The `top_n` most probable tokens after temperature, as (token, probability) pairs
        (src/runtime/sampler.cpp:143-197).  A host-side helper for inspection, not on the step path."""
        z = logits_row.float()
        if params.temperature != 1.0 and params.temperature > 0:
            z = z / params.temperature
        p = torch.softmax(z, 0)
        v, i = torch.topk(p, min(top_n, p.numel()))
        return list(zip(i.tolist(), v.tolist()))
