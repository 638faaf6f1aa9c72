"""A model's launch sequence as data: the operation records that the parts emit when a model is loaded.

A `Plan` is a list of records; each record names an operation and holds the tensors it works on: weights, and
workspace buffers made for the step's token budget (a step uses their first rows).  Nothing in a record
depends on a step: how many tokens, which requests decode and where their pages lie comes with the step.  The
kernel set compiles a plan once (`ops.compile(plan)`): on the GPU into the native executor's records
(include/llmengine_b200/executor.h), which are walked in C++ for every step; in the host tests into a list that a
CPU stand-in interprets.  Either way the parts emit their operations once, in one place.

The reference walks a graph of nodes in topological order and looks the kernel of every node up per run
(src/runtime/executor.cpp:112-142); a plan is that order fixed at load time.

A part written outside this package needs no record kind of its own: `Plan.call(fn)` makes a record that calls
`fn(batch)` in its turn, on the same stream, with the step's batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

ROWS_TOKENS, ROWS_LOGITS = "tokens", "logits"


@dataclass
class Op:
    kind: str
    a: Dict[str, Any] = field(default_factory=dict)


class Plan:
    def __init__(self) -> None:
        self.ops: List[Op] = []

    def _add(self, kind: str, **a: Any) -> None:
        self.ops.append(Op(kind, a))

    def embedding(self, table: torch.Tensor, out: torch.Tensor) -> None:
        """out[t] = table[token_ids[t]] as 32-bit, for the step's tokens."""
        self._add("embedding", table=table, out=out)

    def rmsnorm(self, x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: str = ROWS_TOKENS) -> None:
        """x += delta (if given), out = rmsnorm(x) * gain; `rows` = "logits": only the step's wanted rows,
        gathered into the first rows of `out`."""
        self._add("rmsnorm", x=x, gain=gain, eps=float(eps), out=out, delta=delta, rows=rows)

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], rows: str = ROWS_TOKENS) -> None:
        """out = x w^T for the step's tokens (or its wanted rows); `out` None: the step's logits."""
        self._add("linear", x=x, w=w, out=out, rows=rows)

    def linear_swiglu(self, x: torch.Tensor, w_gate_up: torch.Tensor, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        """out = silu(x Wg^T) * (x Wu^T) with w_gate_up = [Wg | Wu] by rows; `gate_up` is the workspace of the form
        that runs the product and the activation as two kernels."""
        self._add("linear_swiglu", x=x, w_gate_up=w_gate_up, gate_up=gate_up, out=out)

    def qkv_post(self, *, q_in, k_in, v_in, num_heads: int, num_kv_heads: int, head_dim: int, q_gain=None, k_gain=None,
                 eps: float = 0.0, cos_sin=None, q_out=None, k_out=None, cache=None, group: int = 0) -> None:
        """Per-head norm (with gains), rotation (with a table) and cache write (with a cache) of what is given."""
        self._add("qkv_post", q_in=q_in, k_in=k_in, v_in=v_in, num_heads=num_heads, num_kv_heads=num_kv_heads,
                  head_dim=head_dim, q_gain=q_gain, k_gain=k_gain, eps=float(eps), cos_sin=cos_sin, q_out=q_out,
                  k_out=k_out, cache=cache, group=group)

    def attend(self, *, q, out, cache, group: int, num_heads: int, num_kv_heads: int, head_dim: int, window: int,
               scale: float, scratch=None) -> None:
        """Attention of every token of the step over its request's cache; queries finished."""
        self._add("attend", q=q, out=out, cache=cache, group=group, num_heads=num_heads, num_kv_heads=num_kv_heads,
                  head_dim=head_dim, window=window, scale=float(scale), scratch=scratch)

    def attention(self, *, qkv, q, out, cache, writes: bool, group: int, num_heads: int, num_kv_heads: int, head_dim: int,
                  window: int, scale: float, q_gain=None, k_gain=None, eps: float = 0.0, cos_sin=None, scratch=None) -> None:
        """From the raw q|k|v projections to the attention output: norm, rotation (cos_sin None: none), cache write
        (if `writes`) and attention; the executor fuses them where a kernel does all of it."""
        self._add("attention", qkv=qkv, q=q, out=out, cache=cache, writes=bool(writes), group=group, num_heads=num_heads,
                  num_kv_heads=num_kv_heads, head_dim=head_dim, window=window, scale=float(scale), q_gain=q_gain,
                  k_gain=k_gain, eps=float(eps), cos_sin=cos_sin, scratch=scratch)

    def call(self, fn: Callable[[Any], None], what: str = "") -> None:
        """`fn(batch)` is called in its turn with the step's `StepBatch`, on the step's stream."""
        self._add("call", fn=fn, what=what)
