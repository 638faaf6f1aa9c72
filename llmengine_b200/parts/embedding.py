"""Token embedding and the output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..engine.plan import ROWS_LOGITS, Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """x[t,:] = E[ids[t],:] as 32-bit, no scaling (src/runtime/kernels/cpu_kernels.cpp:262-274)."""

    def __init__(self, rt: Runtime, prefix: str, vocab_size: int, hidden_size: int):
        super().__init__(rt, prefix)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name("weight"): WeightSpec((self.vocab, self.hidden))}

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t[self.name("weight")].contiguous()

    def shared_tensor(self, name: str) -> Optional[torch.Tensor]:
        return self.table if name == self.name("weight") else None

    def emit(self, plan: Plan) -> torch.Tensor:
        x = self.rt.workspace("residual", self.hidden, torch.float32)
        plan.embedding(self.table, x)
        return x

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        x = self.emit(plan)
        run_alone(self.rt, plan, StepBatch.bare(token_ids.numel(), token_ids.device, token_ids=token_ids))
        return x[: token_ids.numel()]


@register_part("head", "lm_head")
class LMHead(Part):
    """logits = h W^T in 32-bit, no bias, no scaling (src/model/transformer_graph_builder.cpp:287).
    With `tied_to` (the name of the embedding's tensor), W is that table: stored once, used twice
    (src/io/gguf_weight_loader.cpp:46-50)."""

    def __init__(self, rt: Runtime, prefix: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None,
                 tied: bool = False):
        super().__init__(rt, prefix)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.tied_to = tied_to
        self.tied = bool(tied) or tied_to is not None
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {self.name("weight"): WeightSpec((self.vocab, self.hidden))}

    def tied_tensors(self) -> Dict[str, str]:
        return {self.name("weight"): self.tied_to} if self.tied_to is not None else {}

    def receive_tied(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.tie(tensors[self.name("weight")])

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = t[self.name("weight")].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"{self.prefix}: a table of shape {tuple(table.shape)} cannot serve a head of "
                             f"{(self.vocab, self.hidden)}")
        self.weight = table

    def emit(self, plan: Plan, h: torch.Tensor) -> None:
        plan.linear(h, self.weight, None, rows=ROWS_LOGITS)      # into the step's logits

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        from ..engine.batch import StepBatch
        logits = self.rt.buffer("logits", h.shape[0], self.vocab, torch.float32)
        plan = Plan()
        self.emit(plan, h)
        rows = torch.arange(h.shape[0], dtype=torch.int32, device=h.device)
        run_alone(self.rt, plan, StepBatch.bare(h.shape[0], h.device, logit_rows=rows, logits=logits))
        return logits
