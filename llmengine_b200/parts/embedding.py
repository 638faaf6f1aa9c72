"""Token embedding and the output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, Runtime, WeightSpec, register_part


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

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = self.rt.buffer("residual", token_ids.numel(), self.hidden, torch.float32)
        return self.rt.ops.embedding(token_ids, self.table, x)


@register_part("head", "lm_head")
class LMHead(Part):
    """logits = h W^T in 32-bit, no bias, no scaling (src/model/transformer_graph_builder.cpp:287).
    With `tied`, W is the embedding table: stored once, used twice
    (src/io/gguf_weight_loader.cpp:46-50)."""

    def __init__(self, rt: Runtime, prefix: str, vocab_size: int, hidden_size: int, tied: bool = False):
        super().__init__(rt, prefix)
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {self.name("weight"): WeightSpec((self.vocab, self.hidden))}

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = t[self.name("weight")].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.rt.buffer("logits", h.shape[0], self.vocab, torch.float32)
        return self.rt.ops.linear(h, self.weight, logits)
