"""What one step hands to the model: the tokens of the batch and, for each of them,
where it stands in its request and where its cache entries live.

The reference passes a single `pos_offset` per launch, so one run serves one sequence
(src/runtime/kernels/cuda_kernels.cu:430-431), and builds padded block tables only for
decode-only batches (include/minillm/runtime/cache/paged_attention_scheduler.h:11-20).
Here every token carries its own position and request row, so prompt portions and single
decoded tokens of different requests share one launch sequence.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class GroupView:
    """Per cache group (layers with the same page size and retention): the block table of
    every request of the batch and the physical cache row of every token."""

    page_size: int
    window: int
    block_tables: torch.Tensor      # int32 [R, max_blocks]; -1 where no page is held
    slot_mapping: torch.Tensor      # int32 [T]: page * page_size + slot-in-page; -1 = do not store
    max_blocks: int


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    q_lens: List[int]               # host copy: tokens of each request in this step
    start_positions: List[int]      # host copy: tokens each request had cached before the step
    token_ids: torch.Tensor         # int32 [T]
    positions: torch.Tensor         # int32 [T] absolute position in the request
    token_request: torch.Tensor     # int32 [T] block-table row (the state slot) of the token's request
    cu_q_lens: torch.Tensor         # int32 [R+1] prefix sums of q_lens
    ctx_lens: torch.Tensor          # int32 [R] cached length of each request after this step
    state_slots: torch.Tensor       # int32 [R] the request's fixed-size state slot
    first_portion: torch.Tensor     # int32 [R] 1 when the request has nothing cached before this step
    logit_rows: torch.Tensor        # int32 [NL] token rows whose logits are wanted
    decode_rows: torch.Tensor       # int32 [ND] batch rows of the requests with exactly one token in this step
    portion_rows: torch.Tensor      # int32 [NP] batch rows of the other requests
    groups: List[GroupView] = field(default_factory=list)
    assume_ctx: Optional[int] = None   # set when the step is (to be) captured: size launches for this context length
    logits: Optional[torch.Tensor] = None   # [NL, vocab] 32-bit: where the step's logits go

    @classmethod
    def bare(cls, num_tokens: int, device, token_ids: Optional[torch.Tensor] = None,
             logit_rows: Optional[torch.Tensor] = None, logits: Optional[torch.Tensor] = None) -> "StepBatch":
        """A step without requests or caches: `num_tokens` rows for operations that need nothing else
        (a part that is run by itself)."""
        e = torch.zeros(0, dtype=torch.int32, device=device)
        return cls(num_tokens=num_tokens, num_requests=0, q_lens=[], start_positions=[],
                   token_ids=token_ids if token_ids is not None else e, positions=e, token_request=e, cu_q_lens=e,
                   ctx_lens=e, state_slots=e, first_portion=e, logit_rows=logit_rows if logit_rows is not None else e,
                   decode_rows=e, portion_rows=e, groups=[], logits=logits)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_ctx_len(self) -> int:
        return max((s + q for s, q in zip(self.start_positions, self.q_lens)), default=0)

    @property
    def max_portion_len(self) -> int:
        return max((q for q in self.q_lens if q != 1), default=0)

    @property
    def max_decode_ctx(self) -> int:
        if self.assume_ctx is not None:
            return self.assume_ctx
        return max((s + 1 for s, q in zip(self.start_positions, self.q_lens) if q == 1), default=0)

    @property
    def decode_only(self) -> bool:
        return all(q == 1 for q in self.q_lens)


from ..parts.base import PagedKVView, StateView  # noqa: E402,F401  (their home is beside the cache specs)
