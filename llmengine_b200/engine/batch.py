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


@dataclass
class PagedKVView:
    """The cache a paged mixer run works on."""

    kv: torch.Tensor                # [pages, 2, kv_heads, page_size, head_dim]
    group: int                      # index into StepBatch.groups
    writes: bool                    # False when the run reads another run's cache


@dataclass
class StateView:
    """The fixed-size states of a stateful mixer run: row `batch.state_slots[r]` belongs to request r."""

    state: torch.Tensor             # [slots, *shape]
