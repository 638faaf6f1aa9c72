"""A model assembled from a `ModelSpec`: embedding, the blocks in their execution order,
final norm and head.  It knows no architecture: everything comes from the spec and the
part registries."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec
from ..parts.base import Part, Runtime, WeightSpec, build_part


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec, self.rt = spec, rt
        self.embedding = build_part("embedding", spec.embedding, rt, spec.embedding_prefix)
        self.blocks = [build_part("block", ls.block.with_params(layer=ls), rt, ls.prefix) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, rt, spec.final_norm_prefix)
        self.head = build_part("head", spec.lm_head, rt, spec.lm_head_prefix)
        self.order = spec.order

    # ------------------------------------------------------------------ weights
    def parts(self) -> List[Part]:
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for p in self.parts():
            for n, s in p.weight_specs().items():
                if n in out:
                    raise ValueError(f"two parts claim the tensor {n!r}")
                out[n] = s
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights({n: tensors[n] for n in p.weight_specs()})
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.table)

    # ------------------------------------------------------------------ caches
    def cache_specs(self) -> List[Tuple[object, Optional[int]]]:
        """For each run of the order: (what its mixer keeps, the run whose cache it reads instead)."""
        return [(self.blocks[r.layer].cache_spec(), r.cache_from) for r in self.order]

    # ------------------------------------------------------------------ compute
    def forward(self, batch, caches) -> Optional[torch.Tensor]:
        """Runs the batch's tokens through every run of the order and returns 32-bit logits
        [len(batch.logit_rows), vocab] (None when no logits are wanted)."""
        x = self.embedding.forward(batch.token_ids)
        delta = None
        for i, run in enumerate(self.order):
            x, delta = self.blocks[run.layer].forward(x, delta, batch, caches[i])
        if batch.logit_rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, delta=delta, out_rows=batch.logit_rows)
        return self.head.forward(h)
