"""A model assembled from a `ModelSpec`: embedding, the blocks in their execution order,
final norm and head.  It knows no architecture: everything comes from the spec and the
part registries."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.spec import ModelSpec
from ..parts.base import (Part, Runtime, WeightSpec, build_part, emit_block, emit_embedding, emit_head, emit_norm)
from .plan import ROWS_LOGITS, Plan


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec, self.rt = spec, rt
        self.embedding = build_part("embedding", spec.embedding, rt, spec.embedding_prefix)
        self.blocks = [build_part("block", ls.block.with_params(layer=ls), rt, ls.prefix) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, rt, spec.final_norm_prefix)
        self.head = build_part("head", spec.lm_head, rt, spec.lm_head_prefix)
        self.order = spec.order
        self._compiled = None
        self._compiled_for = None

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

    def tied_tensors(self) -> Dict[str, str]:
        """Tensor names that a part shares with another part instead of storing them (own name -> source)."""
        out: Dict[str, str] = {}
        for p in self.parts():
            out.update(p.tied_tensors())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights({n: tensors[n] for n in p.weight_specs()})
        for p in self.parts():
            tied = p.tied_tensors()
            if not tied:
                continue
            got = {}
            for own, source in tied.items():
                found = [t for q in self.parts() for t in [q.shared_tensor(source)] if t is not None]
                if not found:
                    raise ValueError(f"{own!r} is tied to {source!r}, which no part of the model offers")
                got[own] = found[0]
            p.receive_tied(got)
        self._compiled = None

    # ------------------------------------------------------------------ caches
    def cache_specs(self) -> List[Tuple[object, Optional[int]]]:
        """For each run of the order: (what its mixer keeps, the run whose cache it reads instead)."""
        return [(self.blocks[r.layer].cache_spec(), r.cache_from) for r in self.order]

    # ------------------------------------------------------------------ compute
    def plan(self, caches) -> Plan:
        """The model's launch sequence: every part emits its records, in the order the layers run."""
        plan = Plan()
        x = emit_embedding(plan, self.embedding, self.spec.hidden_size)
        delta = None
        for i, run in enumerate(self.order):
            x, delta = emit_block(plan, self.blocks[run.layer], x, delta, caches[i])
        h = emit_norm(plan, self.final_norm, x, delta=delta, rows=ROWS_LOGITS)
        emit_head(plan, self.head, h)
        return plan

    def forward(self, batch, caches) -> Optional[torch.Tensor]:
        """Runs the batch's tokens through every run of the order and returns 32-bit logits
        [len(batch.logit_rows), vocab] (None when no logits are wanted)."""
        if self._compiled is None or self._compiled_for is not caches:
            self._compiled = self.rt.ops.compile(self.plan(caches))
            self._compiled_for = caches
        n = batch.logit_rows.numel()
        batch.logits = self.rt.buffer("logits", n, self.spec.vocab_size, torch.float32) if n else None
        self.rt.batch = batch
        self._compiled.run(batch)
        return batch.logits
