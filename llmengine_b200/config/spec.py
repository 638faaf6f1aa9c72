"""Data that describes a model: which parts each layer is made of and in which
order the layers run.

A model is described without code: a `ModelSpec` lists the layers (`LayerSpec`),
each layer names its parts (`PartSpec`: a kind registered in
`llmengine_b200.parts` plus that part's sizes and constants), and `order` says
which layer runs when.  The reference assembles one fixed layer body in a loop
(src/model/transformer_graph_builder.cpp:152-277); here the same body is one
`LayerSpec` value per layer so that a model may mix different mixers and
feed-forwards layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind and its own parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(more)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges, by role.

    `parts` maps a role name to a part; which roles exist is the block kind's business (the pre-norm residual
    block reads "mixer", "mixer_norm", "feed_forward" and "feed_forward_norm"; a block with a post-norm, one
    shared norm for parallel branches or no feed-forward names its own).  The four keyword arguments are a
    shorthand for those four roles.  `prefix` is the layer's tensor-name prefix in the weight file; the parts'
    own tensor names are appended to it by the block.
    """

    prefix: str
    block: PartSpec
    mixer: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    parts: Mapping[str, PartSpec] = field(default_factory=dict)

    def __post_init__(self) -> None:
        merged = dict(self.parts)
        for role in ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm"):
            given = getattr(self, role)
            if given is not None:
                if role in merged and merged[role] != given:
                    raise ValueError(f"layer {self.prefix!r}: the part {role!r} is given twice")
                merged[role] = given
            elif role in merged:
                object.__setattr__(self, role, merged[role])
        object.__setattr__(self, "parts", merged)


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order.

    `layer` indexes `ModelSpec.layers`; a layer may appear in several runs (its
    weights are shared, each run keeps a cache of its own).  `cache_from`, when
    set, is the index *in the order* of an earlier run whose cache this run
    reads instead of keeping its own (it then writes nothing).
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerRun, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    # tensor-name prefixes of the parts that stand outside the layers
    embedding_prefix: str = "embedding"
    final_norm_prefix: str = "final_norm"
    lm_head_prefix: str = "lm_head"

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("a model needs a non-empty layer order")
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < i:
                    raise ValueError(
                        f"order[{i}].cache_from={run.cache_from} must name an earlier entry of the order")
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(
                        f"order[{i}].cache_from={run.cache_from} names a run that itself borrows a cache")
