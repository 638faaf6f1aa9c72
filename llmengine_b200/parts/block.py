"""How a layer arranges its mixer, feed-forward and norms."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LayerSpec
from ..engine.plan import Plan
from .base import (Part, Runtime, WeightSpec, build_part, emit_feed_forward, emit_mixer, emit_norm, register_part,
                   run_alone)


@register_part("block", "prenorm_residual")
class PreNormResidualBlock(Part):
    """x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x))
    (src/model/transformer_graph_builder.cpp:207-274: the un-normed x is the residual).

    The residual stream `x` stays 32-bit.  A contribution is not added where it is produced:
    it travels as `delta` to the next norm, whose kernel adds it to `x` and normalises in one
    pass.  The block reads the parts "mixer", "mixer_norm", "feed_forward" and "feed_forward_norm" of its
    layer; the names under which their tensors are stored come with the spec.
    """

    def __init__(self, rt: Runtime, prefix: str, layer: LayerSpec, mixer_name: str = "mixer",
                 feed_forward_name: str = "feed_forward", mixer_norm_name: str = "mixer_norm",
                 feed_forward_norm_name: str = "feed_forward_norm"):
        super().__init__(rt, prefix)
        need = ("mixer", "mixer_norm", "feed_forward", "feed_forward_norm")
        missing = [n for n in need if n not in layer.parts]
        if missing:
            raise ValueError(f"layer {prefix!r}: a prenorm_residual block needs the parts {', '.join(missing)}")
        self.mixer_norm = build_part("norm", layer.parts["mixer_norm"], rt, self.name(mixer_norm_name))
        self.mixer = build_part("mixer", layer.parts["mixer"], rt, self.name(mixer_name))
        self.ffn_norm = build_part("norm", layer.parts["feed_forward_norm"], rt, self.name(feed_forward_norm_name))
        self.ffn = build_part("feed_forward", layer.parts["feed_forward"], rt, self.name(feed_forward_name))
        self.parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
        self.capture_safe = all(p.capture_safe and hasattr(p, "emit") for p in self.parts)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for p in self.parts:
            out.update(p.weight_specs())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load_weights({n: tensors[n] for n in p.weight_specs()})

    def cache_spec(self):
        return self.mixer.cache_spec()

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor], cache) -> Tuple[torch.Tensor, torch.Tensor]:
        hidden = x.shape[1]
        h = emit_norm(plan, self.mixer_norm, x, delta=delta)
        a = emit_mixer(plan, self.mixer, h, cache, hidden)
        h = emit_norm(plan, self.ffn_norm, x, delta=a)
        return x, emit_feed_forward(plan, self.ffn, h, hidden)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch, cache) -> Tuple[torch.Tensor, torch.Tensor]:
        plan = Plan()
        x, out = self.emit(plan, x, delta, cache)
        run_alone(self.rt, plan, batch)
        return x, out[: x.shape[0]]
