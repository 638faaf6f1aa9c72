"""How a layer arranges its mixer, feed-forward and norms."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LayerSpec
from .base import Part, Runtime, WeightSpec, build_part, register_part


@register_part("block", "prenorm_residual")
class PreNormResidualBlock(Part):
    """x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x))
    (src/model/transformer_graph_builder.cpp:207-274: the un-normed x is the residual).

    The residual stream `x` stays 32-bit.  A contribution is not added where it is produced:
    it travels as `delta` to the next norm, whose kernel adds it to `x` and normalises in one
    pass.  The names under which the four parts' tensors are stored come with the spec.
    """

    def __init__(self, rt: Runtime, prefix: str, layer: LayerSpec, mixer_name: str = "mixer",
                 feed_forward_name: str = "feed_forward", mixer_norm_name: str = "mixer_norm",
                 feed_forward_norm_name: str = "feed_forward_norm"):
        super().__init__(rt, prefix)
        self.mixer_norm = build_part("norm", layer.mixer_norm, rt, self.name(mixer_norm_name))
        self.mixer = build_part("mixer", layer.mixer, rt, self.name(mixer_name))
        self.ffn_norm = build_part("norm", layer.feed_forward_norm, rt, self.name(feed_forward_norm_name))
        self.ffn = build_part("feed_forward", layer.feed_forward, rt, self.name(feed_forward_name))
        self.parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
        self.capture_safe = all(p.capture_safe for p in self.parts)

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

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], batch, cache) -> Tuple[torch.Tensor, torch.Tensor]:
        h = self.mixer_norm.forward(x, delta=delta)
        a = self.mixer.forward(h, batch, cache)
        h = self.ffn_norm.forward(x, delta=a)
        return x, self.ffn.forward(h, batch)
