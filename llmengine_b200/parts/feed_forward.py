"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict

import torch

from .base import Part, Runtime, WeightSpec, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down( silu(gate(h)) * up(h) ), no biases; silu(g) = g / (1 + exp(-g))
    (src/model/transformer_graph_builder.cpp:261-274; src/runtime/kernels/cpu_kernels.cpp:848-859).
    The gate and up matrices are stored as one [gate | up] matrix so that one product serves both."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        super().__init__(rt, prefix)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.name("gate_proj.weight"): WeightSpec((self.inter, self.hidden)),
            self.name("up_proj.weight"): WeightSpec((self.inter, self.hidden)),
            self.name("down_proj.weight"): WeightSpec((self.hidden, self.inter)),
        }

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([t[self.name("gate_proj.weight")], t[self.name("up_proj.weight")]], 0).contiguous()
        self.w_down = t[self.name("down_proj.weight")].contiguous()

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        rt, ops = self.rt, self.rt.ops
        T = h.shape[0]
        act = rt.buffer("act", T, self.inter, rt.dtype)
        fused = getattr(ops, "linear_swiglu_supports", None)
        if fused is not None and fused(h, self.w_gate_up, act):
            ops.linear_swiglu(h, self.w_gate_up, act)         # product and activation in one kernel
        else:
            gate_up = rt.buffer("gate_up", T, 2 * self.inter, rt.dtype)
            ops.linear(h, self.w_gate_up, gate_up)
            ops.swiglu(gate_up, act)
        delta = rt.buffer("ffn_out", T, self.hidden, torch.float32)
        return ops.linear(act, self.w_down, delta)
