"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict

import torch

from ..engine.plan import Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down( silu(gate(h)) * up(h) ), no biases; silu(g) = g / (1 + exp(-g))
    (src/model/transformer_graph_builder.cpp:261-274; src/runtime/kernels/cpu_kernels.cpp:848-859).
    The gate and up matrices are stored as one [gate | up] matrix so that one product serves both; where a
    kernel carries the activation in its epilogue the [T, 2 * intermediate] product never exists in memory."""

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

    def emit(self, plan: Plan, h: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        act = rt.workspace("act", self.inter, rt.dtype)
        gate_up = rt.workspace("gate_up", 2 * self.inter, rt.dtype)
        plan.linear_swiglu(h, self.w_gate_up, gate_up, act)
        delta = rt.workspace("ffn_out", self.hidden, torch.float32)
        plan.linear(act, self.w_down, delta)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]
