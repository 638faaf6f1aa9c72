"""RMS norm over the residual stream, fused with the pending residual add."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..engine.plan import ROWS_LOGITS, ROWS_TOKENS, Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = (x * 1/sqrt(mean(x^2) + eps)) * gain, eps inside the root, gain used as stored
    (src/runtime/kernels/cpu_kernels.cpp:225-256).  The reference adds the residual with a
    separate Add node before the norm (src/model/transformer_graph_builder.cpp:251-257); here
    the norm kernel takes the not-yet-added contribution `delta` and does both."""

    def __init__(self, rt: Runtime, prefix: str, size: int, eps: float):
        super().__init__(rt, prefix)
        self.size = int(size)
        self.eps = float(eps)
        self.gain: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name("weight"): WeightSpec((self.size,), role="vector", init="gain")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name("weight")]

    def emit(self, plan: Plan, x: torch.Tensor, delta: Optional[torch.Tensor] = None, rows: str = ROWS_TOKENS) -> torch.Tensor:
        out = self.rt.workspace("normed" if rows == ROWS_TOKENS else "normed_rows", self.size, self.rt.dtype)
        plan.rmsnorm(x, self.gain, self.eps, out, delta=delta, rows=rows)
        return out

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        out = self.emit(plan, x, delta=delta, rows=ROWS_TOKENS if out_rows is None else ROWS_LOGITS)
        run_alone(self.rt, plan, StepBatch.bare(x.shape[0], x.device, logit_rows=out_rows))
        return out[: x.shape[0] if out_rows is None else out_rows.numel()]
