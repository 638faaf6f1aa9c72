"""Position encodings applied to queries and keys."""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .base import Part, Runtime, register_part


@register_part("position", "rope")
class RotaryEncoding(Part):
    """Rotate-half rotary encoding: the pairs (d, d + head_dim/2) of each head are rotated by
    the angle pos * theta^(-2d/head_dim) (src/runtime/kernels/cpu_kernels.cpp:302-336;
    src/runtime/kernels/cuda_kernels.cu:430-450).

    The reference evaluates powf, the product with the position and cosf/sinf in 32-bit inside
    the kernel.  Here the same 32-bit angle (32-bit power, 32-bit product) is formed once on
    the host for every position, its cosine and sine are evaluated in 64-bit and rounded once
    to 32-bit, and the kernels read that table: every kernel and every way of batching sees
    identical values.
    """

    needs_apply = False           # the fused kernels rotate with `rotary_table()`

    def __init__(self, rt: Runtime, prefix: str, head_dim: int, theta: float, max_positions: int):
        super().__init__(rt, prefix)
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {head_dim}")
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)

    @staticmethod
    def build_table(head_dim: int, theta: float, max_positions: int) -> torch.Tensor:
        half = head_dim // 2
        d = np.arange(half, dtype=np.float32)
        expo = (np.float32(-2.0) * d) / np.float32(head_dim)                       # 32-bit exponent
        inv = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
        pos = np.arange(max_positions, dtype=np.float32)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)                     # 32-bit angle
        table = np.concatenate([np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))], axis=1)
        return torch.from_numpy(table.astype(np.float32))

    def rotary_table(self) -> Optional[torch.Tensor]:
        """[max_positions, head_dim]: cos of the head_dim/2 angles, then their sin."""
        key = ("rope", self.head_dim, self.theta, self.max_positions)
        return self.rt.shared_table(key, lambda: self.build_table(self.head_dim, self.theta, self.max_positions))

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor,
              num_heads: int, num_kv_heads: int) -> None:
        """Unfused form: rotate q [T, nh*hd] and k [T, nkv*hd] in place."""
        self.rt.ops.qkv_post(q_in=q, k_in=k, v_in=None, num_heads=num_heads, num_kv_heads=num_kv_heads,
                             head_dim=self.head_dim, cos_sin=self.rotary_table(), positions=positions,
                             q_out=q, k_out=k)


@register_part("position", "none")
class NoPositionEncoding(Part):
    """Queries and keys are used as they are."""

    needs_apply = False           # nothing to do for queries and keys: a fused kernel may skip `apply`

    def __init__(self, rt: Runtime, prefix: str, **_ignored):
        super().__init__(rt, prefix)

    def rotary_table(self) -> Optional[torch.Tensor]:
        return None

    def apply(self, q, k, positions, num_heads, num_kv_heads) -> None:
        return None
