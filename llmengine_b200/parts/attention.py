"""Grouped-query attention over the paged cache, with optional per-head QK norm and a
position encoding chosen by the configuration."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..engine.plan import Plan
from .base import PagedKVSpec, Part, Runtime, WeightSpec, build_part, register_part, run_alone


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q, k, v projections (no bias) -> per-head RMS norm of q and k with one gain vector each and
    `qk_norm_eps` (None = no QK norm) -> position encoding -> keys and values stored in the cache
    -> causal attention, query head h reading key/value head h // (num_heads // num_kv_heads),
    scores scaled by 1/sqrt(head_dim) -> output projection.
    (src/model/transformer_graph_builder.cpp:214-248; attention arithmetic in
    src/runtime/kernels/cpu_kernels.cpp:338-420.)

    `window` = 0 attends to every earlier key; W > 0 to the last W keys (the query's own
    included), which the reference does not have.

    The three projections are stored as one matrix [q | k | v] so that one product serves them.
    """

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qk_norm_eps: Optional[float], position_encoding: PartSpec, window: int = 0):
        super().__init__(rt, prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        self.hidden, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window = int(window)
        self.q_size, self.kv_size = self.nh * self.hd, self.nkv * self.hd
        self.scale = 1.0 / math.sqrt(self.hd)
        self.position = build_part("position", position_encoding, rt, prefix)
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    # ------------------------------------------------------------------ weights
    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {
            self.name("q_proj.weight"): WeightSpec((self.q_size, self.hidden)),
            self.name("k_proj.weight"): WeightSpec((self.kv_size, self.hidden)),
            self.name("v_proj.weight"): WeightSpec((self.kv_size, self.hidden)),
            self.name("o_proj.weight"): WeightSpec((self.hidden, self.q_size)),
        }
        if self.eps is not None:
            s[self.name("q_norm.weight")] = WeightSpec((self.hd,), role="vector", init="gain")
            s[self.name("k_norm.weight")] = WeightSpec((self.hd,), role="vector", init="gain")
        return s

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([t[self.name("q_proj.weight")], t[self.name("k_proj.weight")],
                                t[self.name("v_proj.weight")]], dim=0).contiguous()
        self.w_o = t[self.name("o_proj.weight")].contiguous()
        if self.eps is not None:
            qg, kg = t[self.name("q_norm.weight")], t[self.name("k_norm.weight")]
            if qg.dtype != kg.dtype:          # one kernel launch takes one gain type
                qg, kg = qg.float(), kg.float()
            self.q_gain, self.k_gain = qg.contiguous(), kg.contiguous()

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.nkv, self.hd, self.window)

    # ------------------------------------------------------------------ compute
    def emit(self, plan: Plan, h: torch.Tensor, cache) -> torch.Tensor:
        """q|k|v product -> norm, position encoding, cache write, attention -> output product.  Which kernels serve
        a step (one that norms, rotates, stores and attends in one launch for steps of single tokens; the tensor-core
        kernels for prompt portions; the plain kernel) is the executor's choice, step by step."""
        rt = self.rt
        qs, kvs = self.q_size, self.kv_size
        writes = cache.writes
        width = qs + 2 * kvs if writes else qs
        qkv = rt.workspace("qkv", width, rt.dtype)
        plan.linear(h, self.w_qkv[:width], qkv)
        q = rt.workspace("q", qs, rt.dtype)
        out = rt.workspace("attn_out", qs, rt.dtype)
        scratch = rt.attention_scratch(self.nh, self.nkv, self.hd)
        common = dict(cache=cache.kv, group=cache.group, num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd)
        norm = dict(q_gain=self.q_gain, k_gain=self.k_gain, eps=self.eps or 0.0)
        table = self.position.rotary_table()
        if table is not None or not getattr(self.position, "needs_apply", True):
            plan.attention(qkv=qkv, q=q, out=out, writes=writes, window=self.window, scale=self.scale, cos_sin=table,
                           scratch=scratch, **common, **norm)
        else:
            # a position encoding without a rotary table: norm, then the part's own `apply`, then the write
            k = rt.workspace("k", kvs, rt.dtype) if writes else None
            plan.qkv_post(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs] if writes else None, v_in=None, q_out=q, k_out=k,
                          num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd, **norm)
            plan.call(lambda batch: self.position.apply(rt.rows(q), rt.rows(k), batch.positions, self.nh, self.nkv),
                      f"position encoding of {self.prefix}")
            if writes:
                plan.qkv_post(q_in=None, k_in=k, v_in=qkv[:, qs + kvs:], **common)
            plan.attend(q=q, out=out, window=self.window, scale=self.scale, scratch=scratch, **common)
        delta = rt.workspace("mixer_out", self.hidden, torch.float32)
        plan.linear(out, self.w_o, delta)
        return delta

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        plan = Plan()
        delta = self.emit(plan, h, cache)
        run_alone(self.rt, plan, batch)
        return delta[: h.shape[0]]
