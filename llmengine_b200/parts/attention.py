"""Grouped-query attention over the paged cache, with optional per-head QK norm and a
position encoding chosen by the configuration."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from .base import PagedKVSpec, Part, Runtime, WeightSpec, build_part, register_part


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
    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        rt, ops = self.rt, self.rt.ops
        T = h.shape[0]
        group = batch.groups[cache.group]
        qs, kvs = self.q_size, self.kv_size
        writes = cache.writes
        width = qs + 2 * kvs if writes else qs
        qkv = rt.buffer("qkv", T, width, rt.dtype)
        ops.linear(h, self.w_qkv[:width], qkv)
        q_in = qkv[:, :qs]
        k_in = qkv[:, qs:qs + kvs] if writes else None
        v_in = qkv[:, qs + kvs:] if writes else None
        table = self.position.rotary_table()
        out = rt.buffer("attn_out", T, qs, rt.dtype)
        if self._decode_fused(batch, table, T):
            # a step of single new tokens: norm, rotation and cache write happen inside the attention kernel
            n_dec = batch.decode_rows.numel()
            splits = self.decode_splits(n_dec, batch.max_decode_ctx)
            scratch = None
            if splits > 1:
                need = ops.attention_decode_scratch_floats(self.hd, n_dec, self.nh, splits)
                scratch = rt.buffer("attention_scratch", 1, need, torch.float32, exact=True, zero=True)   # its counters start at zero
            ops.attention_decode_fused(qkv=qkv, q_gain=self.q_gain, k_gain=self.k_gain, eps=self.eps or 0.0, cos_sin=table,
                                       write_kv=writes, cache=cache.kv, out=out, rows=batch.decode_rows,
                                       cu_q_lens=batch.cu_q_lens, ctx_lens=batch.ctx_lens, table_rows=batch.state_slots,
                                       block_tables=group.block_tables, num_heads=self.nh, num_kv_heads=self.nkv,
                                       head_dim=self.hd, page_size=group.page_size, window=self.window, scale=self.scale,
                                       splits=splits, scratch=scratch)
            delta = rt.buffer("mixer_out", T, self.hidden, torch.float32)
            return ops.linear(out, self.w_o, delta)
        q = rt.buffer("q", T, qs, rt.dtype)
        norm = dict(q_gain=self.q_gain, k_gain=self.k_gain, eps=self.eps or 0.0)
        common = dict(num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd)
        if table is not None:
            ops.qkv_post(q_in=q_in, k_in=k_in, v_in=v_in, **common, **norm, cos_sin=table,
                         positions=batch.positions, q_out=q, cache=cache.kv if writes else None,
                         slot_mapping=group.slot_mapping, page_size=group.page_size)
        else:
            # a position encoding without a rotary table: norm, then the part's own `apply`, then the write
            k = rt.buffer("k", T, kvs, rt.dtype) if writes else None
            ops.qkv_post(q_in=q_in, k_in=k_in, v_in=None, **common, **norm, q_out=q, k_out=k)
            self.position.apply(q, k, batch.positions, self.nh, self.nkv)
            if writes:
                ops.qkv_post(q_in=None, k_in=k, v_in=v_in, **common, cache=cache.kv,
                             slot_mapping=group.slot_mapping, page_size=group.page_size)
        self.attend(q, cache.kv, out, batch, group)
        delta = rt.buffer("mixer_out", T, self.hidden, torch.float32)
        return ops.linear(out, self.w_o, delta)

    def _decode_fused(self, batch, table, T: int) -> bool:
        """Whether this step's attention can take the raw projections: the tensor-core kernels serve this head
        size, every request brings exactly one token, and the position encoding is either the rotary table or
        none at all (a part with an `apply` of its own needs the unfused path)."""
        rt, ops = self.rt, self.rt.ops
        if not (rt.kernels == "fast" and hasattr(ops, "attention_decode_fused") and hasattr(ops, "fast_attention_supports")
                and ops.fast_attention_supports(self.hd, rt.dtype)):
            return False
        if batch.portion_rows.numel() or batch.decode_rows.numel() != T:
            return False
        return table is not None or not getattr(self.position, "needs_apply", True)

    def attend(self, q, kv, out, batch, group) -> None:
        """Attention of every token of the batch over its request's cache.  bfloat16 with head sizes
        the tensor-core kernels are built for: requests with one new token go to the split-context
        decode kernel, the others to a portion kernel (the tcgen05 one for head sizes 64 and 128 with
        pages it can load by TMA, else the mma.sync one).  Everything else (32-bit, other head sizes,
        `kernels="plain"`) goes to the plain kernel, which serves every case."""
        rt, ops = self.rt, self.rt.ops
        common = dict(q=q, cache=kv, out=out, block_tables=group.block_tables, num_heads=self.nh,
                      num_kv_heads=self.nkv, head_dim=self.hd, page_size=group.page_size, window=self.window,
                      scale=self.scale)
        fast = (rt.kernels == "fast" and hasattr(ops, "fast_attention_supports")
                and ops.fast_attention_supports(self.hd, q.dtype))
        if not fast:
            ops.attention_plain(positions=batch.positions, token_request=batch.token_request, **common)
            return
        meta = dict(cu_q_lens=batch.cu_q_lens, ctx_lens=batch.ctx_lens, table_rows=batch.state_slots)
        n_dec = batch.decode_rows.numel()
        if batch.portion_rows.numel():
            tc = (hasattr(ops, "tc_attention_supports")
                  and ops.tc_attention_supports(self.hd, q.dtype, self.nh, self.nkv, group.page_size))
            portions = ops.attention_portions_tc if tc else ops.attention_portions
            portions(rows=batch.portion_rows, max_q_len=batch.max_portion_len, **meta, **common)
        if n_dec:
            splits = self.decode_splits(n_dec, batch.max_decode_ctx)
            scratch = None
            if splits > 1:
                need = ops.attention_decode_scratch_floats(self.hd, n_dec, self.nh, splits)
                scratch = rt.buffer("attention_scratch", 1, need, torch.float32, exact=True, zero=True)   # its counters start at zero
            ops.attention_decode(rows=batch.decode_rows, splits=splits, scratch=scratch, **meta, **common)

    def decode_splits(self, n_requests: int, max_ctx: int) -> int:
        """Blocks per (request, key/value head): as many as fit the GPU in one wave (148 SMs, two blocks
        each), never more than there are 64-key groups in the longest (windowed) context.  Up to 8 splits
        run as one thread-block cluster and merge through shared memory, which is worth more than a finer
        split while a block's share stays short (measured at batch 1 and 2,048 keys: 8.3 us with 8 splits,
        8.9 us with 16, 11 us with 32)."""
        span = min(max_ctx, self.window) if self.window > 0 else max_ctx
        groups = max(1, -(-span // 64) + (1 if self.window > 0 else 0))
        blocks = n_requests * self.nkv * (-(-(self.nh // self.nkv) // 16))
        splits = max(1, min(groups, (2 * 148) // blocks, 64))
        if splits > 8 and span <= 8 * 1024:
            splits = 8
        return splits
