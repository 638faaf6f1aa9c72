"""The plain implementation: Qwen3 dense, whole sequences, no cache, one
function per part, written from the reference's formulas.

It shares no code with the engine: it reads config.json and model.safetensors
itself (through the `safetensors` package) and computes with elementary tensor
arithmetic on the CPU.  `tests/golden/` holds logits that the reference's own
CPU executor produced for two tiny random models; `test_plain_model.py` checks
this file against them, so it does not rest on the formulas alone.

Every function cites the reference lines it restates (paths are relative to
the reference project's root).

`round_to` selects where values are rounded to bfloat16, to mirror the engine's
bfloat16 path (weights, the inputs of each matrix product and the cached keys
and values); the arithmetic itself is always 32-bit.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F32 = torch.float32


def _r(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F32)


# --------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t,:] = E[ids[t],:], no scaling (src/runtime/kernels/cpu_kernels.cpp:262-274).
    An id outside the table is an error (src/runtime/kernels/cpu_kernel_adapter.cpp:73-78)."""
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise IndexError("token id outside the vocabulary")
    return table[ids].to(F32)


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * 1/sqrt(mean(x^2) + eps) * gain, eps inside the root, gain used as stored
    (src/runtime/kernels/cpu_kernels.cpp:225-256; src/runtime/kernels/cuda_kernels.cu:360-378)."""
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return (x * (1.0 / torch.sqrt(ms + eps))) * gain.to(F32)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x W^T with W stored [out, in], no bias (src/runtime/kernels/cpu_kernel_adapter.cpp:107-124)."""
    return x @ w.to(F32).t()


def qk_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm over each head's `head_dim` values with one gain vector shared by all heads and the
    layer norms' eps; x is [T, heads, head_dim]
    (src/model/transformer_graph_builder.cpp:224-234; src/runtime/kernels/cpu_kernel_adapter.cpp:752-781)."""
    return rms_norm(x, gain, eps)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half pairs (d, d + head_dim/2) by angle pos * theta^(-2d/head_dim), angle in 32-bit
    (src/runtime/kernels/cpu_kernels.cpp:302-336; src/runtime/kernels/cuda_kernels.cu:430-450).
    x is [T, heads, head_dim]."""
    hd = x.shape[-1]
    half = hd // 2
    d = torch.arange(half, dtype=F32)
    inv = torch.pow(torch.tensor(theta, dtype=F32), (-2.0 * d) / hd)          # powf(base, -2d/hd)
    ang = positions.to(F32)[:, None] * inv[None, :]                           # fp32 product
    # cos/sin of the 32-bit angle, evaluated in 64-bit and rounded once
    co = torch.cos(ang.double()).to(F32)[:, None, :]
    si = torch.sin(ang.double()).to(F32)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * co - b * si, a * si + b * co], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over whole sequences.  q [T, nh, hd]; k, v [T, nkv, hd].
    Query head h uses key/value head h // (nh // nkv); scores are (q.k) * 1/sqrt(hd); keys after
    the query are masked; softmax with the maximum subtracted
    (src/runtime/kernels/cpu_kernels.cpp:338-420,444-448; src/runtime/kernels/cuda_kernels.cu:511-515).
    `window` W > 0 keeps only keys j with p - W < j <= p (the reference has no window: W = 0)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window > 0:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty(T, nh, hd, dtype=F32)
    for h in range(nh):
        s = (q[:, h] @ k[:, h // g].t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        s = s - s.max(-1, keepdim=True).values
        e = torch.exp(s)
        out[:, h] = (e / e.sum(-1, keepdim=True)) @ v[:, h // g]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """(g / (1 + exp(-g))) * u (src/runtime/kernels/cpu_kernels.cpp:848-859;
    src/runtime/kernels/cuda_kernels.cu:184-186,245-248)."""
    return (gate / (1.0 + torch.exp(-gate))) * up


# --------------------------------------------------------------------- model
class PlainQwen3:
    """Whole-sequence forward pass in the node order of
    src/model/transformer_graph_builder.cpp:129-294 (use_qk_norm on)."""

    def __init__(self, model_dir: str, round_to: Optional[torch.dtype] = None):
        from safetensors import safe_open

        with open(os.path.join(model_dir, "config.json")) as f:
            c = json.load(f)
        self.c = c
        self.round_to = round_to
        self.L = c["num_hidden_layers"]
        self.nh = c["num_attention_heads"]
        self.nkv = c.get("num_key_value_heads", self.nh)
        self.hd = c.get("head_dim", c["hidden_size"] // self.nh)
        self.eps = float(c["rms_norm_eps"])
        self.theta = float(c["rope_theta"])
        self.V = c["vocab_size"]
        self.windows = [0] * self.L
        if c.get("use_sliding_window"):
            types = c.get("layer_types") or [
                "sliding_attention" if i >= c.get("max_window_layers", self.L) else "full_attention"
                for i in range(self.L)]
            self.windows = [c["sliding_window"] if t == "sliding_attention" else 0 for t in types]
        order = c.get("layer_order") or list(range(self.L))
        self.order = [(e, None) if isinstance(e, int) else (e[0], e[1]) for e in order]
        self.w: Dict[str, torch.Tensor] = {}
        with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
            for name in f.keys():
                t = f.get_tensor(name).to(F32)
                # matrices take the rounding of the engine's compute type; gain vectors keep theirs
                self.w[name] = _r(t, round_to) if t.dim() == 2 else t
        if c.get("tie_word_embeddings", False):
            self.w["lm_head.weight"] = self.w["model.embed_tokens.weight"]

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        """[len(ids), vocab] logits of every position."""
        w, rt = self.w, self.round_to
        T = len(ids)
        pos = torch.arange(T)
        x = embedding(w["model.embed_tokens.weight"], ids)
        kept: List[Optional[tuple]] = []
        for run, (l, cache_from) in enumerate(self.order):
            p = f"model.layers.{l}."
            h = _r(rms_norm(x, w[p + "input_layernorm.weight"], self.eps), rt)
            q = _r(linear(h, w[p + "self_attn.q_proj.weight"]), rt).view(T, self.nh, self.hd)
            q = _r(rope(qk_norm(q, w[p + "self_attn.q_norm.weight"], self.eps), pos, self.theta), rt)
            if cache_from is None:
                k = _r(linear(h, w[p + "self_attn.k_proj.weight"]), rt).view(T, self.nkv, self.hd)
                v = _r(linear(h, w[p + "self_attn.v_proj.weight"]), rt).view(T, self.nkv, self.hd)
                k = _r(rope(qk_norm(k, w[p + "self_attn.k_norm.weight"], self.eps), pos, self.theta), rt)
                kept.append((k, v))
            else:
                k, v = kept[cache_from]
                kept.append(None)
            a = _r(attention(q, k, v, self.windows[l]).reshape(T, self.nh * self.hd), rt)
            x = linear(a, w[p + "self_attn.o_proj.weight"]) + x          # residual_add_1: o_proj + x
            h = _r(rms_norm(x, w[p + "post_attention_layernorm.weight"], self.eps), rt)
            g = _r(linear(h, w[p + "mlp.gate_proj.weight"]), rt)
            u = _r(linear(h, w[p + "mlp.up_proj.weight"]), rt)
            x = linear(_r(swiglu(g, u), rt), w[p + "mlp.down_proj.weight"]) + x   # residual_add_2
        h = _r(rms_norm(x, w["model.norm.weight"], self.eps), rt)
        return linear(h, w["lm_head.weight"])


# --------------------------------------------------------------------- sampling
def plain_sample(logits: torch.Tensor, *, greedy: bool = True, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 0.0, repetition_penalty: float = 1.0, history: Sequence[int] = (),
                 u: float = 0.5) -> int:
    """One token from one row of logits, in the order of src/runtime/sampler.cpp:11-141:
    repetition penalty once per occurrence in `history`, temperature, softmax, top-k, top-p,
    then argmax (greedy) or the first candidate whose running probability reaches `u`.
    The candidates are walked in vocabulary order and `u` is given by the caller; the
    reference walks them in sorted order with a Mersenne-twister draw."""
    z = logits.to(F32).clone()
    V = z.numel()
    if repetition_penalty != 1.0:
        for t in history:
            if 0 <= t < V:
                z[t] = z[t] / repetition_penalty if z[t] > 0 else z[t] * repetition_penalty
    if temperature != 1.0 and temperature > 0.0:
        z = z * (1.0 / temperature)
    m = z.max()
    if not torch.isfinite(m):
        p = torch.full((V,), 1.0 / V)
    else:
        e = torch.exp(z - m)
        p = e / e.sum()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if 0.0 < top_p < 1.0:
        sp = torch.sort(torch.where(keep, p, torch.zeros(())), descending=True).values
        cum = torch.cumsum(sp, 0)
        cutoff = int((cum >= top_p).nonzero()[0]) if bool((cum >= top_p).any()) else V - 1
        keep &= p >= sp[cutoff]
    if greedy:
        return int(torch.argmax(torch.where(keep, p, torch.full((), -1.0))))
    pc = torch.where(keep, p, torch.zeros(()))
    cum = torch.cumsum(pc.double(), 0) / float(pc.double().sum())
    idx = (cum >= u).nonzero()
    return int(idx[0]) if idx.numel() else int(keep.nonzero()[-1])
