"""Interfaces of the parts a layer is made of, and the registries that build
them from `PartSpec` values.

A part gets its sizes and constants as constructor parameters, declares the
tensors it needs (`weight_specs`), receives them on the device (`load_weights`)
and computes through the kernel module of its `Runtime`.  No part knows which
model, layer or architecture it belongs to.

Categories and what each must provide
-------------------------------------
norm            `forward(x, out_rows=None, delta=None) -> h`: `x` is the 32-bit residual stream
                [T, size]; with `delta` the part first adds it to `x` in place; with `out_rows`
                (int32 indices) only those rows are normalised and returned.
position        `rotary_table()` -> a [max_positions, head_dim] 32-bit table (cos | sin) for the fused
                kernel, or None; then `apply(q, k, positions)` must rotate q and k in place.
mixer           `cache_spec()` -> `PagedKVSpec`, `StateSpec` or None;
                `forward(h, batch, cache) -> delta [T, hidden]`.
feed_forward    `forward(h, batch) -> delta [T, hidden]`.
block           arranges one mixer, one feed-forward and their norms:
                `forward(x, delta, batch, cache) -> (x, delta)`, where `delta` is a contribution
                not yet added to the residual stream `x` (the next norm adds it).
embedding       `forward(token_ids, out) -> x`.
head            `forward(h) -> logits` (32-bit).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part needs.  `role` decides the stored type: a "matrix" is an operand of a
    matrix product and takes the engine's compute type; a "vector" keeps 32-bit storage when the
    file has it so (else the file's 16-bit type); a "table" is integer data kept as int32.
    `init` is used by the random-weights mode: "normal" ~ N(0, 0.02), "gain" ~ 1 + N(0, 0.1)."""

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKVSpec:
    """A mixer that keeps keys and values of earlier tokens in pages.
    `window` = 0 keeps all of them; W > 0 only needs the last W positions."""

    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps a state of fixed size per request (zeroed when a request starts)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base class: holds the runtime and the tensor-name prefix."""

    # False for a part whose forward reads device data on the host (it then cannot be captured in a
    # CUDA graph, and steps of a model that holds such a part always run eagerly)
    capture_safe = True

    def __init__(self, rt: "Runtime", prefix: str):
        self.rt = rt
        self.prefix = prefix

    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Full tensor name -> spec, for every tensor this part (and its sub-parts) reads."""
        return {}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by `weight_specs`, already on the device."""

    def name(self, leaf: str) -> str:
        return f"{self.prefix}.{leaf}" if self.prefix else leaf


class Runtime:
    """What every part computes with: the device, the activation type, the kernel module and a
    workspace of reusable buffers."""

    def __init__(self, ops: Any, device: torch.device, dtype: torch.dtype, max_tokens: int, kernels: str = "fast"):
        self.ops = ops
        self.device = device
        self.dtype = dtype                 # type of matrix-product operands: bfloat16 or float32
        self.max_tokens = max_tokens
        self.kernels = kernels
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple[str, torch.dtype, int, int], torch.Tensor] = {}   # the views handed out, by shape
        self._tables: Dict[Any, torch.Tensor] = {}

    def buffer(self, name: str, rows: int, cols: int, dtype: torch.dtype, exact: bool = False,
               zero: bool = False) -> torch.Tensor:
        """A [rows, cols] view of a persistent buffer: the same name gives the same memory every
        step (so captured steps can be replayed), grown only when a larger shape is asked for.
        `exact`: the buffer is not indexed by tokens, make it only as large as asked for.
        `zero`: the memory is zeroed when it is allocated (not at later calls)."""
        view = self._views.get((name, dtype, rows, cols))
        if view is not None:
            return view
        key = (name, dtype)
        need = max(rows, 1) * cols
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < need:
            self._views = {k: v for k, v in self._views.items() if k[:2] != key}   # they show the old memory
            full = self.max_tokens * cols
            itemsize = torch.empty((), dtype=dtype).element_size()
            # token-indexed buffers are made for the step's token budget at once; very wide ones
            # (logits) only as large as asked for
            cap = max(need, full) if (not exact and full * itemsize <= (256 << 20)) else need
            buf = (torch.zeros if zero else torch.empty)(cap, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        view = buf[: rows * cols].view(rows, cols)
        if len(self._views) < 4096:
            self._views[(name, dtype, rows, cols)] = view
        return view

    def shared_table(self, key: Any, make: Callable[[], torch.Tensor]) -> torch.Tensor:
        """Constant tables (rotary cos/sin) built once per distinct key and shared by all layers."""
        t = self._tables.get(key)
        if t is None:
            t = make().to(self.device)
            self._tables[key] = t
        return t


_REGISTRIES: Dict[str, Dict[str, Callable[..., Part]]] = {
    c: {} for c in ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
}


def register_part(category: str, kind: str) -> Callable[[Callable[..., Part]], Callable[..., Part]]:
    """Class decorator: `@register_part("mixer", "my_mixer")`.  The class is built as
    `cls(rt, prefix, **spec.params)`."""
    if category not in _REGISTRIES:
        raise ValueError(f"unknown part category {category!r}; known: {', '.join(_REGISTRIES)}")

    def deco(cls: Callable[..., Part]) -> Callable[..., Part]:
        if kind in _REGISTRIES[category]:
            raise ValueError(f"{category} kind {kind!r} is already registered")
        _REGISTRIES[category][kind] = cls
        return cls

    return deco


def unregister_part(category: str, kind: str) -> None:
    _REGISTRIES[category].pop(kind, None)


def build_part(category: str, spec: PartSpec, rt: Runtime, prefix: str) -> Part:
    reg = _REGISTRIES[category]
    if spec.kind not in reg:
        raise KeyError(f"no {category} of kind {spec.kind!r} is registered; known: {', '.join(sorted(reg)) or '(none)'}")
    try:
        return reg[spec.kind](rt, prefix, **dict(spec.params))
    except TypeError as e:
        raise TypeError(f"building {category} {spec.kind!r} at {prefix!r}: {e}") from None


def registered(category: str):
    return sorted(_REGISTRIES[category])
