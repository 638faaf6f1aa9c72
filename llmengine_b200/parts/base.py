"""Interfaces of the parts a layer is made of, and the registries that build
them from `PartSpec` values.

A part gets its sizes and constants as constructor parameters, declares the
tensors it needs (`weight_specs`), receives them on the device (`load_weights`)
and computes through the kernel module of its `Runtime`.  No part knows which
model, layer or architecture it belongs to.

Categories and what each must provide
-------------------------------------
A part says what it computes in one of two ways.  `emit(plan, ...)` appends operation records to the
model's plan when the model is loaded (engine/plan.py); its tensor arguments and results are workspace
buffers made for the step's token budget, of which a step uses the first rows.  That is what the parts of
this package do: their launch sequence then runs in the native executor.  Or `forward(...)`, which computes
a step's rows directly with tensor operations when the step runs; the model wraps it into a `call` record.
A part that has `emit` gets a `forward` of the same meaning for free (`run_alone`).

norm            `emit(plan, x, delta=None, rows="tokens") -> h` / `forward(x, delta=None, out_rows=None) -> h`:
                `x` is the 32-bit residual stream [T, size]; with `delta` the part first adds it to `x`
                in place; with rows="logits" / `out_rows` (int32 indices) only those rows are normalised.
position        `rotary_table()` -> a [max_positions, head_dim] 32-bit table (cos | sin) for the fused
                kernel, or None; then `apply(q, k, positions, nh, nkv)` must rotate q and k in place.
mixer           `cache_spec()` -> a cache spec (`PagedKVSpec`, `StateSpec`, one of your own) or None;
                `emit(plan, h, cache) -> delta` / `forward(h, batch, cache) -> delta [T, hidden]`.
feed_forward    `emit(plan, h) -> delta` / `forward(h, batch) -> delta [T, hidden]`.
block           arranges mixer, feed-forward and norms: `emit(plan, x, delta, cache) -> (x, delta)` /
                `forward(x, delta, batch, cache) -> (x, delta)`, where `delta` is a contribution
                not yet added to the residual stream `x` (the next norm adds it).
embedding       `emit(plan) -> x` / `forward(token_ids) -> x`.
head            `emit(plan, h)` (writes the step's logits) / `forward(h) -> logits` (32-bit).

Cache specs
-----------
What a mixer keeps between steps is described by an object with: `paged` (True: keys-and-values-like
data in pages with a block table per request; False: a state of fixed size per request), `window` (paged:
0 keeps every position, W > 0 only the last W), `allocate(count, page_size, dtype, device)` (the device
tensor for `count` pages or request slots), `bytes_per_token(dtype)` (paged: what one cached token costs,
for sizing the pool), `zero_on_start` (state: cleared when a request starts) and
`view(tensor, group, writes)` (what the mixer is handed).  The cache manager and the engine use only these.
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


@dataclass
class PagedKVView:
    """The cache a paged mixer run works on."""

    kv: torch.Tensor                # [pages, 2, kv_heads, page_size, head_dim]
    group: int                      # index into StepBatch.groups
    writes: bool                    # False when the run reads another run's cache


@dataclass
class StateView:
    """The fixed-size states of a stateful mixer run: row `batch.state_slots[r]` belongs to request r."""

    state: torch.Tensor             # [slots, *shape]


@dataclass(frozen=True)
class PagedKVSpec:
    """A mixer that keeps keys and values of earlier tokens in pages.
    `window` = 0 keeps all of them; W > 0 only needs the last W positions."""

    num_kv_heads: int
    head_dim: int
    window: int = 0
    paged = True

    def allocate(self, count: int, page_size: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        # a page of one head is a contiguous [page_size, head_dim] block: one TMA box, one run of vector loads
        return torch.zeros(count, 2, self.num_kv_heads, page_size, self.head_dim, dtype=dtype, device=device)

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        return 2 * self.num_kv_heads * self.head_dim * torch.empty((), dtype=dtype).element_size()

    def view(self, tensor: torch.Tensor, group: Optional[int], writes: bool) -> PagedKVView:
        return PagedKVView(tensor, group, writes)


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps a state of fixed size per request (zeroed when a request starts)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
    paged = False
    window = 0
    zero_on_start = True

    def allocate(self, count: int, page_size: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.zeros(count, *self.shape, dtype=self.dtype, device=device)

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        return 0

    def view(self, tensor: torch.Tensor, group: Optional[int], writes: bool) -> StateView:
        return StateView(tensor)


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

    def tied_tensors(self) -> Dict[str, str]:
        """Tensors this part does not store but shares with another part: its own tensor name -> the name of
        the tensor (declared by some other part) that it uses.  A weight file that still holds a copy under the
        part's own name is accepted, and the copy ignored."""
        return {}

    def receive_tied(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the shared tensors named by `tied_tensors` (own name -> the other part's device tensor)."""

    def shared_tensor(self, name: str) -> Optional[torch.Tensor]:
        """The device tensor this part holds for its weight `name`, if another part may share it."""
        return None


class Runtime:
    """What every part computes with: the device, the activation type, the kernel module and a
    workspace of reusable buffers."""

    def __init__(self, ops: Any, device: torch.device, dtype: torch.dtype, max_tokens: int, kernels: Any = "fast",
                 max_requests: int = 64):
        self.ops = ops
        self.device = device
        self.dtype = dtype                 # type of matrix-product operands: bfloat16 or float32
        self.max_tokens = max_tokens
        self.max_requests = max_requests   # most requests in one step
        self.kernels = kernels
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[Tuple[str, torch.dtype, int, int], torch.Tensor] = {}   # the views handed out, by shape
        self._tables: Dict[Any, torch.Tensor] = {}
        self.batch = None                  # the StepBatch of the step that is running (for `call` records)

    def workspace(self, name: str, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """The [max_tokens, cols] buffer of this name: what `emit` hands from one record to the next."""
        return self.buffer(name, self.max_tokens, cols, dtype)

    def attention_scratch(self, num_heads: int, num_kv_heads: int, head_dim: int) -> Optional[torch.Tensor]:
        """Scratch memory of the split-context decode attention, large enough for any step of this engine (one
        buffer for all layers; its leading ticket counters start at zero and every launch leaves them so)."""
        need = getattr(self.ops, "attention_scratch_floats", None)
        n = need(self.max_requests, num_heads, num_kv_heads, head_dim) if need is not None else 0
        if n <= 0:
            return None
        return self.buffer("attention_scratch", 1, n, torch.float32, exact=True, zero=True).view(-1)

    def rows(self, t: Optional[torch.Tensor], n: Optional[int] = None) -> Optional[torch.Tensor]:
        """The first rows of a workspace buffer: those of the running step's tokens (or `n` of them)."""
        if t is None:
            return None
        return t[: (self.batch.num_tokens if n is None else n)]

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


# ----------------------------------------------------------------------------- emitting, for parts with and without `emit`
def run_alone(rt: Runtime, plan, batch) -> None:
    """Compile a plan and run it once for `batch` (a part used by itself: tests, tools)."""
    outer, rt.batch = rt.batch, batch          # a part may run another part by itself from inside a step
    try:
        rt.ops.compile(plan).run(batch)
    finally:
        rt.batch = outer


def _copy_rows(dst: torch.Tensor, src: torch.Tensor) -> None:
    if src.data_ptr() != dst.data_ptr():
        dst[: src.shape[0]].copy_(src)


def emit_embedding(plan, part: Part, hidden: int) -> torch.Tensor:
    if hasattr(part, "emit"):
        return part.emit(plan)
    rt = part.rt
    x = rt.workspace("residual", hidden, torch.float32)
    plan.call(lambda batch: _copy_rows(x, part.forward(batch.token_ids)), f"embedding {part.prefix}")
    return x


def emit_norm(plan, part: Part, x: torch.Tensor, delta: Optional[torch.Tensor] = None, rows: str = "tokens") -> torch.Tensor:
    if hasattr(part, "emit"):
        return part.emit(plan, x, delta=delta, rows=rows)
    rt = part.rt
    out = rt.workspace("normed_called" if rows == "tokens" else "normed_rows_called", x.shape[1], rt.dtype)

    def call(batch):
        y = part.forward(rt.rows(x), delta=rt.rows(delta), out_rows=batch.logit_rows if rows != "tokens" else None)
        _copy_rows(out, y.to(out.dtype))
    plan.call(call, f"norm {part.prefix}")
    return out


def emit_mixer(plan, part: Part, h: torch.Tensor, cache, hidden: int) -> torch.Tensor:
    if hasattr(part, "emit"):
        return part.emit(plan, h, cache)
    rt = part.rt
    out = rt.workspace("mixer_out_called", hidden, torch.float32)
    plan.call(lambda batch: _copy_rows(out, part.forward(rt.rows(h), batch, cache).float()), f"mixer {part.prefix}")
    return out


def emit_feed_forward(plan, part: Part, h: torch.Tensor, hidden: int) -> torch.Tensor:
    if hasattr(part, "emit"):
        return part.emit(plan, h)
    rt = part.rt
    out = rt.workspace("ffn_out_called", hidden, torch.float32)
    plan.call(lambda batch: _copy_rows(out, part.forward(rt.rows(h), batch).float()), f"feed_forward {part.prefix}")
    return out


def emit_block(plan, part: Part, x: torch.Tensor, delta: Optional[torch.Tensor], cache):
    if hasattr(part, "emit"):
        return part.emit(plan, x, delta, cache)
    rt = part.rt
    out = rt.workspace("block_out_called", x.shape[1], torch.float32)

    def call(batch):
        x2, d2 = part.forward(rt.rows(x), rt.rows(delta), batch, cache)
        _copy_rows(x, x2)
        if d2 is None:                       # nothing is left to be added (a block that ends on a norm)
            rt.rows(out).zero_()
        else:
            _copy_rows(out, d2.float())
    plan.call(call, f"block {part.prefix}")
    return x, out


def emit_head(plan, part: Part, h: torch.Tensor) -> None:
    if hasattr(part, "emit"):
        part.emit(plan, h)
        return
    plan.call(lambda batch: batch.logits.copy_(part.forward(h[: batch.logits.shape[0]])), f"head {part.prefix}")


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
