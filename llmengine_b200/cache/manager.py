"""The cache manager: pages of keys and values with a block table per request, one pool per
group of layers with the same needs, and slots for per-request state of fixed size.

What is kept from the reference's PagedKVCache (src/runtime/cache/paged_kv_cache.cpp): a
last-in-first-out free list that hands out page 0 first (:48-52), a used-bitmap that catches a
double free (:282-286), all-or-nothing reservation that leaves the state untouched when pages
run out (:327-349), one block table per request shared by all layers of a group.  What is
new: groups (layers that keep every key, layers that keep a window of them: each group has
pages and block tables of its own, and a window group gives pages back as soon as the window
has passed them), state slots, runs that read another run's cache, and device-resident block
tables that are patched when a request gets or loses a page instead of being rebuilt each step.

This file is host logic only and needs no GPU; the device tensors are made by `allocate_device`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch



class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """Not enough free pages (or no free slot); nothing was changed."""


class PagePool:
    """Free pages of one group.  LIFO: the page freed last is handed out first."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs a positive number of pages, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._used = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._used[p] = True
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._used[p]:
                raise CacheError(f"page {p} is freed but is not in use")
        for p in pages:
            self._used[p] = False
            self._free.append(p)

    def check(self, held: Sequence[int]) -> None:
        """Every page is either free or held exactly once."""
        held = list(held)
        if len(set(held)) != len(held):
            raise CacheError("a page is held twice")
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        if set(held) & set(self._free):
            raise CacheError("a page is both held and free")
        if len(held) + len(self._free) != self.num_pages:
            raise CacheError(f"{self.num_pages - len(held) - len(self._free)} pages are lost")


@dataclass
class Group:
    """Layers (runs of the order) whose caches grow and shrink together."""

    page_size: int
    window: int                       # 0 = every position is kept
    pool: PagePool
    runs: List[int] = field(default_factory=list)
    max_blocks: int = 0
    committed: int = 0                # pages promised to admitted requests (admission control)

    def first_needed_block(self, length: int) -> int:
        """Blocks below this index hold only positions that no later query can see."""
        if self.window <= 0:
            return 0
        return max(0, length - self.window + 1) // self.page_size

    def peak_pages(self, total_tokens: int, max_portion: int) -> int:
        """Most pages a request of `total_tokens` holds at once when it is fed at most
        `max_portion` tokens a step."""
        full = -(-total_tokens // self.page_size)
        if self.window <= 0:
            return full
        span = self.window - 1 + max_portion
        return min(full, -(-span // self.page_size) + 1)


@dataclass
class RequestState:
    slot: int
    length: int = 0
    blocks: List[List[int]] = field(default_factory=list)   # per group; -1 = given back
    committed: List[int] = field(default_factory=list)      # per group: pages promised at admission


class CacheManager:
    """Pages, block tables and state slots for up to `max_requests` live requests.

    `specs[i] = (cache spec | None, cache_from)` for run i of the layer order.  A cache spec is any object with
    `paged`, `window`, `allocate(count, page_size, dtype, device)`, `bytes_per_token(dtype)` and, for states,
    `zero_on_start` (parts/base.py describes them); the manager asks nothing else of it.
    """

    def __init__(self, specs: Sequence[Tuple[object, Optional[int]]], page_size: int, max_cached_tokens: int,
                 max_requests: int, max_request_len: int):
        if page_size <= 0 or max_cached_tokens <= 0 or max_requests <= 0 or max_request_len <= 0:
            raise CacheError("page_size, max_cached_tokens, max_requests and max_request_len must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_request_len = max_request_len
        self.specs = list(specs)
        self.groups: List[Group] = []
        self.run_group: List[Optional[int]] = []     # run -> group index (paged runs)
        self.run_owner: List[int] = []               # run -> run whose tensor it uses
        by_key: Dict[Tuple[int, int], int] = {}
        num_pages = -(-max_cached_tokens // page_size)
        max_blocks = -(-max_request_len // page_size)
        for i, (spec, cache_from) in enumerate(self.specs):
            owner = i if cache_from is None else cache_from
            self.run_owner.append(owner)
            if cache_from is not None:
                if self.specs[cache_from][0] != spec:
                    raise CacheError(f"run {i} cannot read the cache of run {cache_from}: "
                                     f"{spec} differs from {self.specs[cache_from][0]}")
                self.run_group.append(self.run_group[cache_from])
                continue
            if spec is not None and getattr(spec, "paged", False):
                key = (page_size, int(getattr(spec, "window", 0)))
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(Group(page_size, key[1], PagePool(num_pages), max_blocks=max_blocks))
                self.groups[by_key[key]].runs.append(i)
                self.run_group.append(by_key[key])
            else:
                self.run_group.append(None)
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self.requests: Dict[Hashable, RequestState] = {}
        # host mirror of the device block tables, one row per slot
        self.tables = [np.full((max_requests, g.max_blocks), -1, dtype=np.int32) for g in self.groups]
        self._dirty: List[Dict[int, Tuple[int, int]]] = [dict() for _ in self.groups]   # slot -> [lo, hi) changed
        self.kv: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.tables_dev: List[torch.Tensor] = []
        self._new_slots: List[int] = []

    # ------------------------------------------------------------------ device side
    def allocate_device(self, dtype: torch.dtype, device: torch.device) -> None:
        """Make the page tensor of every owning paged run (for the attention of this package
        [pages, 2, kv_heads, page_size, head_dim]), the state tensor [slots, ...] of every stateful run, each as
        its spec lays it out, and the device block tables."""
        for i, (spec, cache_from) in enumerate(self.specs):
            if cache_from is not None or spec is None:
                continue
            if getattr(spec, "paged", False):
                g = self.groups[self.run_group[i]]
                self.kv[i] = spec.allocate(g.pool.num_pages, g.page_size, dtype, device)
            else:
                self.state[i] = spec.allocate(self.max_requests, self.page_size, dtype, device)
        self.tables_dev = [torch.from_numpy(t).to(device) for t in self.tables]
        self._patch_ring = [(None, None) for _ in range(8)]
        self._patch_next = 0

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        return sum(int(s.bytes_per_token(dtype)) for s, c in self.specs
                   if s is not None and c is None and getattr(s, "paged", False))

    def flush(self) -> None:
        """Bring the device block tables and the states of newly started requests up to date, without
        waiting for the device: the changed table entries travel as (position, value) pairs through a
        small ring of pinned buffers and are scattered into the tables by the stream."""
        if not self.tables_dev:
            self._dirty = [dict() for _ in self.groups]
            self._new_slots = []
            return
        for gi, dirty in enumerate(self._dirty):
            if not dirty:
                continue
            width = self.tables[gi].shape[1]
            idx = np.concatenate([np.arange(slot * width + lo, slot * width + hi, dtype=np.int64)
                                  for slot, (lo, hi) in dirty.items()])
            val = self.tables[gi].reshape(-1)[idx]
            dirty.clear()
            n = idx.size
            ring = self._patch_ring
            slot_i = self._patch_next % len(ring)
            self._patch_next += 1
            pinned, event = ring[slot_i]
            if pinned is None or pinned.shape[1] < n:
                pinned = torch.empty(2, max(n, 1024), dtype=torch.int64)
                if self.tables_dev[gi].is_cuda:
                    pinned = pinned.pin_memory()
                event = torch.cuda.Event() if self.tables_dev[gi].is_cuda else None
                ring[slot_i] = (pinned, event)
            elif event is not None:
                event.synchronize()                       # the copy that last used this buffer has been issued long ago
            pinned[0, :n] = torch.from_numpy(idx)
            pinned[1, :n] = torch.from_numpy(val.astype(np.int64))
            dev = pinned[:, :n].to(self.tables_dev[gi].device, non_blocking=True)
            if event is not None:
                event.record()
            self.tables_dev[gi].view(-1).index_copy_(0, dev[0], dev[1].to(torch.int32))
        for slot in self._new_slots:
            for run, st in self.state.items():
                if getattr(self.specs[run][0], "zero_on_start", True):
                    st[slot].zero_()
        self._new_slots = []

    # ------------------------------------------------------------------ requests
    def has(self, req: Hashable) -> bool:
        return req in self.requests

    def length(self, req: Hashable) -> int:
        return self.requests[req].length

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.free_count

    def add_request(self, req: Hashable) -> RequestState:
        if req in self.requests:
            raise CacheError(f"request {req!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are in use")
        st = RequestState(slot=self._free_slots.pop(), blocks=[[] for _ in self.groups],
                          committed=[0 for _ in self.groups])
        self.requests[req] = st
        self._new_slots.append(st.slot)
        return st

    def _mark(self, gi: int, slot: int, lo: int, hi: int) -> None:
        old = self._dirty[gi].get(slot)
        self._dirty[gi][slot] = (lo, hi) if old is None else (min(lo, old[0]), max(hi, old[1]))

    def reserve(self, req: Hashable, new_length: int) -> None:
        """Make sure pages exist for positions < new_length in every group.  All or nothing."""
        st = self.requests[req]
        if new_length > self.max_request_len:
            raise CacheError(f"request {req!r} would reach {new_length} tokens, the limit is {self.max_request_len}")
        need = []
        for gi, g in enumerate(self.groups):
            n = max(0, -(-new_length // g.page_size) - len(st.blocks[gi]))
            if n > g.pool.free_count:
                raise OutOfPages(
                    f"request {req!r} needs {n} more pages of group {gi} (window {g.window}), {g.pool.free_count} are free")
            need.append(n)
        for gi, (g, n) in enumerate(zip(self.groups, need)):
            if not n:
                continue
            first = len(st.blocks[gi])
            pages = g.pool.alloc(n)
            st.blocks[gi].extend(pages)
            self.tables[gi][st.slot, first:first + n] = pages
            self._mark(gi, st.slot, first, first + n)

    def advance(self, req: Hashable, new_length: int) -> None:
        """The request now holds `new_length` tokens; pages that every window has passed go back."""
        st = self.requests[req]
        if new_length < st.length:
            raise CacheError("a request cannot shrink")
        st.length = new_length
        for gi, g in enumerate(self.groups):
            stop = min(g.first_needed_block(new_length), len(st.blocks[gi]))
            gone = [(b, p) for b, p in enumerate(st.blocks[gi][:stop]) if p >= 0]
            if gone:
                g.pool.free([p for _, p in gone])
                for b, _ in gone:
                    st.blocks[gi][b] = -1
                self.tables[gi][st.slot, gone[0][0]:gone[-1][0] + 1] = -1
                self._mark(gi, st.slot, gone[0][0], gone[-1][0] + 1)

    def free_request(self, req: Hashable) -> None:
        st = self.requests.pop(req, None)
        if st is None:
            raise CacheError(f"request {req!r} is not live")
        for gi, g in enumerate(self.groups):
            g.pool.free([p for p in st.blocks[gi] if p >= 0])
            n = len(st.blocks[gi])
            if n:
                self.tables[gi][st.slot, :n] = -1
                self._mark(gi, st.slot, 0, n)
            g.committed -= st.committed[gi]
        self._free_slots.append(st.slot)

    def forget_request(self, req: Hashable) -> None:
        """Undo `add_request` for a request that never ran: it must hold no pages."""
        st = self.requests.pop(req, None)
        if st is None:
            raise CacheError(f"request {req!r} is not live")
        if any(p >= 0 for b in st.blocks for p in b) or any(st.committed):
            raise CacheError(f"request {req!r} holds pages or promises: it cannot be forgotten")
        self._free_slots.append(st.slot)
        if st.slot in self._new_slots:
            self._new_slots.remove(st.slot)

    # ------------------------------------------------------------------ admission control
    def try_commit(self, req: Hashable, total_tokens: int, max_portion: int) -> bool:
        """Promise the request the pages it will need at its peak, in every group, or promise nothing.
        A scheduler that admits only what it could commit never runs out of pages later."""
        st = self.requests[req]
        peaks = [g.peak_pages(total_tokens, max_portion) for g in self.groups]
        if any(g.committed + p > g.pool.num_pages for g, p in zip(self.groups, peaks)):
            return False
        for gi, (g, p) in enumerate(zip(self.groups, peaks)):
            g.committed += p
            st.committed[gi] = p
        return True

    def fits_at_all(self, total_tokens: int, max_portion: int) -> bool:
        return total_tokens <= self.max_request_len and all(
            g.peak_pages(total_tokens, max_portion) <= g.pool.num_pages for g in self.groups)

    # ------------------------------------------------------------------ lookups for the step
    def slot_mapping(self, req: Hashable, group: int, start: int, count: int) -> np.ndarray:
        """Physical cache rows (page * page_size + slot-in-page) of positions start..start+count-1."""
        st = self.requests[req]
        ps = self.groups[group].page_size
        pos = np.arange(start, start + count, dtype=np.int64)
        blocks = np.asarray(st.blocks[group], dtype=np.int64)[pos // ps]
        if (blocks < 0).any():
            raise CacheError(f"request {req!r}: a position in [{start}, {start + count}) has no page")
        return (blocks * ps + pos % ps).astype(np.int32)

    def check_invariants(self) -> None:
        for gi, g in enumerate(self.groups):
            held = [p for st in self.requests.values() for p in st.blocks[gi] if p >= 0]
            g.pool.check(held)
            for st in self.requests.values():
                row = self.tables[gi][st.slot]
                n = len(st.blocks[gi])
                if list(row[:n]) != st.blocks[gi] or (row[n:] != -1).any():
                    raise CacheError("a block table row does not match its request")
        slots = [st.slot for st in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots) or \
                len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("state slots are lost or held twice")
