"""The step function: one call runs one batch of (request, its next tokens) through the model,
from the cache that earlier steps left, and returns the logits at the wanted places.

The reference's Executor::run serves one sequence per run with a fixed token count
(src/runtime/executor.cpp:45-77) and advances the cache length once per run, after all
layers (src/runtime/runtime_context.cpp:222-243; the paged path latches the write position in
src/runtime/kernels/cpu_kernel_adapter.cpp:482-492).  `Engine.step` keeps those rules — every
layer of a step writes at the same positions, lengths move once per step — for a batch that
mixes prompt portions of some requests with single decoded tokens of others.

The engine has no policy: which requests run, how prompts are cut and when requests end is
decided by the caller (the scheduler, or a trace).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheError, CacheManager, OutOfPages
from ..config import EngineConfig, config_from_dict, load_config
from ..parts.base import Runtime
from ..weights import load_model_weights, random_model_weights
from .batch import GroupView, StepBatch
from .model import Model


class StepError(ValueError):
    """The batch was refused; no state was changed."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them (0-based,
    within `tokens`) whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Engine:
    SHORT_CONTEXT = 8192        # captured decode steps come in two kinds: every context up to here, and longer ones

    def __init__(self, model_dir: Optional[str] = None, *, config=None, random_seed: Optional[int] = None,
                 engine_config: Optional[EngineConfig] = None, ops=None):
        """`model_dir`: a folder with config.json and model.safetensors.  Or `config` (a typed
        configuration, or a dict of config.json keys) with `random_seed` for random weights made
        on the device.  `ops` replaces the CUDA kernel set (tests of the host logic only)."""
        self.ec = ec = engine_config or EngineConfig()
        if model_dir is not None:
            self.config = load_config(model_dir)
        elif config is not None:
            self.config = config_from_dict(config) if isinstance(config, dict) else config
        else:
            raise ValueError("Engine needs a model folder or a configuration")
        self.device = torch.device(ec.device)
        self.dtype = torch.bfloat16 if ec.dtype == "bfloat16" else torch.float32
        if ops is None:
            from ..kernels.ops import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        self.spec = self.config.model_spec()
        self.max_model_len = min(ec.max_model_len or self.spec.max_positions, self.spec.max_positions)
        if hasattr(ops, "choose_kernels"):
            ops.choose_kernels(ec.kernels)
        self.rt = Runtime(ops, self.device, self.dtype, ec.max_num_batched_tokens, ec.kernels, ec.max_num_seqs)
        self.model = Model(self.spec, self.rt)
        if model_dir is not None:
            load_model_weights(self.model, self.config, model_dir, self.dtype, self.device)
        else:
            if random_seed is None:
                raise ValueError("a configuration without a model folder needs random_seed")
            random_model_weights(self.model, random_seed, self.dtype, self.device)
        self.vocab_size = self.spec.vocab_size

        specs = self.model.cache_specs()
        tokens = ec.max_cached_tokens or self._tokens_from_free_memory(specs)
        self.cache = CacheManager(specs, ec.page_size, tokens, ec.max_num_seqs, self.max_model_len)
        self.cache.allocate_device(self.dtype, self.device)
        self._caches = []
        for i, (spec, cache_from) in enumerate(specs):
            owner = self.cache.run_owner[i]
            if spec is None:
                self._caches.append(None)
                continue
            tensor = self.cache.kv[owner] if getattr(spec, "paged", False) else self.cache.state[owner]
            self._caches.append(spec.view(tensor, self.cache.run_group[i], cache_from is None))
        self._init_metadata()
        self.steps = 0
        # decode-only steps are captured in CUDA graphs, one per batch size, after one eager step of that size
        self.graphs_enabled = (bool(ec.use_cuda_graphs) and self.device.type == "cuda"
                               and all(p.capture_safe and hasattr(p, "emit") for p in self.model.parts()))
        self._graphs: Dict[tuple, tuple] = {}
        self._graph_seen: set = set()
        self._graph_pool = None

    # ------------------------------------------------------------------ sizing
    def _tokens_from_free_memory(self, specs) -> int:
        per_token = sum(int(s.bytes_per_token(self.dtype)) for s, c in specs
                        if s is not None and c is None and getattr(s, "paged", False))
        if per_token == 0:
            return self.ec.page_size
        if self.device.type != "cuda":
            return self.ec.max_num_seqs * min(self.max_model_len, 4096)
        free, _ = torch.cuda.mem_get_info(self.device)
        # leave room for the step's workspace: roughly 64 bytes per hidden value of each token of the budget
        workspace = self.ec.max_num_batched_tokens * self.spec.hidden_size * 64 + (2 << 30)
        usable = max(0, int(free * self.ec.gpu_memory_fraction) - workspace)
        tokens = usable // per_token
        cap = self.ec.max_num_seqs * self.max_model_len
        tokens = min(tokens, cap)
        if tokens < self.ec.page_size:
            raise CacheError("no device memory is left for the cache after the weights")
        return int(tokens)

    # ------------------------------------------------------------------ step metadata
    def _init_metadata(self) -> None:
        T, R, G = self.ec.max_num_batched_tokens, self.ec.max_num_seqs, len(self.cache.groups)
        self._T_cap, self._R_cap = T, R
        names = ["token_ids", "positions", "token_request", "logit_rows"] + [f"slot_mapping{g}" for g in range(G)]
        self._off: Dict[str, slice] = {}
        o = 0
        for n in names:
            self._off[n] = slice(o, o + T)
            o += T
        for n, ln in (("cu_q_lens", R + 1), ("ctx_lens", R), ("state_slots", R), ("first_portion", R),
                      ("decode_rows", R), ("portion_rows", R)):
            self._off[n] = slice(o, o + ln)
            o += ln
        self._meta_len = o
        pin = self.device.type == "cuda"
        self._staging = [torch.zeros(o, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._staging_np = [s.numpy() for s in self._staging]
        self._staging_ev = [torch.cuda.Event() if pin else None for _ in range(2)]
        self._staging_used = [False, False]
        self._meta_dev = torch.zeros(o, dtype=torch.int32, device=self.device)

    def _build_batch(self, entries: List[StepEntry], starts: List[int]) -> StepBatch:
        i = self.steps & 1
        if self._staging_ev[i] is not None and self._staging_used[i]:
            self._staging_ev[i].synchronize()
        h = self._staging_np[i]
        off = self._off
        q_lens = [len(e.tokens) for e in entries]
        T, R = sum(q_lens), len(entries)
        cu = np.zeros(R + 1, dtype=np.int32)
        cu[1:] = np.cumsum(q_lens)
        tok = h[off["token_ids"]]
        pos = h[off["positions"]]
        treq = h[off["token_request"]]
        rows: List[int] = []
        for r, (e, s) in enumerate(zip(entries, starts)):
            a, b = int(cu[r]), int(cu[r + 1])
            st = self.cache.requests[e.request]
            tok[a:b] = np.asarray(e.tokens, dtype=np.int32)
            pos[a:b] = np.arange(s, s + (b - a), dtype=np.int32)
            treq[a:b] = st.slot
            for g in range(len(self.cache.groups)):
                h[off[f"slot_mapping{g}"]][a:b] = self.cache.slot_mapping(e.request, g, s, b - a)
            rows.extend(a + int(w) for w in e.want)
            h[off["ctx_lens"]][r] = s + (b - a)
            h[off["state_slots"]][r] = st.slot
            h[off["first_portion"]][r] = 1 if s == 0 else 0
        h[off["cu_q_lens"]][: R + 1] = cu
        dec = [r for r, q in enumerate(q_lens) if q == 1]
        por = [r for r, q in enumerate(q_lens) if q != 1]
        h[off["decode_rows"]][:len(dec)] = dec
        h[off["portion_rows"]][:len(por)] = por
        NL = len(rows)
        h[off["logit_rows"]][:NL] = np.asarray(rows, dtype=np.int32) if NL else 0
        self._meta_dev.copy_(self._staging[i], non_blocking=True)
        if self._staging_ev[i] is not None:
            self._staging_ev[i].record()
            self._staging_used[i] = True
        d = self._meta_dev

        def view(name: str, n: int) -> torch.Tensor:
            s = off[name]
            return d[s.start:s.start + n]

        groups = [GroupView(g.page_size, g.window, self.cache.tables_dev[gi], view(f"slot_mapping{gi}", T), g.max_blocks)
                  for gi, g in enumerate(self.cache.groups)]
        return StepBatch(
            num_tokens=T, num_requests=R, q_lens=q_lens, start_positions=list(starts),
            token_ids=view("token_ids", T), positions=view("positions", T), token_request=view("token_request", T),
            cu_q_lens=view("cu_q_lens", R + 1), ctx_lens=view("ctx_lens", R), state_slots=view("state_slots", R),
            first_portion=view("first_portion", R), logit_rows=view("logit_rows", NL),
            decode_rows=view("decode_rows", len(dec)), portion_rows=view("portion_rows", len(por)), groups=groups)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], end: Sequence[Hashable] = (),
             device_tokens: Optional[tuple] = None) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch.  Returns 32-bit logits [wanted, vocab] on the device,
        in the order of the entries and of their `want` lists (None if nothing is wanted); the tensor
        is overwritten by the next step.  Requests named in `end` give back what they hold after the
        step.  A request is created by its first entry.  A refused batch changes nothing.

        `device_tokens = (tensor, indices)`: for a step of single tokens, entry r's token is not the
        (placeholder) value in the entry but `tensor[indices[r]]`, an int32 tensor on the device (the
        output of the previous step's sampler): the step can be launched before the host has seen it."""
        entries = [e for e in entries if len(e.tokens) > 0]
        fast = self._decode_step(entries, end, device_tokens)
        if fast is not NotImplemented:
            return fast
        if device_tokens is not None:
            raise StepError("tokens on the device are only taken for a step of single tokens of live requests")
        seen = set()
        total = 0
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            total += n
            toks = np.asarray(e.tokens)
            if toks.ndim != 1 or not np.issubdtype(toks.dtype, np.integer):
                raise StepError(f"request {e.request!r}: tokens must be a flat list of integers")
            if toks.min() < 0 or toks.max() >= self.vocab_size:
                # the reference's CPU embedding refuses such ids too (src/runtime/kernels/cpu_kernel_adapter.cpp:73-78)
                raise StepError(f"request {e.request!r}: a token id is outside the vocabulary [0, {self.vocab_size})")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
            if len(set(int(w) for w in e.want)) != len(e.want):
                # the final norm adds the pending contribution into each wanted row once per mention
                raise StepError(f"request {e.request!r}: a place is wanted twice")
        for r in end:
            if r not in seen and not self.cache.has(r):
                raise StepError(f"request {r!r} is ended but is not live")
        if total > self._T_cap:
            raise StepError(f"the step has {total} tokens, the budget is {self._T_cap} (max_num_batched_tokens)")
        if len(entries) > self._R_cap:
            raise StepError(f"the step has {len(entries)} requests, the limit is {self._R_cap} (max_num_seqs)")
        starts = []
        for e in entries:
            s = self.cache.length(e.request) if self.cache.has(e.request) else 0
            if s + len(e.tokens) > self.max_model_len:
                raise StepError(f"request {e.request!r} would reach {s + len(e.tokens)} tokens, "
                                f"the model's limit is {self.max_model_len}")
            starts.append(s)

        # reserve: new requests and pages, undone together if anything is short
        created = []
        grown = []
        try:
            for e, s in zip(entries, starts):
                if not self.cache.has(e.request):
                    self.cache.add_request(e.request)
                    created.append(e.request)
                before = [len(b) for b in self.cache.requests[e.request].blocks]
                grown.append((e.request, before))
                self.cache.reserve(e.request, s + len(e.tokens))
        except (OutOfPages, CacheError) as err:
            self._undo(created, grown)
            raise StepError(f"the step does not fit the cache: {err}") from None

        logits = None
        if entries:
            batch = self._build_batch(list(entries), starts)
            self.cache.flush()
            logits = self._forward(batch)
            for e, s in zip(entries, starts):
                self.cache.advance(e.request, s + len(e.tokens))
            self.steps += 1
        for r in end:
            self.cache.free_request(r)
        return logits

    @property
    def takes_device_tokens(self) -> bool:
        """Whether `step(..., device_tokens=...)` is served: by every model (any number of cache groups, with or
        without a window, with or without state slots)."""
        return True

    def _decode_step(self, entries, end, device_tokens=None):
        """The common case made cheap on the host: every entry is one token of a live request that wants
        its logits.  Same checks and same effects as the general path, computed with whole-batch array
        operations instead of per-request ones.  Returns NotImplemented when the batch is of another kind."""
        R = len(entries)
        if R == 0 or R > self._R_cap:
            return NotImplemented
        reqs = self.cache.requests
        states = []
        for e in entries:
            st = reqs.get(e.request)
            if st is None or len(e.tokens) != 1 or len(e.want) != 1 or e.want[0] != 0:
                return NotImplemented
            states.append(st)
        if len({id(st) for st in states}) != R:
            return NotImplemented                          # a request twice: let the general path refuse it
        for r in end:
            if r not in reqs:
                return NotImplemented
        toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
        if toks.min() < 0 or toks.max() >= self.vocab_size:
            return NotImplemented
        lengths = np.fromiter((st.length for st in states), dtype=np.int64, count=R)
        if lengths.max() + 1 > self.max_model_len:
            return NotImplemented
        slots = np.fromiter((st.slot for st in states), dtype=np.int64, count=R)
        groups = self.cache.groups
        growing = set()
        for gi, g in enumerate(groups):
            grow = np.nonzero(lengths % g.page_size == 0)[0]       # these requests step onto a new page of this group
            short = [int(i) for i in grow if len(states[i].blocks[gi]) * g.page_size <= lengths[i]]
            if len(short) > g.pool.free_count:
                return NotImplemented                      # the general path raises the error and undoes nothing
            growing.update(short)
        for i in sorted(growing):
            self.cache.reserve(entries[i].request, int(lengths[i]) + 1)
        i = self.steps & 1
        if self._staging_ev[i] is not None and self._staging_used[i]:
            self._staging_ev[i].synchronize()
        h, off = self._staging_np[i], self._off
        ar = np.arange(R, dtype=np.int32)
        h[off["token_ids"]][:R] = toks
        h[off["positions"]][:R] = lengths
        h[off["token_request"]][:R] = slots
        for gi, g in enumerate(groups):
            ps = g.page_size
            h[off[f"slot_mapping{gi}"]][:R] = self.cache.tables[gi][slots, lengths // ps].astype(np.int64) * ps + lengths % ps
        h[off["logit_rows"]][:R] = ar
        h[off["cu_q_lens"]][:R + 1] = np.arange(R + 1, dtype=np.int32)
        h[off["ctx_lens"]][:R] = lengths + 1
        h[off["state_slots"]][:R] = slots
        h[off["first_portion"]][:R] = lengths == 0
        h[off["decode_rows"]][:R] = ar
        if device_tokens is not None:
            h[off["portion_rows"]][:R] = np.asarray(device_tokens[1], dtype=np.int32)   # unused in a decode step: carries the indices
        self._meta_dev.copy_(self._staging[i], non_blocking=True)
        if self._staging_ev[i] is not None:
            self._staging_ev[i].record()
            self._staging_used[i] = True
        d = self._meta_dev

        def view(name: str, n: int) -> torch.Tensor:
            s = off[name]
            return d[s.start:s.start + n]

        if device_tokens is not None:
            torch.index_select(device_tokens[0], 0, view("portion_rows", R), out=view("token_ids", R))
        views = [GroupView(g.page_size, g.window, self.cache.tables_dev[gi], view(f"slot_mapping{gi}", R), g.max_blocks)
                 for gi, g in enumerate(groups)]
        batch = StepBatch(
            num_tokens=R, num_requests=R, q_lens=[1] * R, start_positions=lengths.tolist(),
            token_ids=view("token_ids", R), positions=view("positions", R), token_request=view("token_request", R),
            cu_q_lens=view("cu_q_lens", R + 1), ctx_lens=view("ctx_lens", R), state_slots=view("state_slots", R),
            first_portion=view("first_portion", R), logit_rows=view("logit_rows", R),
            decode_rows=view("decode_rows", R), portion_rows=view("portion_rows", 0), groups=views)
        self.cache.flush()
        logits = self._forward(batch)
        if any(g.window for g in groups):
            for e, n in zip(entries, lengths):             # pages that a window has passed go back
                self.cache.advance(e.request, int(n) + 1)
        else:
            for st in states:
                st.length += 1
        self.steps += 1
        for r in end:
            self.cache.free_request(r)
        return logits

    def _forward(self, batch: StepBatch) -> Optional[torch.Tensor]:
        """Eager launch sequence, or the replay of a captured one for decode-only steps in which every
        request wants its logits.  What a captured step bakes in is only the number of requests; tokens,
        positions, lengths and block tables are data in device buffers that are rewritten before each replay."""
        R = batch.num_requests
        if not (self.graphs_enabled and batch.decode_only and batch.logit_rows.numel() == R):
            return self.model.forward(batch, self._caches)
        # launch shapes must serve every context length that replays of the capture will meet: one capture for
        # contexts up to SHORT_CONTEXT (where few blocks per request, merged inside a cluster, are fastest) and
        # one for everything up to the longest sequence
        short = batch.max_ctx_len <= self.SHORT_CONTEXT < self.max_model_len
        key = (R, short)
        rec = self._graphs.get(key)
        if rec is not None:
            graph, logits, launches, _keep = rec
            graph.replay()
            self.ops.launches += launches
            return logits
        batch.assume_ctx = self.SHORT_CONTEXT if short else self.max_model_len
        if key not in self._graph_seen:                 # first step of this kind: eager, so every buffer exists
            self._graph_seen.add(key)
            return self.model.forward(batch, self._caches)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = self.ops.launches
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(batch, self._caches)
        launches = self.ops.launches - before
        self.ops.launches = before
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        # the captured kernels hold raw pointers into the workspace: keep those buffers alive with the graph
        self._graphs[key] = (graph, logits, launches, dict(self.rt._buffers))
        graph.replay()
        self.ops.launches += launches
        return logits

    def _undo(self, created, grown) -> None:
        """Take back what a refused batch had reserved, last first, so that the free lists (last in, first
        out) and the free slots stand exactly as before: the pages a later request gets do not depend on
        whether a batch was refused in between."""
        for req, before in reversed(grown):
            st = self.cache.requests[req]
            for gi in reversed(range(len(before))):
                n = before[gi]
                extra = st.blocks[gi][n:]
                if extra:
                    self.cache.groups[gi].pool.free([p for p in reversed(extra) if p >= 0])
                    del st.blocks[gi][n:]
                    self.cache.tables[gi][st.slot, n:n + len(extra)] = -1
                    self.cache._mark(gi, st.slot, n, n + len(extra))
        for req in reversed(created):
            self.cache.forget_request(req)

    def free(self, request: Hashable) -> None:
        self.cache.free_request(request)

    def check_kernels(self) -> None:
        """Raise if a bounded wait inside a kernel ever gave up (synchronises the device)."""
        libs = getattr(self.ops, "_libs", {})
        status = self.ops.linear_tc_status() if "gemm_tcgen05" in libs else 0
        for key in libs:
            if key.startswith("attention_tc@HEAD_DIM="):
                status = status or self.ops.attention_tc_status(int(key.split("=")[1]))
        if status:
            raise RuntimeError(f"a tcgen05 kernel gave up waiting (code {status}): its results are not valid")
