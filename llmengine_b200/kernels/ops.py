"""Python face of the CUDA kernels: loads the compiled libraries and launches
their `extern "C"` entry points on torch tensors, on torch's current stream.

There is no fallback: without a CUDA device, or if a library cannot be compiled
or loaded, `CudaOps` raises `KernelsUnavailable`.

A model does not call these methods one by one: its parts emit a plan once (engine/plan.py), `compile` turns
it into the records of the native executor (csrc/executor.cu, include/llmengine_b200/executor.h), and every
step is one call that walks them in C++.  Which kernel serves an operation for a step's shape is decided there,
in one place; `choose` exchanges single kernels (`EngineConfig.kernels`).  The only library matrix product is the
bfloat16 product of 17 to 127 tokens (and of larger steps whose tiles would not fill the GPU), which goes to
cuBLAS (the reference also hands its dense products to cuBLAS: src/runtime/kernels/cuda_kernels.cu:892-908);
the 32-bit product is this package's own FMA kernel.  The methods below that launch one kernel directly are what
the kernel tests and tools use.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional

import torch

from . import build
from . import executor as ex


class KernelsUnavailable(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


_F32, _BF16 = 0, 1
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return _F32
    if dt == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class _QkvArgs(Structure):
    _fields_ = [
        ("q_in", c_void_p), ("k_in", c_void_p), ("v_in", c_void_p),
        ("q_stride", c_longlong), ("k_stride", c_longlong), ("v_stride", c_longlong),
        ("q_gain", c_void_p), ("k_gain", c_void_p), ("gain_dtype", c_int), ("eps", c_float),
        ("cos_sin", c_void_p), ("positions", c_void_p), ("max_positions", c_int),
        ("q_out", c_void_p), ("k_out", c_void_p), ("cache", c_void_p), ("slot_mapping", c_void_p),
        ("tokens", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("page_size", c_int),
    ]


class _AttnArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("cache", c_void_p), ("out", c_void_p), ("positions", c_void_p),
        ("token_request", c_void_p), ("block_tables", c_void_p), ("max_blocks", c_int),
        ("tokens", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("page_size", c_int),
        ("window", c_int), ("scale", c_float),
    ]


class _FastAttnArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("cache", c_void_p), ("out", c_void_p), ("rows", c_void_p), ("cu_q_lens", c_void_p),
        ("ctx_lens", c_void_p), ("table_rows", c_void_p), ("block_tables", c_void_p), ("scratch", c_void_p),
        ("max_blocks", c_int), ("n_rows", c_int), ("nh", c_int), ("nkv", c_int), ("page_size", c_int),
        ("window", c_int), ("splits", c_int), ("scale", c_float),
    ]


class _FusedQkv(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("stride", c_longlong), ("q_gain", c_void_p), ("k_gain", c_void_p), ("gain_dtype", c_int),
        ("eps", c_float), ("cos_sin", c_void_p), ("max_positions", c_int), ("write_kv", c_int),
    ]


class _TcAttnArgs(Structure):
    _fields_ = [
        ("out", c_void_p), ("cache", c_void_p), ("rows", c_void_p), ("cu_q_lens", c_void_p), ("ctx_lens", c_void_p),
        ("table_rows", c_void_p), ("block_tables", c_void_p),
        ("max_blocks", c_int), ("n_rows", c_int), ("nh", c_int), ("nkv", c_int), ("page_size", c_int),
        ("window", c_int), ("scale", c_float),
    ]


class _SampleArgs(Structure):
    _fields_ = [
        ("logits", c_void_p), ("ld", c_longlong), ("rows", c_int), ("vocab", c_int),
        ("greedy", c_void_p), ("temperature", c_void_p), ("top_k", c_void_p), ("top_p", c_void_p),
        ("u", c_void_p), ("out", c_void_p),
    ]


class CudaOps:
    """The kernel set the parts compute with.  One instance per engine."""

    def __init__(self, device: torch.device):
        if not torch.cuda.is_available():
            raise KernelsUnavailable(
                "no CUDA device is visible: this engine runs only on a GPU (sm_100a) and has no CPU fallback")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelsUnavailable(f"device {device} is not a CUDA device")
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._libs: Dict[str, ctypes.CDLL] = {}
        self._sms = None
        self._direct = 0           # kernels launched through the methods below (the executor counts its own)
        self._xlib = self._lib("executor")
        ex.declare(self._xlib)
        with torch.cuda.device(self.device):
            self._ex = self._xlib.llme_executor_create(self._device_index)
        if not self._ex:
            raise KernelsUnavailable(f"the step executor cannot use device {device}")

    def __del__(self):
        try:
            if getattr(self, "_ex", None):
                self._xlib.llme_executor_destroy(self._ex)
                self._ex = None
        except Exception:
            pass

    # ------------------------------------------------------------------ the executor
    @property
    def launches(self) -> int:
        """Kernels of this package launched so far (library products are not counted)."""
        return self._direct + int(self._xlib.llme_executor_launches(self._ex))

    @launches.setter
    def launches(self, value: int) -> None:
        self._direct = int(value) - int(self._xlib.llme_executor_launches(self._ex))

    def choose(self, op: str, variant: str) -> None:
        """Which implementation an operation takes from now on (operations and variants: executor.h)."""
        if self._xlib.llme_executor_choose(self._ex, op.encode(), variant.encode()) != 0:
            raise KernelError(self._xlib.llme_executor_error(self._ex).decode())

    def chosen(self, op: str) -> str:
        return self._xlib.llme_executor_chosen(self._ex, op.encode()).decode()

    def choose_kernels(self, kernels) -> None:
        """`EngineConfig.kernels`: "fast", "plain", or a mapping operation -> variant applied on top of "fast"."""
        if isinstance(kernels, str):
            self.choose("*", kernels)
            return
        self.choose("*", "fast")
        for op, variant in dict(kernels).items():
            self.choose(op, variant)

    @property
    def plain_gemm(self) -> str:
        return self.chosen("linear")

    @plain_gemm.setter
    def plain_gemm(self, variant: str) -> None:
        self.choose("linear", variant)

    def attention_scratch_floats(self, max_requests: int, num_heads: int, num_kv_heads: int, head_dim: int) -> int:
        return int(self._xlib.llme_attention_scratch_floats(self._ex, max_requests, num_heads, num_kv_heads, head_dim))

    def decode_splits(self, requests: int, num_heads: int, num_kv_heads: int, head_dim: int, window: int, max_ctx: int) -> int:
        return int(self._xlib.llme_decode_splits(self._ex, requests, num_heads, num_kv_heads, head_dim, window, max_ctx))

    _ENTRY_POINTS = {
        "elementwise": {"embedding": "llme_embedding", "rmsnorm": "llme_rmsnorm", "qkv_post": "llme_qkv_post",
                        "swiglu": "llme_swiglu"},
        "gemm_f32": {"gemm_f32": "llme_gemm_nt_f32"},
        "gemm_skinny": {"gemm_skinny": "llme_gemm_skinny_bf16", "gemm_skinny_swiglu": "llme_gemm_skinny_swiglu_bf16"},
        "gemm_tcgen05": {"gemm_tc": "llme_gemm_tc_bf16", "gemm_tc_swiglu": "llme_gemm_tc_swiglu_bf16"},
        "attention_plain": {"attention_plain": "llme_attention_plain"},
        "attention_fast": {"attention_portion/{hd}": "llme_attention_portion", "attention_decode/{hd}": "llme_attention_decode",
                           "attention_decode_fused/{hd}": "llme_attention_decode_fused",
                           "attention_decode_scratch/{hd}": "llme_attention_decode_scratch_floats",
                           "attention_decode_clusters/{hd}": "llme_attention_decode_clusters"},
        "attention_tc": {"attention_tc/{hd}": "llme_attention_tc"},
    }

    def _register(self, key: str, lib: ctypes.CDLL) -> None:
        """Hand a kernel library's entry points (and its error text) to the executor, by name."""
        name, _, rest = key.partition("@")
        hd = rest.partition("=")[2]
        for entry, symbol in self._ENTRY_POINTS.get(name, {}).items():
            entry = entry.format(hd=hd)
            fn = ctypes.cast(getattr(lib, symbol), c_void_p)
            self._xlib.llme_executor_register(self._ex, entry.encode(), fn)
            self._xlib.llme_executor_register(self._ex, f"error/{entry.split('/')[0]}".encode(),
                                              ctypes.cast(lib.llme_last_error, c_void_p))

    def _libraries_for(self, plan) -> list:
        """The kernel libraries a plan can reach with the present choices: what has to be compiled for this model."""
        need = []

        def want(n):
            if n not in need:
                need.append(n)
        fast_attention = self.chosen("attention") == "fast"
        for op in plan.ops:
            a = op.a
            if op.kind in ("embedding", "rmsnorm", "qkv_post", "attention"):
                want("elementwise")
            if op.kind in ("linear", "linear_swiglu"):
                if a["x"].dtype == torch.float32:
                    want("gemm_f32")
                elif self.chosen("linear") != "plain":
                    if self.chosen("linear.decode") != "cublas":
                        want("gemm_skinny")
                    if self.chosen("linear") != "cublas":
                        want("gemm_tcgen05")
                if op.kind == "linear_swiglu":
                    want("elementwise")
            if op.kind in ("attend", "attention"):
                hd, dt = a["head_dim"], a["q"].dtype
                if fast_attention and self.fast_attention_supports(hd, dt):
                    want(f"attention_fast@HEAD_DIM={hd}")
                    if hd in (64, 128) and self.chosen("attention.portion") == "tcgen05":
                        want(f"attention_tc@HEAD_DIM={hd}")
                else:
                    want("attention_plain")
        return need

    def compile(self, plan) -> "CompiledPlan":
        """The native records of a plan, ready to run step after step."""
        self.require(*self._libraries_for(plan))
        return CompiledPlan(self, plan)

    # ------------------------------------------------------------------ loading
    def require(self, *names: str) -> None:
        """Compile (if needed) and load the named libraries."""
        missing = [n for n in names if n not in self._libs]
        if not missing:
            return
        try:
            paths = build.ensure_built(missing)
        except build.BuildError as e:
            raise KernelsUnavailable(str(e)) from None
        for n in missing:
            try:
                lib = ctypes.CDLL(paths[n])
            except OSError as e:
                raise KernelsUnavailable(f"cannot load {paths[n]}: {e}") from None
            lib.llme_last_error.restype = c_char_p
            self._libs[n] = lib
            if n != "executor" and getattr(self, "_ex", None):
                self._register(n, lib)

    def _lib(self, name: str) -> ctypes.CDLL:
        lib = self._libs.get(name)
        if lib is None:
            self.require(name)
            lib = self._libs[name]
        return lib

    def _check(self, lib: ctypes.CDLL, rc: int, what: str) -> None:
        self._direct += 1
        if rc != 0:
            msg = lib.llme_last_error().decode("utf-8", "replace")
            raise KernelError(f"{what}: {msg} (code {rc})")

    def _stream(self) -> c_void_p:
        # the current stream's handle; the raw getter costs a fraction of a microsecond, the Stream object ten
        if _raw_stream is not None:
            return c_void_p(_raw_stream(self._device_index))
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    # ------------------------------------------------------------------ kernels
    def embedding(self, ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        lib = self._lib("elementwise")
        assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
        rc = lib.llme_embedding(c_void_p(ids.data_ptr()), c_void_p(table.data_ptr()), c_int(_code(table.dtype)),
                                c_void_p(out.data_ptr()), c_int(ids.numel()), c_int(table.shape[1]),
                                c_int(table.shape[0]), self._stream())
        self._check(lib, rc, "embedding")
        return out

    def rmsnorm(self, x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        lib = self._lib("elementwise")
        assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
        assert delta is None or (delta.is_contiguous() and delta.shape == x.shape)
        n_out = out.shape[0]
        assert (rows.numel() if rows is not None else x.shape[0]) == n_out
        rc = lib.llme_rmsnorm(c_void_p(x.data_ptr()), c_void_p(_ptr(delta)),
                              c_int(_code(delta.dtype) if delta is not None else 0),
                              c_void_p(gain.data_ptr()), c_int(_code(gain.dtype)),
                              c_void_p(out.data_ptr()), c_int(_code(out.dtype)), c_void_p(_ptr(rows)),
                              c_int(n_out), c_int(x.shape[1]), c_float(eps), self._stream())
        self._check(lib, rc, "rmsnorm")
        return out

    def qkv_post(self, *, q_in, k_in, v_in, num_heads: int, num_kv_heads: int, head_dim: int,
                 q_gain=None, k_gain=None, eps: float = 0.0, cos_sin=None, positions=None,
                 q_out=None, k_out=None, cache=None, slot_mapping=None, page_size: int = 0) -> None:
        """QK norm, rotation and cache write for `tokens` rows; see csrc/elementwise.cu."""
        lib = self._lib("elementwise")
        ref = q_in if q_in is not None else (k_in if k_in is not None else v_in)
        tokens = ref.shape[0]
        outs = [t for t in (q_out, k_out, cache) if t is not None]
        if not outs:
            return
        out_dtype = outs[0].dtype
        assert all(t.dtype == out_dtype for t in outs)
        for t in (q_in, k_in, v_in):
            assert t is None or (t.dtype == ref.dtype and t.stride(-1) == 1)
        gains = [g for g in (q_gain, k_gain) if g is not None]
        assert all(g.dtype == gains[0].dtype for g in gains)
        a = _QkvArgs(
            _ptr(q_in), _ptr(k_in), _ptr(v_in),
            q_in.stride(0) if q_in is not None else 0, k_in.stride(0) if k_in is not None else 0,
            v_in.stride(0) if v_in is not None else 0,
            _ptr(q_gain), _ptr(k_gain), _code(gains[0].dtype) if gains else 0, eps,
            _ptr(cos_sin), _ptr(positions), cos_sin.shape[0] if cos_sin is not None else 0,
            _ptr(q_out), _ptr(k_out), _ptr(cache), _ptr(slot_mapping),
            tokens, num_heads, num_kv_heads, head_dim, page_size)
        rc = lib.llme_qkv_post(byref(a), c_int(_code(ref.dtype)), c_int(_code(out_dtype)), self._stream())
        self._check(lib, rc, "qkv_post")

    def attention_plain(self, *, q, cache, out, positions, token_request, block_tables, num_heads: int,
                        num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float) -> torch.Tensor:
        lib = self._lib("attention_plain")
        assert q.dtype == cache.dtype == out.dtype and q.is_contiguous() and out.is_contiguous()
        assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
        a = _AttnArgs(q.data_ptr(), cache.data_ptr(), out.data_ptr(), positions.data_ptr(), token_request.data_ptr(),
                      block_tables.data_ptr(), block_tables.shape[1], q.shape[0], num_heads, num_kv_heads, head_dim,
                      page_size, window, scale)
        rc = lib.llme_attention_plain(byref(a), c_int(_code(q.dtype)), self._stream())
        self._check(lib, rc, "attention_plain")
        return out

    @staticmethod
    def fast_attention_supports(head_dim: int, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128

    def _fast_lib(self, head_dim: int) -> ctypes.CDLL:
        key = f"attention_fast@HEAD_DIM={head_dim}"
        lib = self._lib(key)
        if not getattr(lib, "_llme_ready", False):
            lib.llme_attention_decode_scratch_floats.restype = c_longlong
            assert lib.llme_attention_head_dim() == head_dim
            lib._llme_ready = True
        return lib

    def _fast_args(self, q, cache, out, rows, cu_q_lens, ctx_lens, table_rows, block_tables, num_heads, num_kv_heads,
                   page_size, window, scale, splits=1, scratch=None) -> "_FastAttnArgs":
        assert q.dtype == cache.dtype == out.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous()
        assert block_tables.is_contiguous() and cache.is_contiguous()
        return _FastAttnArgs(q.data_ptr(), cache.data_ptr(), out.data_ptr(), rows.data_ptr(), cu_q_lens.data_ptr(),
                             ctx_lens.data_ptr(), table_rows.data_ptr(), block_tables.data_ptr(), _ptr(scratch),
                             block_tables.shape[1], rows.numel(), num_heads, num_kv_heads, page_size, window, splits,
                             scale)

    def attention_portions(self, *, q, cache, out, rows, cu_q_lens, ctx_lens, table_rows, block_tables, num_heads: int,
                           num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                           max_q_len: int) -> None:
        """Tensor-core attention for the requests `rows` of the batch, each with a portion of any length."""
        lib = self._fast_lib(head_dim)
        a = self._fast_args(q, cache, out, rows, cu_q_lens, ctx_lens, table_rows, block_tables, num_heads,
                            num_kv_heads, page_size, window, scale)
        rc = lib.llme_attention_portion(byref(a), c_int(max_q_len), self._stream())
        self._check(lib, rc, "attention_portions")

    def tc_attention_supports(self, head_dim: int, dtype: torch.dtype, num_heads: int, num_kv_heads: int,
                              page_size: int) -> bool:
        """Whether the tcgen05 portion kernel takes this shape (head size 64 or 128, pages of 8..128 that
        divide 128 or multiples of 128, a group size that divides 128)."""
        if not (dtype == torch.bfloat16 and head_dim in (64, 128)):
            return False
        g = num_heads // num_kv_heads
        pages_ok = page_size >= 8 and (128 % page_size == 0 if page_size <= 128 else page_size % 128 == 0)
        return pages_ok and 128 % g == 0

    def attention_portions_tc(self, *, q, cache, out, rows, cu_q_lens, ctx_lens, table_rows, block_tables,
                              num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                              scale: float, max_q_len: int) -> None:
        """The portion attention on the tcgen05 tensor cores (TMA-fed, scores and outputs in tensor memory)."""
        lib = self._lib(f"attention_tc@HEAD_DIM={head_dim}")
        assert q.dtype == cache.dtype == out.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous()
        assert cache.is_contiguous() and block_tables.is_contiguous()
        a = _TcAttnArgs(out.data_ptr(), cache.data_ptr(), rows.data_ptr(), cu_q_lens.data_ptr(), ctx_lens.data_ptr(),
                        table_rows.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], rows.numel(), num_heads,
                        num_kv_heads, page_size, window, scale)
        total_rows = cache.shape[0] * cache.shape[1] * cache.shape[2] * cache.shape[3]
        rc = lib.llme_attention_tc(c_void_p(q.data_ptr()), c_longlong(q.shape[0]), c_longlong(total_rows), byref(a),
                                   c_int(max_q_len), self._stream())
        self._check(lib, rc, "attention_tc")

    def attention_tc_status(self, head_dim: int) -> int:
        return int(self._lib(f"attention_tc@HEAD_DIM={head_dim}").llme_attention_tc_status())

    def attention_decode_scratch_floats(self, head_dim: int, n_rows: int, num_heads: int, splits: int) -> int:
        return int(self._fast_lib(head_dim).llme_attention_decode_scratch_floats(c_int(n_rows), c_int(num_heads), c_int(splits)))

    def attention_decode(self, *, q, cache, out, rows, cu_q_lens, ctx_lens, table_rows, block_tables, num_heads: int,
                         num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, splits: int,
                         scratch: Optional[torch.Tensor]) -> None:
        """Tensor-core attention for the requests `rows`, each with exactly one new token; the context
        of each is split over `splits` blocks whose partial results meet in `scratch`.  The first 65536
        words of `scratch` are counters: zero before the first call, left zero by every call."""
        lib = self._fast_lib(head_dim)
        if splits > 1:
            need = self.attention_decode_scratch_floats(head_dim, rows.numel(), num_heads, splits)
            assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need
        a = self._fast_args(q, cache, out, rows, cu_q_lens, ctx_lens, table_rows, block_tables, num_heads,
                            num_kv_heads, page_size, window, scale, splits, scratch)
        rc = lib.llme_attention_decode(byref(a), self._stream())
        self._check(lib, rc, "attention_decode")

    def attention_decode_fused(self, *, qkv, q_gain, k_gain, eps: float, cos_sin, write_kv: bool, cache, out, rows,
                               cu_q_lens, ctx_lens, table_rows, block_tables, num_heads: int, num_kv_heads: int,
                               head_dim: int, page_size: int, window: int, scale: float, splits: int,
                               scratch: Optional[torch.Tensor]) -> None:
        """attention_decode() on the raw q|k|v projections `qkv` [T, (nh + 2 nkv) * hd] (or [T, nh * hd] when nothing
        is stored): the kernel norms and rotates the heads itself and, if `write_kv`, stores the new keys and
        values in the cache before it attends."""
        lib = self._fast_lib(head_dim)
        if splits > 1:
            need = self.attention_decode_scratch_floats(head_dim, rows.numel(), num_heads, splits)
            assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need
        assert qkv.dtype == cache.dtype == out.dtype == torch.bfloat16 and qkv.stride(1) == 1 and out.is_contiguous()
        assert block_tables.is_contiguous() and cache.is_contiguous()
        assert (q_gain is None) == (k_gain is None) and (q_gain is None or q_gain.dtype == k_gain.dtype)
        a = _FastAttnArgs(None, cache.data_ptr(), out.data_ptr(), rows.data_ptr(), cu_q_lens.data_ptr(),
                          ctx_lens.data_ptr(), table_rows.data_ptr(), block_tables.data_ptr(), _ptr(scratch),
                          block_tables.shape[1], rows.numel(), num_heads, num_kv_heads, page_size, window, splits, scale)
        f = _FusedQkv(qkv.data_ptr(), qkv.stride(0), _ptr(q_gain), _ptr(k_gain),
                      _code(q_gain.dtype) if q_gain is not None else 0, float(eps or 0.0), _ptr(cos_sin),
                      cos_sin.shape[0] if cos_sin is not None else 0, 1 if write_kv else 0)
        rc = lib.llme_attention_decode_fused(byref(a), byref(f), self._stream())
        self._check(lib, rc, "attention_decode_fused")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        lib = self._lib("elementwise")
        assert gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape[1] == 2 * out.shape[1]
        rc = lib.llme_swiglu(c_void_p(gate_up.data_ptr()), c_int(_code(gate_up.dtype)), c_void_p(out.data_ptr()),
                             c_int(_code(out.dtype)), c_int(out.shape[0]), c_int(out.shape[1]), self._stream())
        self._check(lib, rc, "swiglu")
        return out

    def _run_one(self, record) -> None:
        """One operation through the executor, for all rows of its input (what `linear` and `linear_swiglu` below do):
        the executor's choice of kernel, outside any model."""
        from ..engine.batch import StepBatch
        from ..engine.plan import Plan
        plan = Plan()
        record(plan)
        rows = plan.ops[0].a["x"].shape[0]
        if rows > 0:
            self.compile(plan).run(StepBatch.bare(rows, self.device))

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[M,N] = x[M,K] @ w[N,K]^T by the kernel the executor chooses for this shape.  32-bit operands: this
        package's FMA kernel (never a reduced-precision mode).  bfloat16 operands: the weight-streaming kernel for
        up to 16 rows, the tcgen05 kernel for 128 rows or more when its tiles fill the GPU, else cuBLAS with 32-bit
        accumulation; the output in `out`'s type."""
        assert w.shape[1] == x.shape[1] and out.shape == (x.shape[0], w.shape[0])
        self._run_one(lambda plan: plan.linear(x, w, out))
        return out

    def linear_swiglu_supports(self, x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> bool:
        """Whether a kernel with the activation in its epilogue exists for this product (a handful of rows: the
        weight-streaming kernel; 128 rows or more: the tcgen05 kernel; bfloat16, 16-byte aligned rows)."""
        M, K = x.shape
        return (x.dtype == w_gate_up.dtype == out.dtype == torch.bfloat16 and (0 < M <= 16 or M >= 128) and K % 8 == 0
                and x.stride(1) == 1 and w_gate_up.stride(1) == 1 and out.stride(1) == 1 and x.stride(0) % 8 == 0
                and w_gate_up.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and out.shape[1] >= 8
                and x.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)

    def linear_swiglu(self, x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[M, I] = silu(x @ Wg^T) * (x @ Wu^T) with w_gate_up = [Wg | Wu] stacked by rows: in one kernel where the
        executor has one for the shape, else the product and the activation kernel behind it."""
        M, K = x.shape
        inter = out.shape[1]
        assert w_gate_up.shape == (2 * inter, K) and out.shape[0] == M
        gate_up = torch.empty(M, 2 * inter, dtype=x.dtype, device=x.device)
        self._run_one(lambda plan: plan.linear_swiglu(x, w_gate_up, gate_up, out))
        return out

    def linear_tc(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[M,N] = x[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory)."""
        lib = self._lib("gemm_tcgen05")
        M, K = x.shape
        N = w.shape[0]
        assert x.dtype == w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
        rc = lib.llme_gemm_tc_bf16(c_void_p(x.data_ptr()), c_longlong(x.stride(0)), c_void_p(w.data_ptr()),
                                   c_longlong(w.stride(0)), c_void_p(out.data_ptr()), c_int(_code(out.dtype)),
                                   c_longlong(out.stride(0)), c_int(M), c_int(N), c_int(K), self._stream())
        self._check(lib, rc, "gemm_tcgen05")
        return out

    def gemm_tc_pairing(self, how: str) -> None:
        """Whether the tcgen05 product runs on pairs of SMs (tcgen05 with .cta_group::2, 256-row tiles): "auto" (from
        129 tokens on), "single" (never) or "pair" (always).  For tests and measurements."""
        self._lib("gemm_tcgen05").llme_gemm_tc_pairing(c_int({"auto": 0, "single": 1, "pair": 2}[how]))

    def gemm_skinny_form(self, how: str) -> None:
        """The weight-streaming product with two blocks an SM ("two"), in its lighter form with three ("three", up to 8
        tokens) or as the kernel chooses by how its row groups fill their rounds ("auto").  For tests and measurements."""
        self._lib("gemm_skinny").llme_gemm_skinny_dense(c_int({"auto": 0, "two": 1, "three": 2}[how]))

    def linear_tc_status(self) -> int:
        """0 if no bounded wait of the tcgen05 kernels ever gave up (synchronises the device)."""
        return int(self._lib("gemm_tcgen05").llme_gemm_tc_status())

    def random_fill(self, out: torch.Tensor, key: int, start: int, scale: float, offset: float,
                    round_bf16_first: bool = False) -> torch.Tensor:
        """out.flatten()[i] = offset + scale * z(key, start + i): the device twin of weights.loader.counter_normal."""
        lib = self._lib("utility")
        assert out.is_contiguous()
        from ctypes import c_ulonglong
        rc = lib.llme_random_fill(c_void_p(out.data_ptr()), c_int(_code(out.dtype)), c_ulonglong(key & ((1 << 64) - 1)),
                                  c_longlong(start), c_longlong(out.numel()), c_float(scale), c_float(offset),
                                  c_int(1 if round_bf16_first else 0), self._stream())
        self._check(lib, rc, "random_fill")
        return out

    def read_stream(self, data: torch.Tensor, sink: torch.Tensor, blocks_per_sm: int = 4) -> None:
        """Reads `data` once and stores nothing: what the memory delivers to a kernel that only loads."""
        lib = self._lib("utility")
        nbytes = data.numel() * data.element_size()
        rc = lib.llme_read_stream(c_void_p(data.data_ptr()), c_longlong(nbytes), c_void_p(sink.data_ptr()),
                                  c_int(blocks_per_sm), self._stream())
        self._check(lib, rc, "read_stream")

    def repetition_penalty(self, logits, rows, tokens, counts, penalty) -> None:
        lib = self._lib("sampling")
        rc = lib.llme_repetition_penalty(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)),
                                         c_void_p(rows.data_ptr()), c_void_p(tokens.data_ptr()),
                                         c_void_p(counts.data_ptr()), c_void_p(penalty.data_ptr()),
                                         c_int(rows.numel()), c_int(logits.shape[1]), self._stream())
        self._check(lib, rc, "repetition_penalty")

    def sample(self, logits: torch.Tensor, *, greedy, temperature, top_k, top_p, u, out: torch.Tensor) -> torch.Tensor:
        lib = self._lib("sampling")
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
        a = _SampleArgs(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(greedy),
                        _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(u), out.data_ptr())
        rc = lib.llme_sample(byref(a), self._stream())
        self._check(lib, rc, "sample")
        return out


class CompiledPlan:
    """A plan as the native executor holds it.  `run(batch)` is one call into C++ that launches the whole step on
    torch's current stream."""

    def __init__(self, ops: CudaOps, plan) -> None:
        self.ops = ops
        self._lib = ops._xlib
        self._keep: list = [plan]
        self._handle = self._lib.llme_plan_create(ops._ex)
        self._failure: Optional[BaseException] = None
        self._step = ex.Step()
        for i, op in enumerate(plan.ops):
            if op.kind == "call":
                fn = ex.CallFn(self._guard(op.a["fn"]))
                self._keep.append(fn)
                kind, rec = ex.OP_CALL, ex.CallOp(fn, None)
            else:
                kind, rec = ex.records(op, self._keep)
            if self._lib.llme_plan_add(self._handle, kind, byref(rec), ctypes.sizeof(rec)) < 0:
                raise KernelError(f"operation {i} ({op.kind}): {self._lib.llme_executor_error(ops._ex).decode()}")

    def __del__(self):
        try:
            if self._handle:
                self._lib.llme_plan_destroy(self._handle)
                self._handle = None
        except Exception:
            pass

    def _guard(self, fn):
        """A part that runs in Python inside the native walk: its exception is kept and raised after the walk."""
        def call(_user, _step, _stream):
            try:
                fn(self._batch)
                return 0
            except BaseException as e:          # noqa: BLE001  (re-raised by run)
                self._failure = e
                return -2
        return call

    def run(self, batch, first: int = 0, count: int = -1) -> None:
        s = self._step
        s.num_tokens, s.num_requests = batch.num_tokens, batch.num_requests
        s.num_logit_rows = batch.logit_rows.numel()
        s.num_decode, s.num_portion = batch.decode_rows.numel(), batch.portion_rows.numel()
        s.max_portion_len, s.max_decode_ctx = batch.max_portion_len, batch.max_decode_ctx
        s.token_ids, s.positions, s.token_request = batch.token_ids.data_ptr(), batch.positions.data_ptr(), batch.token_request.data_ptr()
        s.cu_q_lens, s.ctx_lens, s.state_slots = batch.cu_q_lens.data_ptr(), batch.ctx_lens.data_ptr(), batch.state_slots.data_ptr()
        s.first_portion, s.logit_rows = batch.first_portion.data_ptr(), batch.logit_rows.data_ptr()
        s.decode_rows, s.portion_rows = batch.decode_rows.data_ptr(), batch.portion_rows.data_ptr()
        s.logits = batch.logits.data_ptr() if batch.logits is not None else None
        s.blas = torch.cuda.current_blas_handle()
        if len(batch.groups) > ex.MAX_GROUPS:
            raise KernelError(f"a step has {len(batch.groups)} cache groups, the executor takes {ex.MAX_GROUPS}")
        s.num_groups = len(batch.groups)
        for i, g in enumerate(batch.groups):
            sg = s.groups[i]
            sg.block_tables, sg.slot_mapping = g.block_tables.data_ptr(), g.slot_mapping.data_ptr()
            sg.max_blocks, sg.page_size, sg.window = g.block_tables.shape[1], g.page_size, g.window
        self._batch = batch
        rc = self._lib.llme_plan_run(self._handle, byref(s), first, count, self.ops._stream())
        self._batch = None
        if rc != 0:
            failure, self._failure = self._failure, None
            if failure is not None:
                raise failure
            raise KernelError(self._lib.llme_executor_error(self.ops._ex).decode())
