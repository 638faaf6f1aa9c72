"""Python face of the CUDA kernels: loads the compiled libraries and launches
their `extern "C"` entry points on torch tensors, on torch's current stream.

There is no fallback: without a CUDA device, or if a library cannot be compiled
or loaded, `CudaOps` raises `KernelsUnavailable`.  The only library matrix
product is the bfloat16 `linear`, which goes to cuBLAS through `torch.mm` (the
reference also hands its dense products to cuBLAS:
src/runtime/kernels/cuda_kernels.cu:892-908); the 32-bit `linear` runs this
package's own FMA kernel.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional

import torch

from . import build


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
        self.use_tcgen05 = True    # products of 128 tokens or more on this package's tcgen05 kernel, else cuBLAS
        self.plain_gemm = os.environ.get("LLME_GEMM", "auto")   # "auto" | "tcgen05" | "cublas", see _tc_fills_its_waves
        if self.plain_gemm not in ("auto", "tcgen05", "cublas"):
            raise KernelError(f"LLME_GEMM must be auto, tcgen05 or cublas, got {self.plain_gemm!r}")
        self._sms = None
        self.launches = 0          # kernels of this package launched so far (cuBLAS calls are not counted)

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

    def _lib(self, name: str) -> ctypes.CDLL:
        lib = self._libs.get(name)
        if lib is None:
            self.require(name)
            lib = self._libs[name]
        return lib

    def _check(self, lib: ctypes.CDLL, rc: int, what: str) -> None:
        self.launches += 1
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
        if not (self.use_tcgen05 and dtype == torch.bfloat16 and head_dim in (64, 128)):
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

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[M,N] = x[M,K] @ w[N,K]^T.  32-bit operands: this package's FMA kernel (never a
        reduced-precision mode).  bfloat16 operands: cuBLAS with 32-bit accumulation, the output
        in `out`'s type."""
        M, K = x.shape
        N = w.shape[0]
        assert w.shape[1] == K and out.shape == (M, N)
        if x.dtype == torch.float32:
            lib = self._lib("gemm_f32")
            assert out.dtype == torch.float32 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            rc = lib.llme_gemm_nt_f32(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_int(_code(w.dtype)),
                                      c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
                                      c_longlong(x.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                      self._stream())
            self._check(lib, rc, "gemm_f32")
            return out
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        if M == 0:
            return out
        if self.skinny_supports(x, w, out):
            # a handful of tokens: this package's weight-streaming kernel
            lib = self._lib("gemm_skinny")
            rc = lib.llme_gemm_skinny_bf16(c_void_p(x.data_ptr()), c_longlong(x.stride(0)), c_void_p(w.data_ptr()),
                                           c_longlong(w.stride(0)), c_void_p(out.data_ptr()), c_int(_code(out.dtype)),
                                           c_longlong(out.stride(0)), c_int(M), c_int(N), c_int(K), self._stream())
            self._check(lib, rc, "gemm_skinny")
            return out
        if (self.use_tcgen05 and M >= 128 and K % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
                and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and self._tc_fills_its_waves(M, N)):
            # many tokens: this package's tcgen05 kernel (TMA-fed, accumulator in tensor memory)
            return self.linear_tc(x, w, out)
        if out.dtype == torch.bfloat16:
            # torch lets cuBLAS add partial sums in bfloat16 unless told otherwise, and for some shapes (a few
            # tokens, an odd width) cuBLAS then does: results a thousand rounding steps off.  Not here.
            mm = torch.backends.cuda.matmul
            keep = mm.allow_bf16_reduced_precision_reduction
            mm.allow_bf16_reduced_precision_reduction = False
            try:
                torch.mm(x, w.t(), out=out)
            finally:
                mm.allow_bf16_reduced_precision_reduction = keep
        else:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        return out

    def _tc_fills_its_waves(self, M: int, N: int) -> bool:
        """Whether a plain product of this size goes to this package's tcgen05 kernel rather than to cuBLAS.

        The kernel walks over whole 128 x 256 tiles, one block per SM: 256 tiles on 148 SMs take the time of two
        waves for 1.73 waves of work, and there cuBLAS, which balances such a product, is 10-15 % faster (measured
        for 2,048 tokens: 70/50/136 us against 81/58/158 us for the q|k|v, output and down products of the 8B
        shape).  `plain_gemm` = "tcgen05" or "cublas" (or LLME_GEMM in the environment) forces one of them;
        "auto" takes the kernel when its last wave is at least 90 % full."""
        if self.plain_gemm != "auto":
            return self.plain_gemm == "tcgen05"
        tiles = -(-M // 128) * -(-N // (256 if N > 128 else 128))
        sms = self._sm_count()
        waves = -(-tiles // sms)
        return tiles >= 0.9 * waves * sms

    def _sm_count(self) -> int:
        if self._sms is None:
            self._sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        return self._sms

    def skinny_supports(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
        """Whether the weight-streaming kernel for a handful of tokens takes this product."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= 16 and x.shape[1] % 8 == 0
                and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def _tc_swiglu_supports(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
        # its tile is 128 tokens x (128 gate + 128 up) rows; like the plain product it is taken only when its last
        # wave is nearly full (2,048 tokens of the 8B shape: 289 us against 287 us for cuBLAS and a SwiGLU kernel
        # behind it; 256 / 512 / 1,024 tokens: 83 / 106 / 172 us against 69 / 85 / 150 us)
        return (self.use_tcgen05 and x.dtype == w.dtype == out.dtype == torch.bfloat16 and x.shape[0] >= 128
                and self._tc_fills_its_waves(x.shape[0], 2 * out.shape[1])
                and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
                and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and out.shape[1] >= 8
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)

    def linear_swiglu_supports(self, x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> bool:
        """Whether linear_swiglu() takes this product: a handful of tokens (the weight-streaming kernel) or at
        least 128 of them (the tcgen05 kernel), bfloat16."""
        return self.skinny_supports(x, w_gate_up, out) or self._tc_swiglu_supports(x, w_gate_up, out)

    def linear_swiglu(self, x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[M, I] = silu(x @ Wg^T) * (x @ Wu^T) with w_gate_up = [Wg | Wu] stacked by rows, in one kernel;
        only where linear_swiglu_supports() holds."""
        M, K = x.shape
        inter = out.shape[1]
        assert w_gate_up.shape == (2 * inter, K) and out.shape[0] == M
        if self.skinny_supports(x, w_gate_up, out):
            lib = self._lib("gemm_skinny")
            rc = lib.llme_gemm_skinny_swiglu_bf16(c_void_p(x.data_ptr()), c_longlong(x.stride(0)), c_void_p(w_gate_up.data_ptr()),
                                                  c_longlong(w_gate_up.stride(0)), c_void_p(out.data_ptr()),
                                                  c_int(_code(out.dtype)), c_longlong(out.stride(0)), c_int(M), c_int(inter),
                                                  c_int(K), self._stream())
            self._check(lib, rc, "gemm_skinny_swiglu")
            return out
        assert self._tc_swiglu_supports(x, w_gate_up, out)
        lib = self._lib("gemm_tcgen05")
        rc = lib.llme_gemm_tc_swiglu_bf16(c_void_p(x.data_ptr()), c_longlong(x.stride(0)), c_void_p(w_gate_up.data_ptr()),
                                          c_longlong(w_gate_up.stride(0)), c_void_p(out.data_ptr()), c_longlong(out.stride(0)),
                                          c_int(M), c_int(inter), c_int(K), self._stream())
        self._check(lib, rc, "gemm_tcgen05_swiglu")
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
