"""Python face of the native step executor (include/llmengine_b200/executor.h): the ctypes mirror of its records
and the compilation of a `Plan` (engine/plan.py) into them."""
from __future__ import annotations

import ctypes
from ctypes import CFUNCTYPE, POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from typing import Any, Callable, Dict, List, Optional

import torch

MAX_GROUPS = 8
F32, BF16 = 0, 1
ROWS = {"tokens": 0, "logits": 1}
(OP_EMBEDDING, OP_RMSNORM, OP_LINEAR, OP_LINEAR_SWIGLU, OP_QKV_POST, OP_ATTEND, OP_ATTENTION, OP_CALL) = range(1, 9)


def code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class StepGroup(Structure):
    _fields_ = [("block_tables", c_void_p), ("slot_mapping", c_void_p), ("max_blocks", c_int), ("page_size", c_int),
                ("window", c_int)]


class Step(Structure):
    _fields_ = [
        ("num_tokens", c_int), ("num_requests", c_int), ("num_logit_rows", c_int), ("num_decode", c_int),
        ("num_portion", c_int), ("max_portion_len", c_int), ("max_decode_ctx", c_int),
        ("token_ids", c_void_p), ("positions", c_void_p), ("token_request", c_void_p), ("cu_q_lens", c_void_p),
        ("ctx_lens", c_void_p), ("state_slots", c_void_p), ("first_portion", c_void_p), ("logit_rows", c_void_p),
        ("decode_rows", c_void_p), ("portion_rows", c_void_p), ("logits", c_void_p), ("blas", c_void_p),
        ("num_groups", c_int), ("groups", StepGroup * MAX_GROUPS),
    ]


CallFn = CFUNCTYPE(c_int, c_void_p, POINTER(Step), c_void_p)


class EmbeddingOp(Structure):
    _fields_ = [("table", c_void_p), ("table_dtype", c_int), ("vocab", c_int), ("hidden", c_int), ("out", c_void_p)]


class RmsNormOp(Structure):
    _fields_ = [("x", c_void_p), ("delta", c_void_p), ("delta_dtype", c_int), ("gain", c_void_p), ("gain_dtype", c_int),
                ("out", c_void_p), ("out_dtype", c_int), ("size", c_int), ("eps", c_float), ("rows", c_int)]


class LinearOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("x_dtype", c_int), ("w", c_void_p), ("ldw", c_longlong),
                ("w_dtype", c_int), ("out", c_void_p), ("ldo", c_longlong), ("out_dtype", c_int), ("n", c_int), ("k", c_int),
                ("rows", c_int)]


class LinearSwigluOp(Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("dtype", c_int), ("w_gate_up", c_void_p), ("ldw", c_longlong),
                ("gate_up", c_void_p), ("out", c_void_p), ("ldo", c_longlong), ("inter", c_int), ("k", c_int)]


class QkvPostOp(Structure):
    _fields_ = [("q_in", c_void_p), ("k_in", c_void_p), ("v_in", c_void_p), ("q_stride", c_longlong), ("k_stride", c_longlong),
                ("v_stride", c_longlong), ("in_dtype", c_int), ("q_gain", c_void_p), ("k_gain", c_void_p), ("gain_dtype", c_int),
                ("eps", c_float), ("cos_sin", c_void_p), ("max_positions", c_int), ("q_out", c_void_p), ("k_out", c_void_p),
                ("out_dtype", c_int), ("cache", c_void_p), ("group", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int)]


class AttendOp(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("dtype", c_int), ("cache", c_void_p), ("cache_rows", c_longlong),
                ("group", c_int), ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("window", c_int), ("scale", c_float),
                ("scratch", c_void_p), ("scratch_floats", c_longlong)]


class AttentionOp(Structure):
    _fields_ = [("post", QkvPostOp), ("attend", AttendOp), ("qkv", c_void_p), ("qkv_stride", c_longlong), ("rotary", c_int)]


class CallOp(Structure):
    _fields_ = [("fn", CallFn), ("user", c_void_p)]


def declare(lib: ctypes.CDLL) -> None:
    lib.llme_executor_create.restype = c_void_p
    lib.llme_executor_create.argtypes = [c_int]
    lib.llme_executor_destroy.argtypes = [c_void_p]
    lib.llme_executor_register.argtypes = [c_void_p, c_char_p, c_void_p]
    lib.llme_executor_choose.argtypes = [c_void_p, c_char_p, c_char_p]
    lib.llme_executor_chosen.restype = c_char_p
    lib.llme_executor_chosen.argtypes = [c_void_p, c_char_p]
    lib.llme_executor_error.restype = c_char_p
    lib.llme_executor_error.argtypes = [c_void_p]
    lib.llme_executor_launches.restype = c_longlong
    lib.llme_executor_launches.argtypes = [c_void_p]
    lib.llme_attention_scratch_floats.restype = c_longlong
    lib.llme_attention_scratch_floats.argtypes = [c_void_p, c_int, c_int, c_int, c_int]
    lib.llme_decode_splits.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int]
    lib.llme_plan_create.restype = c_void_p
    lib.llme_plan_create.argtypes = [c_void_p]
    lib.llme_plan_destroy.argtypes = [c_void_p]
    lib.llme_plan_add.argtypes = [c_void_p, c_int, c_void_p, c_size_t]
    lib.llme_plan_size.argtypes = [c_void_p]
    lib.llme_plan_run.argtypes = [c_void_p, POINTER(Step), c_int, c_int, c_void_p]


def _qkv_post_record(a: Dict[str, Any]) -> QkvPostOp:
    q_in, k_in, v_in = a.get("q_in"), a.get("k_in"), a.get("v_in")
    ref = q_in if q_in is not None else (k_in if k_in is not None else v_in)
    outs = [t for t in (a.get("q_out"), a.get("k_out"), a.get("cache")) if t is not None]
    if ref is None or not outs:
        raise ValueError("qkv_post: nothing to read or nothing to write")
    for t in (q_in, k_in, v_in):
        assert t is None or (t.dtype == ref.dtype and t.stride(-1) == 1)
    assert all(t.dtype == outs[0].dtype for t in outs)
    gains = [g for g in (a.get("q_gain"), a.get("k_gain")) if g is not None]
    assert all(g.dtype == gains[0].dtype for g in gains)
    cs = a.get("cos_sin")
    return QkvPostOp(ptr(q_in), ptr(k_in), ptr(v_in), q_in.stride(0) if q_in is not None else 0,
                     k_in.stride(0) if k_in is not None else 0, v_in.stride(0) if v_in is not None else 0, code(ref.dtype),
                     ptr(a.get("q_gain")), ptr(a.get("k_gain")), code(gains[0].dtype) if gains else 0, a.get("eps", 0.0),
                     ptr(cs), cs.shape[0] if cs is not None else 0, ptr(a.get("q_out")), ptr(a.get("k_out")),
                     code(outs[0].dtype), ptr(a.get("cache")), a.get("group") or 0, a["num_heads"], a["num_kv_heads"],
                     a["head_dim"])


def _attend_record(a: Dict[str, Any]) -> AttendOp:
    q, out, cache = a["q"], a["out"], a["cache"]
    assert q.dtype == cache.dtype == out.dtype and q.is_contiguous() and out.is_contiguous() and cache.is_contiguous()
    scratch = a.get("scratch")
    rows = 1
    for d in cache.shape[:-1]:
        rows *= int(d)
    return AttendOp(q.data_ptr(), out.data_ptr(), code(q.dtype), cache.data_ptr(), rows, a["group"], a["num_heads"],
                    a["num_kv_heads"], a["head_dim"], a["window"], a["scale"], ptr(scratch),
                    scratch.numel() if scratch is not None else 0)


def records(op, keep: List[Any]):
    """(kind, ctypes record) of one plan operation; `keep` collects what must stay alive with the plan."""
    a = op.a
    keep.extend(v for v in a.values() if isinstance(v, torch.Tensor))
    k = op.kind
    if k == "embedding":
        t, out = a["table"], a["out"]
        assert out.dtype == torch.float32 and t.is_contiguous() and out.is_contiguous()
        return OP_EMBEDDING, EmbeddingOp(t.data_ptr(), code(t.dtype), t.shape[0], t.shape[1], out.data_ptr())
    if k == "rmsnorm":
        x, d, g, out = a["x"], a["delta"], a["gain"], a["out"]
        assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and (d is None or d.is_contiguous())
        return OP_RMSNORM, RmsNormOp(x.data_ptr(), ptr(d), code(d.dtype) if d is not None else 0, g.data_ptr(), code(g.dtype),
                                     out.data_ptr(), code(out.dtype), x.shape[1], a["eps"], ROWS[a["rows"]])
    if k == "linear":
        x, w, out = a["x"], a["w"], a["out"]
        assert x.stride(1) == 1 and w.stride(1) == 1 and w.shape[1] == x.shape[1] and (out is None or out.stride(1) == 1)
        assert out is None or out.shape[1] == w.shape[0]
        return OP_LINEAR, LinearOp(x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), w.stride(0), code(w.dtype), ptr(out),
                                   out.stride(0) if out is not None else 0, code(out.dtype) if out is not None else F32,
                                   w.shape[0], w.shape[1], ROWS[a["rows"]])
    if k == "linear_swiglu":
        x, w, gu, out = a["x"], a["w_gate_up"], a["gate_up"], a["out"]
        assert x.dtype == w.dtype == out.dtype and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
        assert w.shape[0] == 2 * out.shape[1] and w.shape[1] == x.shape[1]
        return OP_LINEAR_SWIGLU, LinearSwigluOp(x.data_ptr(), x.stride(0), code(x.dtype), w.data_ptr(), w.stride(0), ptr(gu),
                                                out.data_ptr(), out.stride(0), out.shape[1], x.shape[1])
    if k == "qkv_post":
        return OP_QKV_POST, _qkv_post_record(a)
    if k == "attend":
        return OP_ATTEND, _attend_record(a)
    if k == "attention":
        qkv, nh, nkv, hd = a["qkv"], a["num_heads"], a["num_kv_heads"], a["head_dim"]
        qs, kvs = nh * hd, nkv * hd
        writes = a["writes"]
        assert qkv.stride(1) == 1 and qkv.shape[1] == (qs + 2 * kvs if writes else qs)
        post = _qkv_post_record(dict(q_in=qkv[:, :qs], k_in=qkv[:, qs:qs + kvs] if writes else None,
                                     v_in=qkv[:, qs + kvs:] if writes else None, q_gain=a.get("q_gain"), k_gain=a.get("k_gain"),
                                     eps=a.get("eps", 0.0), cos_sin=a.get("cos_sin"), q_out=a["q"],
                                     cache=a["cache"] if writes else None, group=a["group"], num_heads=nh, num_kv_heads=nkv,
                                     head_dim=hd))
        return OP_ATTENTION, AttentionOp(post, _attend_record(a), qkv.data_ptr(), qkv.stride(0),
                                         1 if a.get("cos_sin") is not None else 0)
    raise ValueError(f"the executor has no record for the operation {k!r}")
