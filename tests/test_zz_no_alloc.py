"""The decode-attention entry point that allocates nothing (csrc/attention_decode_static.h).

Some users of the kernel library cannot allocate device memory when they call it: a host
application that has handed the whole device to its own arenas and forbids cudaMalloc in the
libraries it loads, or a serving loop that must not stall on an allocation.  For them the
library keeps the scratch memory of the split-context decode attention in a device array of
its own.  This test calls that entry point through its exported C symbol, several times in a row on
different inputs, and checks each output against the regular entry point's, which works on a
scratch buffer that the caller allocates.  The first calls split each context over more blocks
than one thread-block cluster holds, so the blocks' partial results and their ticket counters
really pass through the built-in array, and the second call finds there what the first one left
(partials of another batch shape; counters that must be back at zero).  A last call uses few
splits, which merge inside a cluster and leave the array alone.  It also checks that a call that
would not fit the array is refused.

This file sorts last on purpose: a run that stops at the first failure has by then run every
other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, ctx_lens, nh, nkv, hd, page):
    from test_gpu_kernels import _attention_case
    return _attention_case(nh, nkv, hd, page, ctx_lens, [1] * len(ctx_lens), 0, torch.bfloat16, seed)


def test_static_scratch_entry_point_matches_the_regular_one():
    from llmengine_b200.kernels import build
    from llmengine_b200.kernels.ops import CudaOps, _FastAttnArgs

    nh, nkv, hd, page = 8, 2, 128, 16
    ops = CudaOps(torch.device(DEV))
    path = build.ensure_built([f"attention_decode_static@HEAD_DIM={hd}"])[f"attention_decode_static@HEAD_DIM={hd}"]
    lib = ctypes.CDLL(path)
    lib.llme_last_error.restype = ctypes.c_char_p
    lib.llme_attention_decode_static_capacity.restype = ctypes.c_longlong
    capacity = lib.llme_attention_decode_static_capacity()
    assert capacity == 1 << 20
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # more than 8 splits: merged through scratch memory by the block that finishes last; 5: inside a cluster
    for seed, ctx_lens, splits in ((40, [700, 64, 5, 333], 12), (41, [129, 1000, 65], 16), (43, [900, 2, 257], 5)):
        case = _case(seed, ctx_lens, nh, nkv, hd, page)
        rows = torch.arange(len(ctx_lens), dtype=torch.int32, device=DEV)
        common = dict(q=case["q"], cache=case["cache"], rows=rows, cu_q_lens=case["cu_q_lens"],
                      ctx_lens=case["ctx_lens"], table_rows=case["table_rows"], block_tables=case["block_tables"],
                      num_heads=nh, num_kv_heads=nkv, head_dim=hd, page_size=page, window=0, scale=1 / math.sqrt(hd))
        # the regular entry point, scratch allocated by the caller
        want = torch.full_like(case["q"], float("nan"))
        need = ops.attention_decode_scratch_floats(hd, len(ctx_lens), nh, splits)
        assert 0 < need <= capacity
        ops.attention_decode(out=want, splits=splits, scratch=torch.zeros(need, device=DEV), **common)
        # the entry point with built-in scratch: inputs and outputs only
        got = torch.full_like(case["q"], float("nan"))
        args = _FastAttnArgs(case["q"].data_ptr(), case["cache"].data_ptr(), got.data_ptr(), rows.data_ptr(),
                             case["cu_q_lens"].data_ptr(), case["ctx_lens"].data_ptr(), case["table_rows"].data_ptr(),
                             case["block_tables"].data_ptr(), None, case["block_tables"].shape[1], len(ctx_lens), nh,
                             nkv, page, 0, splits, 1 / math.sqrt(hd))
        rc = lib.llme_attention_decode_static(ctypes.byref(args), stream)
        assert rc == 0, lib.llme_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert (got.float() - want.float()).abs().max().item() < 2e-2          # the tolerance of the kernel tests
        assert torch.equal(got, want), "same kernels, same inputs: the results should be identical"
        assert (got.cpu().float() - case["want"]).abs().max() < 2e-2           # and right, against the plain reference

    # a call that needs more than the array holds is refused, with a message, and launches nothing
    case = _case(42, [70] * 64, 128, 2, hd, page)
    rows = torch.arange(64, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(case["q"])
    big = _FastAttnArgs(case["q"].data_ptr(), case["cache"].data_ptr(), out.data_ptr(), rows.data_ptr(),
                        case["cu_q_lens"].data_ptr(), case["ctx_lens"].data_ptr(), case["table_rows"].data_ptr(),
                        case["block_tables"].data_ptr(), None, case["block_tables"].shape[1], 64, 128, 2, page, 0, 2,
                        1 / math.sqrt(hd))
    assert 65536 + 64 * 128 * 2 * (hd + 2) > capacity
    rc = lib.llme_attention_decode_static(ctypes.byref(big), stream)
    assert rc == -1
    assert "scratch values" in lib.llme_last_error().decode()
    torch.cuda.synchronize()
    assert out.abs().max() == 0
