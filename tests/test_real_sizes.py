"""Logits at the layer sizes that the benchmark times: two layers of the Qwen3-8B shape (hidden 4096, 32 query
and 8 key/value heads of 128, feed-forward 12288, vocabulary 151936, untied head), in 32-bit and in bfloat16,
under the four ways of cutting requests into steps, with pages of 16 and of 64 tokens, against the plain
implementation (src/model/transformer_graph_builder.cpp:129-294 restated in tests/plain_model.py).

The tiny configurations of the other tests never reach what these sizes take: the two 64-column halves of a
128-wide head in the tcgen05 attention, the 16-byte vector paths of the element-wise kernels, the tcgen05
product on tiles that fill the GPU, a head of 151,936 rows, a weight file of several gigabytes.
"""
import os

import pytest
import torch

from helpers import (compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_mixed,
                     trace_portions, trace_whole)

pytestmark = pytest.mark.gpu

SHAPE_8B_2_LAYERS = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "hidden_act": "silu",
}
LENGTHS = [70, 150, 300]


@pytest.fixture(scope="module")
def real_size_model(tmp_path_factory):
    """The model folder (written once, values computed on the GPU: they are the same on any device), the requests
    and the plain implementation's logits in 32-bit and with bfloat16 rounding, computed once on the CPU."""
    from llmengine_b200.config import config_from_dict
    from llmengine_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    from plain_model import PlainQwen3

    d = str(tmp_path_factory.mktemp("real_sizes") / "model")
    write_random_model(config_from_dict(SHAPE_8B_2_LAYERS), 77, d, dtype="bfloat16", device="cuda:0")
    # sharper attention (QK-norm gains x 2): a key that is skipped or read from a wrong place then shows
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n) for n in f.names()}
    tensors = {n: ((t.float() * 2.0).to(t.dtype) if n.endswith(("q_norm.weight", "k_norm.weight")) else t.clone())
               for n, t in tensors.items()}
    del f
    write_safetensors(path, tensors)
    del tensors
    assert os.path.getsize(path) > 3 << 30
    reqs = {f"r{i}": random_ids(n, SHAPE_8B_2_LAYERS["vocab_size"], 300 + i) for i, n in enumerate(LENGTHS)}
    plain = PlainQwen3(d)
    ref32 = {r: plain.logits(ids) for r, ids in reqs.items()}
    del plain
    rounded = PlainQwen3(d, round_to=torch.bfloat16)
    ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
    del rounded
    return d, reqs, ref32, ref16


def _traces(reqs):
    prompt = {r: max(1, len(ids) - 12) for r, ids in reqs.items()}
    return {
        "whole": trace_whole(reqs),
        "bulk_then_single": trace_bulk_then_single(reqs, 32),
        "portions": trace_portions(reqs, sizes=(48, 7, 2, 130, 1, 33, 2, 5)),
        "mixed": trace_mixed(reqs, prompt, max_live=3, seed=5, sizes=(24, 3, 2, 140, 17, 5)),
    }


def _run(model, dtype, page, products, ref, tol):
    d, reqs, _, _ = model
    traces = _traces(reqs)
    pool = max(max_live_tokens(s, 64) for s in traces.values())
    eng = engine_for(d, dtype, pool, page_size=page)
    eng.ops.plain_gemm = products
    worst = {}
    for what, steps in traces.items():
        got = replay(eng, steps, poison=True)
        worst[what] = compare(got, ref, tol, f"8B sizes/{dtype}/page {page}/{products}/{what}")
        eng.cache.check_invariants()
        assert not eng.cache.requests
    eng.check_kernels()
    print(f"8B layer sizes, {dtype}, pages of {page}, products {products}: max |diff| "
          + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()) + f" (tolerance {tol:.2e})")
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("page", [16, 64])
def test_logits_at_real_layer_sizes_32bit(real_size_model, page):
    _run(real_size_model, "float32", page, "auto", real_size_model[2], 1e-4)


@pytest.mark.parametrize("products", ["auto", "tcgen05"])
@pytest.mark.parametrize("page", [16, 64])
def test_logits_at_real_layer_sizes_bfloat16(real_size_model, page, products):
    """`tcgen05`: every product of 128 tokens or more on this package's own kernel (and the tcgen05 attention with
    its two halves carries every portion); `auto`: the choice that serving makes."""
    from test_replay import bf16_tolerance
    _, _, ref32, ref16 = real_size_model
    _run(real_size_model, "bfloat16", page, products, ref16, bf16_tolerance(ref16, ref32))
