"""The plain implementation against logits that the reference's own CPU executor produced
(tests/golden/, made by tests/golden/make_golden.py), and each of its part functions against
hand-checkable facts."""
import math
import os
import sys

import numpy as np
import pytest
import torch

import plain_model as pm
from llmengine_b200.weights import write_safetensors

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from golden_model import GOLDEN_CONFIGS, golden_tokens, golden_weights  # noqa: E402


def _golden_dir(tmp_path, name, seed):
    import json
    cfg = dict(GOLDEN_CONFIGS[name])
    cfg.pop("tokens")
    d = tmp_path / name
    d.mkdir()
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(d / "model.safetensors"), {k: torch.from_numpy(v) for k, v in golden_weights(GOLDEN_CONFIGS[name], seed).items()})
    return str(d)


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_model_matches_the_reference_cpu_executor(tmp_path, name):
    g = np.load(os.path.join(HERE, "golden", f"tiny_{name}.npz"))
    seed = int(g["seed"])
    assert (golden_tokens(GOLDEN_CONFIGS[name], seed) == g["tokens"]).all()
    assert float(g["whole_vs_portions"]) < 1e-6          # the reference agrees with itself across its paged path
    model = pm.PlainQwen3(_golden_dir(tmp_path, name, seed))
    got = model.logits(g["tokens"].tolist())
    want = torch.from_numpy(g["logits"])
    assert got.shape == want.shape
    assert (got - want).abs().max().item() < 5e-6
    assert (got.argmax(-1) == want.argmax(-1)).all()


def test_embedding_rejects_ids_outside_the_table():
    table = torch.randn(10, 4)
    assert torch.equal(pm.embedding(table, [3, 9]), table[[3, 9]])
    with pytest.raises(IndexError):
        pm.embedding(table, [10])


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]])
    g = torch.tensor([2.0, 0.5])
    want = x / math.sqrt((9 + 16) / 2 + 1e-3) * g
    assert torch.allclose(pm.rms_norm(x, g, 1e-3), want, atol=1e-7)


def test_rope_rotates_half_pairs():
    hd = 8
    x = torch.arange(hd, dtype=torch.float32).view(1, 1, hd) + 1
    assert torch.allclose(pm.rope(x, torch.tensor([0]), 10000.0), x)              # position 0: identity
    y = pm.rope(x, torch.tensor([5]), 100.0)[0, 0]
    for d in range(hd // 2):
        a = 5 * 100.0 ** (-2 * d / hd)
        assert abs(y[d] - (x[0, 0, d] * math.cos(a) - x[0, 0, d + 4] * math.sin(a))) < 1e-5
        assert abs(y[d + 4] - (x[0, 0, d] * math.sin(a) + x[0, 0, d + 4] * math.cos(a))) < 1e-5
    assert torch.allclose(y.norm(), x.norm(), atol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nh, nkv, hd = 9, 4, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    out = pm.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 7.0, -3.0
    assert torch.allclose(pm.attention(q, k2, v2)[:5], out[:5])                         # later keys never matter
    s = (k[:4, 0] @ q[3, 1]) / math.sqrt(hd)
    assert torch.allclose(out[3, 1], torch.softmax(s, 0) @ v[:4, 0], atol=1e-6)         # heads 0,1 share kv head 0
    w = pm.attention(q, k, v, window=3)
    s = (k[4:7, 1] @ q[6, 2]) / math.sqrt(hd)
    assert torch.allclose(w[6, 2], torch.softmax(s, 0) @ v[4:7, 1], atol=1e-6)          # keys 4, 5, 6 only


def test_swiglu_formula():
    g, u = torch.tensor([0.0, 2.0, -1.0]), torch.tensor([5.0, 3.0, 2.0])
    want = torch.tensor([0.0, 2 / (1 + math.exp(-2)) * 3, -1 / (1 + math.exp(1)) * 2])
    assert torch.allclose(pm.swiglu(g, u), want, atol=1e-6)


def test_plain_sample_follows_the_reference_order():
    z = torch.tensor([1.0, 3.0, 2.0, -1.0])
    assert pm.plain_sample(z) == 1
    assert pm.plain_sample(torch.full((5,), float("-inf"))) == 0                        # src/runtime/sampler.cpp:41-47
    assert pm.plain_sample(z, repetition_penalty=4.0, history=[1]) == 2                  # 3/4 < 2
    assert pm.plain_sample(torch.tensor([-1.0, -3.0]), repetition_penalty=4.0, history=[0]) == 1   # -1*4 < -3
    p = torch.softmax(z, 0)
    assert pm.plain_sample(z, greedy=False, u=float(p[0]) - 1e-4) == 0
    assert pm.plain_sample(z, greedy=False, u=float(p[0]) + 1e-4) == 1
    assert pm.plain_sample(z, greedy=False, top_k=1, u=0.99) == 1
    assert pm.plain_sample(z, greedy=False, top_p=0.6, u=0.99) == 1                      # p[1] = 0.64 alone reaches 0.6
    assert pm.plain_sample(z, greedy=False, top_p=0.7, u=0.99) == 2                      # needs tokens 1 and 2
