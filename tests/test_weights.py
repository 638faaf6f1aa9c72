"""Weights: the safetensors container, loading by name with one error for everything wrong,
stored types, the tied head, the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from helpers import make_model_dir
from host_ops import HostOps
from llmengine_b200.config import EngineConfig, config_from_dict
from llmengine_b200.engine.engine import Engine
from llmengine_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, write_random_model,
                                    write_safetensors)
from tiny_configs import TINY_A, TINY_B


def _engine(d, dtype="float32"):
    return Engine(d, engine_config=EngineConfig(dtype=dtype, max_cached_tokens=64, max_num_seqs=2,
                                                max_num_batched_tokens=64, device="cpu"), ops=HostOps())


def _rewrite(d, edit):
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    edit(tensors)
    write_safetensors(path, tensors)


def test_container_round_trip_and_agreement_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    ours = str(tmp_path / "ours.safetensors")
    write_safetensors(ours, t, {"note": "x"})
    theirs = load_file(ours)                      # their reader accepts our file
    assert all(torch.equal(theirs[k], v) for k, v in t.items())
    save_file(t, str(tmp_path / "theirs.safetensors"))
    f = SafetensorsFile(str(tmp_path / "theirs.safetensors"))   # our reader accepts theirs
    assert sorted(f.names()) == ["a", "b", "c"]
    assert all(torch.equal(f.tensor(k), v) and f.dtype(k) == v.dtype and f.shape(k) == tuple(v.shape) for k, v in t.items())


def test_truncated_and_malformed_files_are_refused_before_any_copy(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.randn(100)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-40])
    with pytest.raises(SafetensorsError, match="offsets"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(tmp_path / "missing.safetensors"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 1)

    def edit(t):
        del t["model.layers.1.self_attn.k_norm.weight"]
        del t["model.layers.2.mlp.up_proj.weight"]
        t["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(16)
        t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(96, 200, dtype=torch.bfloat16)
    _rewrite(d, edit)
    with pytest.raises(WeightError) as e:
        _engine(d)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.self_attn.k_norm.weight" in msg
    assert "model.layers.2.mlp.up_proj.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.self_attn.rotary.inv_freq" in msg
    assert "wrong shapes (1)" in msg and "[96, 200]" in msg and "[96, 224]" in msg


def test_tied_head_is_the_embedding_table(tmp_path):
    d = make_model_dir(str(tmp_path / "a"), TINY_A, 2)
    assert "lm_head.weight" not in SafetensorsFile(os.path.join(d, "model.safetensors")).names()
    eng = _engine(d)
    assert eng.model.head.weight.data_ptr() == eng.model.embedding.table.data_ptr()   # stored once, used twice
    # a tied model saved with a copy of the table under the head's name still loads, and ignores the copy
    _rewrite(d, lambda t: t.__setitem__("lm_head.weight", torch.zeros(512, 64, dtype=torch.bfloat16)))
    eng = _engine(d)
    assert eng.model.head.weight.data_ptr() == eng.model.embedding.table.data_ptr()
    # an untied model without a head is an error
    d = make_model_dir(str(tmp_path / "b"), TINY_B, 2)
    _rewrite(d, lambda t: t.pop("lm_head.weight"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        _engine(d)


def test_stored_types(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 3, dtype="bfloat16")
    _rewrite(d, lambda t: t.__setitem__("model.norm.weight", t["model.norm.weight"].float()))
    e16, e32 = _engine(d, "bfloat16"), _engine(d, "float32")
    blk = e16.model.blocks[0]
    assert blk.mixer.w_qkv.dtype == torch.bfloat16 and blk.ffn.w_down.dtype == torch.bfloat16
    assert blk.mixer_norm.gain.dtype == torch.bfloat16            # stored in 16 bits: kept
    assert e16.model.final_norm.gain.dtype == torch.float32       # stored in 32 bits: stays so
    assert all(p.dtype == torch.float32 for p in (e32.model.blocks[0].mixer.w_qkv, e32.model.blocks[0].mixer_norm.gain,
                                                  e32.model.embedding.table))
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert torch.equal(e32.model.embedding.table, f.tensor("model.embed_tokens.weight").float())   # widened exactly


def test_reference_style_names_load(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 4)
    want = _engine(d).model.blocks[1].mixer.w_o.clone()

    def rename(t):
        for n in list(t):
            if n.startswith("model.layers."):
                _, _, l, rest = n.split(".", 3)
                rest = (rest.replace("self_attn.", "").replace("mlp.", "").replace("input_layernorm", "attn_norm")
                        .replace("post_attention_layernorm", "ffn_norm"))
                t[f"layer_{l}.{rest}"] = t.pop(n)
        t["tok_embeddings.weight"] = t.pop("model.embed_tokens.weight")
        t["output_norm.weight"] = t.pop("model.norm.weight")
    _rewrite(d, rename)
    assert torch.equal(_engine(d).model.blocks[1].mixer.w_o, want)


def test_random_weights_mode(tmp_path):
    c = config_from_dict(TINY_B)
    a = write_random_model(c, 9, str(tmp_path / "a"))
    b = write_random_model(c, 9, str(tmp_path / "b"))
    other = write_random_model(c, 10, str(tmp_path / "c"))
    fa, fb, fo = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, other))
    assert sorted(fa.names()) == sorted(fb.names()) and len(fa.names()) == 3 * 11 + 3
    assert all(torch.equal(fa.tensor(n), fb.tensor(n)) for n in fa.names())          # same seed, same file
    assert not torch.equal(fa.tensor("lm_head.weight"), fo.tensor("lm_head.weight"))
    w = fa.tensor("model.layers.0.mlp.gate_proj.weight").float()
    g = fa.tensor("model.layers.2.input_layernorm.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.001        # ~ N(0, 0.02)
    assert abs(g.mean().item() - 1.0) < 0.05 and 0.05 < g.std().item() < 0.15         # ~ 1 + N(0, 0.1)
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]
    assert fa.dtype("lm_head.weight") == torch.bfloat16
    f32 = SafetensorsFile(os.path.join(write_random_model(c, 9, str(tmp_path / "d"), dtype="float32"), "model.safetensors"))
    assert f32.dtype("lm_head.weight") == torch.float32
    assert torch.equal(f32.tensor("lm_head.weight").to(torch.bfloat16), fa.tensor("lm_head.weight"))
