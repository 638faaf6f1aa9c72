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


def test_random_values_depend_on_seed_name_and_element_only():
    """Counter-based: any slice of a tensor's stream can be made alone, the engine's on-device weights are the
    file's tensors bit for bit, and nothing depends on the order in which tensors are made."""
    from llmengine_b200.parts import WeightSpec
    from llmengine_b200.weights.loader import _tensor_seed, counter_normal, random_tensor
    whole = random_tensor("x.weight", WeightSpec((37, 11)), 5).reshape(-1)
    piece = 0.02 * counter_normal(_tensor_seed(5, "x.weight"), 100, 60, torch.device("cpu"))
    assert torch.equal(whole[100:160], piece)
    assert not torch.equal(random_tensor("y.weight", WeightSpec((37, 11)), 5).reshape(-1), whole)
    z = counter_normal(1, 0, 1 << 16, torch.device("cpu"))
    assert abs(z.mean().item()) < 0.02 and abs(z.std().item() - 1.0) < 0.02 and z.abs().max().item() <= 6.0


def test_engine_random_weights_equal_the_written_folder(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 12)
    from_file = _engine(d, "bfloat16")
    ec = EngineConfig(dtype="bfloat16", max_cached_tokens=64, max_num_seqs=2, max_num_batched_tokens=64, device="cpu")
    from_seed = Engine(config=TINY_B, random_seed=12, engine_config=ec, ops=HostOps())
    for a, b in zip(from_file.model.blocks, from_seed.model.blocks):
        assert torch.equal(a.mixer.w_qkv, b.mixer.w_qkv) and torch.equal(a.ffn.w_down, b.ffn.w_down)
        assert torch.equal(a.mixer_norm.gain, b.mixer_norm.gain)
    assert torch.equal(from_file.model.head.weight, from_seed.model.head.weight)


def test_a_sharded_folder_loads_like_a_single_file(tmp_path):
    """Large checkpoints come as model-0000i-of-0000n.safetensors with an index; the shards are found through it."""
    c = config_from_dict(TINY_B)
    one = write_random_model(c, 9, str(tmp_path / "one"))
    many = write_random_model(c, 9, str(tmp_path / "many"), shard_bytes=60_000)
    files = sorted(os.listdir(many))
    shards = [f for f in files if f.endswith(".safetensors")]
    assert "model.safetensors" not in files and "model.safetensors.index.json" in files and len(shards) >= 3
    index = json.load(open(os.path.join(many, "model.safetensors.index.json")))
    assert set(index["weight_map"].values()) == set(shards)
    a, b = _engine(one), _engine(many)
    for x, y in zip(a.model.blocks, b.model.blocks):
        assert torch.equal(x.mixer.w_qkv, y.mixer.w_qkv) and torch.equal(x.ffn.w_gate_up, y.ffn.w_gate_up)
    assert torch.equal(a.model.head.weight, b.model.head.weight)
    # a tensor that a shard lacks is reported like any missing tensor
    victim = index["weight_map"]["model.layers.1.mlp.down_proj.weight"]
    path = os.path.join(many, victim)
    f = SafetensorsFile(path)
    kept = {n: f.tensor(n).clone() for n in f.names() if n != "model.layers.1.mlp.down_proj.weight"}
    del f
    write_safetensors(path, kept)
    with pytest.raises(WeightError, match="model.layers.1.mlp.down_proj.weight"):
        _engine(many)
    # the same tensor in two shards is refused
    other = next(s for s in shards if s != victim)
    f = SafetensorsFile(os.path.join(many, other))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del f
    dup = next(iter(kept))
    t[dup] = kept[dup]
    write_safetensors(os.path.join(many, other), t)
    with pytest.raises(WeightError, match="twice"):
        _engine(many)


def test_a_float16_file_loads(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), TINY_A, 3, dtype="float32")
    want = _engine(d, "float32")
    _rewrite(d, lambda t: [t.__setitem__(n, v.to(torch.float16)) for n, v in list(t.items())])
    assert SafetensorsFile(os.path.join(d, "model.safetensors")).dtype("model.norm.weight") == torch.float16
    e32, e16 = _engine(d, "float32"), _engine(d, "bfloat16")
    w = want.model.blocks[0].ffn.w_down
    assert e32.model.blocks[0].ffn.w_down.dtype == torch.float32
    assert torch.equal(e32.model.blocks[0].ffn.w_down, w.to(torch.float16).float())               # widened exactly
    assert e16.model.blocks[0].ffn.w_down.dtype == torch.bfloat16                                 # matrices: the compute type
    assert e16.model.final_norm.gain.dtype == torch.float32                                       # 16-bit float vectors are widened
    assert torch.equal(e16.model.final_norm.gain, want.model.final_norm.gain.to(torch.float16).float())


def test_make_random_model_command(tmp_path):
    from llmengine_b200 import make_random_model
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY_A))
    assert make_random_model.main([str(cfg), str(tmp_path / "out"), "--seed", "9"]) == 0
    ref = write_random_model(config_from_dict(TINY_A), 9, str(tmp_path / "ref"))
    a = SafetensorsFile(str(tmp_path / "out" / "model.safetensors"))
    b = SafetensorsFile(os.path.join(ref, "model.safetensors"))
    assert all(torch.equal(a.tensor(n), b.tensor(n)) for n in b.names())
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"architectures": ["NoSuchModel"]}))
    assert make_random_model.main([str(bad), str(tmp_path / "x")]) == 2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_random_weights_made_on_the_gpu_equal_the_written_folder(tmp_path, dtype):
    """The device generator (one kernel launch per tensor) restates the host generator bit for bit."""
    d = make_model_dir(str(tmp_path / "m"), TINY_B, 12)
    ec = EngineConfig(dtype=dtype, max_cached_tokens=64, max_num_seqs=2, max_num_batched_tokens=64)
    from_file = Engine(d, engine_config=ec)
    from_seed = Engine(config=TINY_B, random_seed=12, engine_config=ec)
    assert from_seed.ops.launches > 0
    for a, b in zip(from_file.model.blocks, from_seed.model.blocks):
        for x, y in ((a.mixer.w_qkv, b.mixer.w_qkv), (a.mixer.w_o, b.mixer.w_o), (a.ffn.w_gate_up, b.ffn.w_gate_up),
                     (a.ffn.w_down, b.ffn.w_down), (a.mixer_norm.gain, b.mixer_norm.gain), (a.mixer.q_gain, b.mixer.q_gain)):
            assert x.dtype == y.dtype and torch.equal(x, y)
    assert torch.equal(from_file.model.head.weight, from_seed.model.head.weight)
    assert torch.equal(from_file.model.embedding.table, from_seed.model.embedding.table)
