"""Configuration: reading config.json keys, refusing what the engine cannot run, the registry."""
import json

import pytest

from llmengine_b200.config import (ARCHITECTURES, ConfigError, EngineConfig, Qwen3Config, config_from_dict,
                                   find_architecture, load_config)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_the_file():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, Qwen3Config)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps, a.tie_word_embeddings,
            a.max_position_embeddings) == (2, 64, 4, 2, 16, 160, 512, 10000.0, 1e-6, True, 256)
    assert (b.q_size, b.kv_size, b.hidden_size) == (256, 64, 96)        # q width differs from the hidden size
    assert b.rope_theta == 1e6 and b.rms_norm_eps == 1e-5 and not b.tie_word_embeddings


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "rms_norm_eps", "max_position_embeddings", "rope_theta"])
def test_a_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_defaults_that_follow_from_other_keys():
    d = dict(TINY_A)
    del d["head_dim"], d["num_key_value_heads"]
    c = config_from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4
    d = dict(TINY_A)
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 5000.0}
    assert config_from_dict(d).rope_theta == 5000.0


@pytest.mark.parametrize("patch,word", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"vocab_size": 0}, "vocab_size"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}, "layer_types"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_refuses_what_it_cannot_run(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_windows_and_order():
    c = config_from_dict(TINY_C)
    assert c.layer_windows == (0, 21, 0)
    assert c.layer_order == ((0, None), (1, None), (2, None), (1, None), (2, 2))
    d = dict(TINY_B, use_sliding_window=True, sliding_window=32, max_window_layers=1)
    assert config_from_dict(d).layer_windows == (0, 32, 32)
    assert config_from_dict(dict(TINY_B, sliding_window=32)).layer_windows == (0, 0, 0)   # switched off by default
    spec = c.model_spec()
    assert [r.layer for r in spec.order] == [0, 1, 2, 1, 2] and spec.order[4].cache_from == 2
    assert spec.layers[1].mixer.params["window"] == 21
    with pytest.raises(ValueError, match="cache_from"):
        config_from_dict(dict(TINY_A, layer_order=[[0, 0], 1])).model_spec()


def test_round_trip_through_a_file(tmp_path):
    for cfg in (TINY_A, TINY_B, TINY_C):
        c = config_from_dict(cfg)
        with open(tmp_path / "config.json", "w") as f:
            json.dump(c.to_dict(), f)
        assert load_config(str(tmp_path)) == c


def test_registry():
    assert "Qwen3ForCausalLM" in ARCHITECTURES
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):      # the message lists what is registered
        find_architecture("NoSuchModel")
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ConfigError):
        load_config("/nonexistent/folder")


def test_reference_tensor_names_are_translated():
    f = Qwen3Config.canonical_tensor_name
    assert f("layer_3.q_proj.weight") == "model.layers.3.self_attn.q_proj.weight"
    assert f("layer_0.attn_norm.weight") == "model.layers.0.input_layernorm.weight"
    assert f("layer_12.ffn_norm.weight") == "model.layers.12.post_attention_layernorm.weight"
    assert f("blk.7.attn_q_norm.weight") == "model.layers.7.self_attn.q_norm.weight"
    assert f("blk.7.ffn_down.weight") == "model.layers.7.mlp.down_proj.weight"
    assert f("tok_embeddings.weight") == f("token_embd.weight") == "model.embed_tokens.weight"
    assert f("output_norm.weight") == "model.norm.weight" and f("output.weight") == "lm_head.weight"
    assert f("model.layers.1.mlp.up_proj.weight") == "model.layers.1.mlp.up_proj.weight"
    with pytest.raises(ConfigError, match="not a number"):            # src/io/gguf_weight_loader.cpp:388-398
        f("blk.x.attn_q.weight")


def test_engine_config_checks():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16" and EngineConfig(dtype="fp32").dtype == "float32"
    for bad in (dict(dtype="float16"), dict(page_size=0), dict(kernels="quick"), dict(max_num_seqs=0)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)
