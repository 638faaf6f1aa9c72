"""The tiny random models and token ids that the golden logits were made from.

Weights come from an integer hash of (seed, tensor name, element index) turned into normal
variates, so that the script that made the golden files and the test that checks them build
bit-identical models on any machine and library version."""
import numpy as np

GOLDEN_CONFIGS = {
    "A": {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
          "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 160,
          "vocab_size": 512, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
          "max_position_embeddings": 256, "hidden_act": "silu", "tokens": 33},
    "B": {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96,
          "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 224,
          "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
          "max_position_embeddings": 512, "hidden_act": "silu", "tokens": 70},
}


def _mix(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint64)
    with np.errstate(over="ignore"):
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        x = x ^ (x >> np.uint64(31))
    return x


def _normal(key: int, n: int) -> np.ndarray:
    """n standard normal variates from an integer key (Box-Muller on hashed uniforms, 64-bit)."""
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = _mix(idx * np.uint64(2) + np.uint64(key) * np.uint64(0x9E3779B97F4A7C15))
        b = _mix(idx * np.uint64(2) + np.uint64(1) + np.uint64(key) * np.uint64(0x9E3779B97F4A7C15))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 0.5) / 2.0 ** 53
    u2 = ((b >> np.uint64(11)).astype(np.float64) + 0.5) / 2.0 ** 53
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def _key(seed: int, name: str) -> int:
    h = seed & 0xFFFFFFFF
    for ch in name.encode():
        h = (h * 1000003 + ch) & 0xFFFFFFFFFFFF
    return h


def golden_weights(cfg: dict, seed: int) -> dict:
    """Checkpoint-named float32 tensors: matrices ~ N(0, 0.02), norm gains ~ 1 + N(0, 0.1)."""
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nh, nkv, hd, I, V = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    out = {}

    def mat(name, n, k):
        out[name] = (0.02 * _normal(_key(seed, name), n * k)).astype(np.float32).reshape(n, k)

    def gain(name, n):
        out[name] = (1.0 + 0.1 * _normal(_key(seed, name), n)).astype(np.float32)

    mat("model.embed_tokens.weight", V, H)
    for l in range(L):
        p = f"model.layers.{l}."
        gain(p + "input_layernorm.weight", H)
        mat(p + "self_attn.q_proj.weight", nh * hd, H)
        mat(p + "self_attn.k_proj.weight", nkv * hd, H)
        mat(p + "self_attn.v_proj.weight", nkv * hd, H)
        mat(p + "self_attn.o_proj.weight", H, nh * hd)
        gain(p + "self_attn.q_norm.weight", hd)
        gain(p + "self_attn.k_norm.weight", hd)
        gain(p + "post_attention_layernorm.weight", H)
        mat(p + "mlp.gate_proj.weight", I, H)
        mat(p + "mlp.up_proj.weight", I, H)
        mat(p + "mlp.down_proj.weight", H, I)
    gain("model.norm.weight", H)
    if not cfg["tie_word_embeddings"]:
        mat("lm_head.weight", V, H)
    return out


def golden_tokens(cfg: dict, seed: int) -> np.ndarray:
    n = cfg["tokens"]
    return (_mix(np.arange(n, dtype=np.uint64) + np.uint64(seed * 7919 + 13)) % np.uint64(cfg["vocab_size"])).astype(np.int32)
