"""Typed configuration of the Qwen3 dense architecture, read from config.json.

The reference keeps the same numbers in `TransformerConfig`
(include/minillm/model/transformer_graph_builder.h:15-30) and fills them from
GGUF metadata (src/io/gguf_weight_loader.cpp:279-354).  Here they come from the
architecture's config.json keys; every size and constant used by the model is
read from the file, and a missing key is an error that names the key.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


class ConfigError(ValueError):
    """config.json is missing a key or holds a value this engine refuses."""


_REQUIRED = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "rms_norm_eps", "max_position_embeddings",
)


def _positive_int(d: Mapping[str, Any], key: str) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config key '{key}' must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    # Per layer: 0 = all earlier keys, W > 0 = only the last W keys (the query's own included).
    layer_windows: Tuple[int, ...]
    # Execution order: (layer index, index in the order of the run whose cache is read, or None).
    layer_order: Tuple[Tuple[int, Optional[int]], ...]
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    ARCHITECTURE = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        archs = d.get("architectures") or [cls.ARCHITECTURE]
        hidden = _positive_int(d, "hidden_size")
        nh = _positive_int(d, "num_attention_heads")
        nkv = _positive_int(d, "num_key_value_heads") if d.get("num_key_value_heads") is not None else nh
        if d.get("head_dim") is not None:
            hd = _positive_int(d, "head_dim")
        else:
            if hidden % nh:
                raise ConfigError("config has no 'head_dim' and hidden_size is not a multiple of num_attention_heads")
            hd = hidden // nh
        if nh % nkv:
            # The reference refuses this at run time (src/runtime/kernels/cpu_kernel_adapter.cpp:448-451).
            raise ConfigError(f"num_attention_heads={nh} must be a multiple of num_key_value_heads={nkv}")
        if hd % 2:
            # Rotate-half pairs (d, d + head_dim/2) need an even head size (src/runtime/kernels/cuda_kernels.cu:1080-1081).
            raise ConfigError(f"head_dim={hd} must be even for rotary position encoding")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported: the feed-forward gate is SiLU")
        if d.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: the projections have no bias")
        theta = cls._rope_theta(d)
        layers = _positive_int(d, "num_hidden_layers")
        windows = cls._windows(d, layers)
        order = cls._order(d, layers)
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        eps = float(d["rms_norm_eps"])
        if not eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {eps!r}")
        return cls(
            architecture=str(archs[0]),
            vocab_size=_positive_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(d, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=hd,
            rms_norm_eps=eps,
            rope_theta=theta,
            max_position_embeddings=_positive_int(d, "max_position_embeddings"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            layer_windows=windows,
            layer_order=order,
            eos_token_id=eos,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )

    @staticmethod
    def _rope_theta(d: Mapping[str, Any]) -> float:
        scaling = d.get("rope_scaling")
        params = d.get("rope_parameters")
        for name, block in (("rope_scaling", scaling), ("rope_parameters", params)):
            if block:
                kind = block.get("rope_type", block.get("type", "default"))
                if kind != "default":
                    raise ConfigError(f"{name} of type {kind!r} is not supported: only plain rotary encoding")
        if "rope_theta" in d:
            theta = float(d["rope_theta"])
        elif params and "rope_theta" in params:
            theta = float(params["rope_theta"])
        else:
            raise ConfigError("config.json lacks required key(s): rope_theta")
        if not theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {theta!r}")
        return theta

    @staticmethod
    def _windows(d: Mapping[str, Any], layers: int) -> Tuple[int, ...]:
        """Which layers see only a window of keys.

        With `use_sliding_window` off (the default) every layer sees all keys.
        With it on, `layer_types` names each layer "full_attention" or
        "sliding_attention"; without that list, layers from `max_window_layers`
        on are windowed.
        """
        if not d.get("use_sliding_window", False):
            return tuple(0 for _ in range(layers))
        window = d.get("sliding_window")
        if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
            raise ConfigError("use_sliding_window=true needs a positive integer 'sliding_window'")
        types = d.get("layer_types")
        if types is None:
            first = int(d.get("max_window_layers", layers))
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(layers)]
        if len(types) != layers:
            raise ConfigError(f"layer_types has {len(types)} entries for {layers} layers")
        out: List[int] = []
        for i, t in enumerate(types):
            if t == "full_attention":
                out.append(0)
            elif t == "sliding_attention":
                out.append(window)
            else:
                raise ConfigError(f"layer_types[{i}]={t!r} is neither 'full_attention' nor 'sliding_attention'")
        return tuple(out)

    @staticmethod
    def _order(d: Mapping[str, Any], layers: int) -> Tuple[Tuple[int, Optional[int]], ...]:
        """Optional key `layer_order`: a list whose entries are a layer index or
        `[layer index, position in this list whose cache is read]`.  Without it
        the layers run once each, first to last."""
        raw = d.get("layer_order")
        if raw is None:
            return tuple((i, None) for i in range(layers))
        out: List[Tuple[int, Optional[int]]] = []
        for e in raw:
            if isinstance(e, int):
                out.append((e, None))
            elif isinstance(e, (list, tuple)) and len(e) == 2:
                out.append((int(e[0]), None if e[1] is None else int(e[1])))
            else:
                raise ConfigError(f"layer_order entry {e!r} must be an index or a [layer, cache_from] pair")
        return tuple(out)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "attention_bias": False,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
        }
        if any(self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = max(self.layer_windows)
            d["layer_types"] = ["sliding_attention" if w else "full_attention" for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
        if self.layer_order != tuple((i, None) for i in range(self.num_hidden_layers)):
            d["layer_order"] = [l if c is None else [l, c] for l, c in self.layer_order]
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def model_spec(self) -> ModelSpec:
        """The layer list of src/model/transformer_graph_builder.cpp:129-294 with
        `use_qk_norm` on, expressed as parts with their constants."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope", {"head_dim": self.head_dim, "theta": self.rope_theta,
                                 "max_positions": self.max_position_embeddings})
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qk_norm_eps": self.rms_norm_eps,
                "window": self.layer_windows[i],
                "position_encoding": rope,
            })
            ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                      "intermediate_size": self.intermediate_size})
            layers.append(LayerSpec(
                prefix=f"model.layers.{i}",
                block=PartSpec("prenorm_residual", {
                    "mixer_name": "self_attn", "feed_forward_name": "mlp",
                    "mixer_norm_name": "input_layernorm", "feed_forward_norm_name": "post_attention_layernorm"}),
                mixer=mixer, mixer_norm=norm, feed_forward=ffn, feed_forward_norm=norm))
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            layers=tuple(layers),
            order=tuple(LayerRun(l, c) for l, c in self.layer_order),
            final_norm=norm,
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                         "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None}),
            embedding_prefix="model.embed_tokens", final_norm_prefix="model.norm", lm_head_prefix="lm_head",
        )
        spec.validate()
        return spec

    # Names that the reference's graph and its GGUF files use for the same tensors
    # (src/io/gguf_weight_loader.cpp:36-52,362-380), translated to the names of the
    # architecture's own checkpoints so that a folder written with either naming loads.
    _LAYER_ALIASES = {
        "attn_norm": "input_layernorm", "q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj",
        "v_proj": "self_attn.v_proj", "o_proj": "self_attn.o_proj", "q_norm": "self_attn.q_norm",
        "k_norm": "self_attn.k_norm", "ffn_norm": "post_attention_layernorm",
        "gate_proj": "mlp.gate_proj", "up_proj": "mlp.up_proj", "down_proj": "mlp.down_proj",
        # GGUF spellings
        "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
        "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
        "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
    }
    _GLOBAL_ALIASES = {
        "tok_embeddings.weight": "model.embed_tokens.weight", "token_embd.weight": "model.embed_tokens.weight",
        "output_norm.weight": "model.norm.weight", "output.weight": "lm_head.weight",
    }

    @classmethod
    def canonical_tensor_name(cls, name: str) -> str:
        """Translate a tensor name of the reference's naming to the checkpoint naming."""
        if name in cls._GLOBAL_ALIASES:
            return cls._GLOBAL_ALIASES[name]
        for lead in ("layer_", "blk."):
            if name.startswith(lead):
                rest = name[len(lead):]
                idx, _, tail = rest.partition(".")
                if not idx.isdigit():
                    raise ConfigError(f"tensor name {name!r}: layer index {idx!r} is not a number")
                part, _, leaf = tail.rpartition(".")
                if part in cls._LAYER_ALIASES:
                    return f"model.layers.{int(idx)}.{cls._LAYER_ALIASES[part]}.{leaf}"
        return name
