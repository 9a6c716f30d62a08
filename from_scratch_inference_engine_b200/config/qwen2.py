"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

Keys, defaults and derived values follow the reference parser
(src/model/model_config.cpp:9-33, include/engine/model_config.hpp:10-28):
`num_key_value_heads` defaults to the head count, `head_dim` to
hidden_size / num_attention_heads, `rope_theta` to 10000, `rms_norm_eps` to 1e-6,
and `model_type == "qwen2"` switches the q/k/v bias on (other model types follow
`attention_bias`).  Keys the reference leaves unread are read here as well:
`architectures` (registry key), `max_position_embeddings` (position limit),
`tie_word_embeddings` (checked against the checkpoint) and the three window keys.
The window keys mean what the published configuration documents: with
`use_sliding_window` the layers from `max_window_layers` on see only the last
`sliding_window` keys, the layers before see all of them.
"""

from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, List, Mapping, Optional

from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine runs."""


def _require(data: Mapping[str, Any], key: str, kind=int):
    if key not in data:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    value = data[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    return kind(value)


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    attention_qkv_bias: bool = True
    hidden_act: str = "silu"
    model_type: str = "qwen2"
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    eos_token_id: Optional[int] = None

    architecture = "Qwen2ForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen2Config":
        hidden = _require(data, "hidden_size")
        layers = _require(data, "num_hidden_layers")
        heads = _require(data, "num_attention_heads")
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive")
        kv_heads = int(data.get("num_key_value_heads", heads))
        head_dim = int(data["head_dim"]) if data.get("head_dim") is not None else hidden // heads
        model_type = str(data.get("model_type", ""))
        qkv_bias = True if model_type == "qwen2" else bool(data.get("attention_bias", False))
        eos = data.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        if data.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is not supported (the reference applies "
                              "plain rotary encoding only)")
        use_window = bool(data.get("use_sliding_window", False))
        config = cls(
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_require(data, "intermediate_size"),
            vocab_size=_require(data, "vocab_size"),
            max_position_embeddings=int(data.get("max_position_embeddings", 0) or 0),
            rope_theta=float(data.get("rope_theta", 10000.0)),
            rms_norm_eps=float(data.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            attention_qkv_bias=qkv_bias,
            hidden_act=str(data.get("hidden_act", "silu")),
            model_type=model_type,
            use_sliding_window=use_window,
            sliding_window=int(data.get("sliding_window", 0) or 0),
            max_window_layers=int(data.get("max_window_layers", layers) or 0),
            eos_token_id=None if eos is None else int(eos),
        )
        config.validate()
        return config

    def to_dict(self) -> Dict[str, Any]:
        data = asdict(self)
        data["attention_bias"] = data.pop("attention_qkv_bias")
        data["architectures"] = [self.architecture]
        if data["eos_token_id"] is None:
            del data["eos_token_id"]
        return data

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        problems: List[str] = []
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"):
            if getattr(self, key) <= 0:
                problems.append(f"{key} must be positive, got {getattr(self, key)}")
        if not problems:
            if self.num_attention_heads % self.num_key_value_heads != 0:
                problems.append(
                    f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                    f"num_key_value_heads ({self.num_key_value_heads})")
            if self.head_dim % 2 != 0:
                problems.append(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if self.hidden_act != "silu":
            problems.append(f"hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        if self.rms_norm_eps < 0:
            problems.append("rms_norm_eps must not be negative")
        if self.rope_theta <= 0:
            problems.append("rope_theta must be positive")
        if self.max_position_embeddings < 0:
            problems.append("max_position_embeddings must not be negative")
        if self.use_sliding_window:
            if self.sliding_window <= 0:
                problems.append("use_sliding_window needs a positive sliding_window")
            if not 0 <= self.max_window_layers <= max(self.num_hidden_layers, 0):
                problems.append("max_window_layers must lie in [0, num_hidden_layers]")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))

    # ------------------------------------------------------------ derived sizes
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> int:
        """Number of keys layer `layer` sees; 0 means all of them."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    # --------------------------------------------------------------------- spec
    def build_spec(self) -> ModelSpec:
        """Lay the configuration out as parts.

        Wiring as in the reference forward (src/model/model.cpp:104-148): per layer
        norm -> attention -> residual -> norm -> SwiGLU -> residual, then a final norm
        and the output head, which is `lm_head.weight` unless the embeddings are tied.
        """
        norm = PartSpec("rmsnorm", {"width": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rotary", {"theta": self.rope_theta, "rotary_dim": self.head_dim,
                                   "max_position": self.max_position_embeddings})
        mlp = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                  "intermediate_size": self.intermediate_size})
        layers = []
        for index in range(self.num_hidden_layers):
            attention = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qkv_bias": self.attention_qkv_bias,
                "window": self.layer_window(index),
                "position": rope,
            })
            layers.append(LayerSpec(
                prefix=f"model.layers.{index}.",
                mixer_name="self_attn.",
                feed_forward_name="mlp.",
                mixer_norm_name="input_layernorm.",
                feed_forward_norm_name="post_attention_layernorm.",
                arrangement="prenorm",
                mixer=attention,
                feed_forward=mlp,
                mixer_norm=norm,
                feed_forward_norm=norm,
            ))
        return ModelSpec(
            architecture=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_position=self.max_position_embeddings,
            embedding_name="model.embed_tokens.weight",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            final_norm=norm,
            final_norm_prefix="model.norm.",
            layers=tuple(layers),
            schedule=tuple(LayerCall(layer=i) for i in range(self.num_hidden_layers)),
        )
