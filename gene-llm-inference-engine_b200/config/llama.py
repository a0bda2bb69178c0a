"""Configuration of the Llama architecture, read from its own config.json keys.

Keys, defaults and refusals follow the reference loader (src/loader/hf_checkpoint.cpp:28-136):
required ``hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, vocab_size``;
optional with defaults ``num_key_value_heads`` (= heads), ``max_position_embeddings`` (2048),
``head_dim`` (hidden / heads), ``rope_theta`` (10000), ``rms_norm_eps`` (1e-6), ``rope_scaling``
(none) and ``tie_word_embeddings`` (false); JSON ``null`` counts as absent.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_INT_LIMIT = 100_000_000


@dataclass(frozen=True)
class RopeScaling:
    """The "llama3" frequency scaling (src/common/rope_style.h:8-13)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position: int

    def to_json(self) -> Dict[str, Any]:
        return {"rope_type": "llama3", "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position}


def _is_int(v: Any) -> bool:
    if isinstance(v, bool):
        return False
    if isinstance(v, int):
        return True
    return isinstance(v, float) and math.isfinite(v) and v == int(v)


def _required_int(cfg: Dict[str, Any], key: str) -> int:
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"config.json has no '{key}'")
    return _checked_int(cfg[key], key)


def _optional_int(cfg: Dict[str, Any], key: str, fallback: int) -> int:
    if key not in cfg or cfg[key] is None:
        return fallback
    return _checked_int(cfg[key], key)


def _checked_int(v: Any, key: str) -> int:
    if not _is_int(v) or not (0 < int(v) <= _INT_LIMIT):
        raise ConfigError(f"config.json: '{key}' has an invalid value ({v!r})")
    return int(v)


def _optional_number(cfg: Dict[str, Any], key: str, fallback: float) -> float:
    v = cfg.get(key)
    if v is None:
        return fallback
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"config.json: '{key}' is not a number ({v!r})")
    return float(v)


def parse_rope_scaling(s: Any) -> Optional[RopeScaling]:
    """None / absent / type "default" mean no scaling; "llama3" is implemented; every other
    type is refused rather than run with wrong positions (src/loader/hf_checkpoint.cpp:57-90)."""
    if s is None:
        return None
    if not isinstance(s, dict):
        raise ConfigError("rope_scaling is not an object")
    kind = None
    for key in ("rope_type", "type"):
        if key in s:
            if not isinstance(s[key], str):
                raise ConfigError(f"rope_scaling.{key} is not a string")
            kind = s[key]
            break
    if kind == "default":
        return None
    if kind != "llama3":
        raise ConfigError(f"rope_scaling type '{kind}' is not supported (only 'llama3')")

    def number(key: str) -> float:
        v = s.get(key)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"rope_scaling.{key} is required for type 'llama3'")
        return float(v)

    factor, low, high = number("factor"), number("low_freq_factor"), number("high_freq_factor")
    original = number("original_max_position_embeddings")
    if not factor >= 1.0:
        raise ConfigError("rope_scaling.factor must be >= 1")
    if not low > 0.0 or not high > low:
        raise ConfigError("rope_scaling needs 0 < low_freq_factor < high_freq_factor")
    if not original >= 1.0 or original > 1e9 or original != int(original):
        raise ConfigError("rope_scaling.original_max_position_embeddings must be a positive integer")
    return RopeScaling(factor, low, high, int(original))


@dataclass(frozen=True)
class LlamaConfig:
    """Typed Llama configuration (the fields of src/loader/checkpoint.h:76-97)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool

    architecture = "LlamaForCausalLM"
    model_type = "llama"

    @property
    def attn_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_json(cls, j: Any) -> "LlamaConfig":
        if not isinstance(j, dict):
            raise ConfigError("config.json is not a JSON object")
        mt = j.get("model_type")
        if isinstance(mt, str) and mt != "llama":
            raise ConfigError(f"unsupported model_type '{mt}' for LlamaForCausalLM (only 'llama')")
        act = j.get("hidden_act")
        if isinstance(act, str) and act != "silu":
            raise ConfigError(f"unsupported hidden_act '{act}'")
        for bias in ("attention_bias", "mlp_bias"):
            if j.get(bias) is True:
                raise ConfigError(f"{bias} = true is not supported")

        hidden = _required_int(j, "hidden_size")
        inter = _required_int(j, "intermediate_size")
        layers = _required_int(j, "num_hidden_layers")
        heads = _required_int(j, "num_attention_heads")
        kv_heads = _optional_int(j, "num_key_value_heads", heads)
        vocab = _required_int(j, "vocab_size")
        max_pos = _optional_int(j, "max_position_embeddings", 2048)
        head_dim = _optional_int(j, "head_dim", 0)
        if head_dim == 0:
            if hidden % heads != 0:
                raise ConfigError("hidden_size is not divisible by num_attention_heads")
            head_dim = hidden // heads
        if heads % kv_heads != 0:
            raise ConfigError("num_attention_heads must be divisible by num_key_value_heads")
        if head_dim % 2 != 0:
            raise ConfigError("head_dim must be even (RoPE rotates pairs)")
        theta = _optional_number(j, "rope_theta", 10000.0)
        if not theta > 0:
            raise ConfigError("rope_theta must be positive")
        eps = _optional_number(j, "rms_norm_eps", 1e-6)
        if not eps >= 0:
            raise ConfigError("rms_norm_eps must be >= 0")
        scaling = parse_rope_scaling(j.get("rope_scaling"))
        tie = j.get("tie_word_embeddings") is True
        return cls(hidden, inter, layers, heads, kv_heads, head_dim, vocab, max_pos, theta, eps, scaling, tie)

    def to_json(self) -> Dict[str, Any]:
        return {
            "architectures": [self.architecture], "model_type": self.model_type,
            "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "vocab_size": self.vocab_size, "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "rope_scaling": self.rope_scaling.to_json() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
        }

    # ------------------------------------------------------------------ translation into parts
    def model_spec(self) -> ModelSpec:
        """Every layer: pre-norm block, causal GQA attention with half-split RoPE, SwiGLU
        (order of operations in src/model/transformer.cpp:379-451)."""
        rope = PartSpec("rope", {
            "head_dim": self.head_dim, "theta": self.rope_theta, "pairing": "half_split",
            "scaling": None if self.rope_scaling is None else {
                "factor": self.rope_scaling.factor, "low_freq_factor": self.rope_scaling.low_freq_factor,
                "high_freq_factor": self.rope_scaling.high_freq_factor,
                "original_max_position": self.rope_scaling.original_max_position},
        })
        mixer = PartSpec("attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "window": None, "scale": 1.0 / math.sqrt(self.head_dim), "position": rope,
        })
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        layer = LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm)
        n = self.num_hidden_layers
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_position=self.max_position_embeddings, layers=[layer] * n,
            schedule=[ScheduleEntry(i) for i in range(n)], final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings)
