"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

The reference reads eight attributes of a loaded configuration object
(engine/model.py:64-80: num_hidden_layers, num_attention_heads,
num_key_value_heads, head_dim with the hidden // heads fallback, hidden_size,
rms_norm_eps, vocab_size, rope_parameters["rope_theta"]). This reader takes the
same keys from the JSON file, plus the ones the reference leaves implicit in its
tensor shapes or never looks at: intermediate_size, tie_word_embeddings,
max_position_embeddings, hidden_act, and the sliding-window keys. No size has a
default here unless the reference has one.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError


def _need(raw: Mapping[str, Any], key: str, kind):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: key '{key}' is missing")
    try:
        value = kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: key '{key}' = {raw[key]!r} is not {kind.__name__}") from exc
    return value


def _positive(name: str, value: int) -> int:
    if value < 1:
        raise ConfigError(f"config.json: key '{name}' must be at least 1, got {value}")
    return value


@dataclass(frozen=True)
class Qwen2Config:
    """Every size and constant of a Qwen2 checkpoint."""

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
    # Sliding window: layers with index >= max_window_layers see only the last
    # `sliding_window` keys when use_sliding_window is set; 0 window means all keys.
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    architecture: str = "Qwen2ForCausalLM"

    @property
    def num_kv_groups(self) -> int:
        """Query heads per key/value head (engine/model.py:55-57)."""
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def attention_scale(self) -> float:
        """head_dim ** -0.5 (engine/model.py:59-62)."""
        return self.head_dim ** -0.5

    def layer_window(self, layer: int) -> int:
        """The window of one layer; 0 stands for every earlier key."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    # ------------------------------------------------------------------ #

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen2Config":
        arch = raw.get("architectures") or ["Qwen2ForCausalLM"]
        hidden = _positive("hidden_size", _need(raw, "hidden_size", int))
        heads = _positive("num_attention_heads", _need(raw, "num_attention_heads", int))
        kv_heads = _positive("num_key_value_heads", _need(raw, "num_key_value_heads", int))
        if raw.get("head_dim"):
            head_dim = _positive("head_dim", int(raw["head_dim"]))
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: 'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}"
                )
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}"
            )
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary pairs")

        theta = cls._rope_theta(raw)
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (the feed-forward is SwiGLU: 'silu')")

        layers = _positive("num_hidden_layers", _need(raw, "num_hidden_layers", int))
        use_window = bool(raw.get("use_sliding_window", False))
        window = 0
        first_windowed = layers
        if use_window:
            window = _positive("sliding_window", _need(raw, "sliding_window", int))
            first_windowed = int(raw.get("max_window_layers", layers))
            if first_windowed < 0:
                raise ConfigError(f"config.json: max_window_layers must not be negative, got {first_windowed}")

        eps = _need(raw, "rms_norm_eps", float)
        if not eps > 0.0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")

        return cls(
            vocab_size=_positive("vocab_size", _need(raw, "vocab_size", int)),
            hidden_size=hidden,
            intermediate_size=_positive("intermediate_size", _need(raw, "intermediate_size", int)),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=eps,
            rope_theta=theta,
            max_position_embeddings=_positive(
                "max_position_embeddings", _need(raw, "max_position_embeddings", int)
            ),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=first_windowed,
            architecture=str(arch[0]),
        )

    @staticmethod
    def _rope_theta(raw: Mapping[str, Any]) -> float:
        """rope_theta as a flat key, or under rope_parameters (engine/model.py:79). Only the
        `default` rotary type exists in the reference (engine/model.py:145-146)."""
        for holder in ("rope_parameters", "rope_scaling"):
            nested = raw.get(holder)
            if isinstance(nested, Mapping):
                kind = nested.get("rope_type", nested.get("type", "default"))
                if kind != "default":
                    raise ConfigError(
                        f"config.json: {holder}.rope_type '{kind}' is not supported (only 'default')"
                    )
        if raw.get("rope_theta") is not None:
            theta = float(raw["rope_theta"])
        elif isinstance(raw.get("rope_parameters"), Mapping) and "rope_theta" in raw["rope_parameters"]:
            theta = float(raw["rope_parameters"]["rope_theta"])
        else:
            raise ConfigError("config.json: key 'rope_theta' is missing (flat or under 'rope_parameters')")
        if not theta > 0.0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta}")
        return theta

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen2Config":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> dict[str, Any]:
        """The config.json that reads back as this configuration."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
        }
        if self.use_sliding_window:
            out["sliding_window"] = self.sliding_window
            out["max_window_layers"] = self.max_window_layers
        return out
