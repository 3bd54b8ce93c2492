"""One registry from the architecture's name (config.json `architectures[0]`) to its model.

An entry holds the typed configuration class and the builder that turns a
configuration into a `ModelSpec`. The reference has a single hard-wired class
(engine/model.py:164, `Qwen2Engine`); here the name decides, everywhere: the
loader, the random-weights writer, generation and trace replay all go through
`resolve`.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .errors import ConfigError
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen2 import Qwen2Config


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    build_spec: Callable[[Any], ModelSpec]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec) -> None:
    ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def resolve(raw: Mapping[str, Any]):
    """(typed configuration, ModelSpec) for the dictionary of a config.json."""
    names = raw.get("architectures")
    if not names:
        raise ConfigError("config.json: key 'architectures' is missing; known: " + ", ".join(sorted(ARCHITECTURES)))
    arch = ARCHITECTURES.get(str(names[0]))
    if arch is None:
        raise ConfigError(
            f"config.json: architecture '{names[0]}' is not registered; known: " + ", ".join(sorted(ARCHITECTURES))
        )
    config = arch.config_class.from_dict(raw)
    return config, arch.build_spec(config)


def resolve_folder(folder: str | Path):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no such file")
    return resolve(json.loads(path.read_text()))


# --------------------------------------------------------------------------- #
# Qwen2 dense decoder (engine/model.py:322-351: per layer norm, attention, residual,
# norm, SwiGLU, residual; then the final norm and the head)
# --------------------------------------------------------------------------- #

def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    rotary = {"kind": "rotary", "head_dim": cfg.head_dim, "theta": cfg.rope_theta}
    layers = []
    for i in range(cfg.num_hidden_layers):
        prefix = f"model.layers.{i}"
        norm = {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        layers.append(
            LayerSpec("pre_norm_residual", dict(
                mixer_norm=PartSpec("rms_norm", norm, f"{prefix}.input_layernorm"),
                mixer=PartSpec(
                    "gqa_attention",
                    {
                        "hidden_size": cfg.hidden_size,
                        "num_heads": cfg.num_attention_heads,
                        "num_kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "qkv_bias": True,  # always present in the reference (engine/model.py:87-92)
                        "scale": cfg.attention_scale,
                        "window": cfg.layer_window(i),
                        "position_encoding": rotary,
                    },
                    f"{prefix}.self_attn",
                ),
                feed_forward_norm=PartSpec("rms_norm", norm, f"{prefix}.post_attention_layernorm"),
                feed_forward=PartSpec(
                    "swiglu",
                    {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size},
                    f"{prefix}.mlp",
                ),
            ))
        )
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec(
            "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "model.embed_tokens"
        ),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm"),
        head=PartSpec(
            "lm_head",
            {
                "vocab_size": cfg.vocab_size,
                "hidden_size": cfg.hidden_size,
                "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
            },
            "lm_head",
        ),
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_spec)
