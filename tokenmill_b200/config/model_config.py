"""Typed model configuration for the Qwen2 dense decoder, read from the keys of its config.json.

Parity with the reference's ``ModelConfig`` (src/infer/config.py:13-69): the same required keys
(``vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads``), the same
defaults for the optional ones (``num_key_value_heads`` = heads, ``max_position_embeddings`` = 32768,
``rms_norm_eps`` = 1e-6, ``tie_word_embeddings`` = False when the key is absent, ``rope_theta`` falling
back to ``rope_parameters.rope_theta`` and then 10000.0), and the same merge of end-of-sequence ids from
``generation_config.json`` and then ``config.json``.

Beyond the reference this config also accepts an explicit ``head_dim`` (default hidden // heads) and
refuses, with a clear error, the options this architecture does not implement (a sliding window, rope
scaling, an activation other than silu) instead of silently ignoring them.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, or names an option the engine does not implement."""


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads")


@dataclass
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 32768
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    attention_bias: bool = True          # Qwen2 always biases q/k/v (src/infer/model/layers.py:139)
    eos_token_ids: list[int] = field(default_factory=list)
    architecture: str = "Qwen2ForCausalLM"

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                              f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotate-half position encoding")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")

    @property
    def num_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_dict(cls, raw: dict[str, Any], generation: dict[str, Any] | None = None) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {missing}")
        if raw.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window=true is not implemented for Qwen2 (the reference engine "
                              "never reads the key); set it to false")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"rope_scaling={raw['rope_scaling']!r} is not implemented")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act={raw['hidden_act']!r} is not implemented (only 'silu')")
        heads = raw["num_attention_heads"]
        rope_theta = raw.get("rope_theta")
        if rope_theta is None:
            rope_theta = (raw.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if raw["hidden_size"] % heads:
                raise ConfigError(f"hidden_size ({raw['hidden_size']}) is not a multiple of "
                                  f"num_attention_heads ({heads}) and no head_dim is given")
            head_dim = raw["hidden_size"] // heads
        eos: list[int] = []
        for source in ([generation] if generation else []) + [raw]:
            val = source.get("eos_token_id")
            if val is None:
                continue
            for tok in val if isinstance(val, list) else [val]:
                if int(tok) not in eos:
                    eos.append(int(tok))
        arch = (raw.get("architectures") or ["Qwen2ForCausalLM"])[0]
        return cls(
            vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"], num_hidden_layers=raw["num_hidden_layers"],
            num_attention_heads=heads, num_key_value_heads=raw.get("num_key_value_heads", heads),
            head_dim=head_dim, max_position_embeddings=raw.get("max_position_embeddings", 32768),
            rope_theta=float(rope_theta), rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", True)),
            eos_token_ids=eos, architecture=arch)

    def to_dict(self) -> dict[str, Any]:
        """The config.json this configuration round-trips through."""
        out: dict[str, Any] = {
            "architectures": [self.architecture], "model_type": "qwen2",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.attention_bias,
            "hidden_act": "silu", "use_sliding_window": False,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def read_config_json(path: str | Path) -> tuple[dict[str, Any], dict[str, Any] | None]:
    """(config.json, generation_config.json or None) of a model folder."""
    path = Path(path)
    cfg_file = path / "config.json"
    if not cfg_file.exists():
        raise ConfigError(f"no config.json in {path}")
    raw = json.loads(cfg_file.read_text())
    gen_file = path / "generation_config.json"
    gen = json.loads(gen_file.read_text()) if gen_file.exists() else None
    return raw, gen
