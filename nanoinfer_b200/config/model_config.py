"""Typed model configuration, read from the architecture's own ``config.json`` keys.

Every size and constant that ``config.json`` gives is carried here and handed to the
parts as parameters; no part and no kernel holds a model size of its own.

Reference: nanoinfer/config.py:32-163 (``ModelConfig.from_hf``: the keys, their defaults
and the rope_theta / sliding-window / attention-bias reading rules) and
cpp/src/config.cpp:63-75 (validation: required sizes positive, heads divisible by
kv heads).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """A config.json that is missing a key, has a wrong type or asks for an unsupported option."""


def _need_int(d: Mapping[str, Any], key: str, *, positive: bool = True) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if positive and v <= 0:
        raise ConfigError(f"config.json: '{key}' must be > 0, got {v}")
    return v


def _opt_int(d: Mapping[str, Any], key: str, default: Optional[int]) -> Optional[int]:
    v = d.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    return v


def _opt_float(d: Mapping[str, Any], key: str, default: float) -> float:
    v = d.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


def read_rope_theta(d: Mapping[str, Any], default: float = 10000.0) -> float:
    """``rope_theta`` at top level, or inside ``rope_parameters`` / ``rope_scaling``.

    Reference: nanoinfer/config.py:13-29.
    """
    theta = d.get("rope_theta")
    if theta is None:
        for key in ("rope_parameters", "rope_scaling"):
            params = d.get(key)
            if isinstance(params, dict) and params.get("rope_theta") is not None:
                theta = params["rope_theta"]
                break
    if theta is None:
        return default
    if isinstance(theta, bool) or not isinstance(theta, (int, float)) or theta <= 0:
        raise ConfigError(f"config.json: rope_theta must be a positive number, got {theta!r}")
    return float(theta)


def read_rope_scaling(d: Mapping[str, Any]) -> Optional[dict]:
    """A real scaling rule, or None for the absent / "default" / "linear" cases.

    Reference: nanoinfer/config.py:118-126.
    """
    for key in ("rope_scaling", "rope_parameters"):
        rs = d.get(key)
        if isinstance(rs, dict):
            rtype = rs.get("rope_type") or rs.get("type")
            if rtype not in (None, "default", "linear"):
                return dict(rs)
    return None


@dataclass(frozen=True)
class ModelConfig:
    """What every decoder architecture in this engine states about itself."""

    architecture: str
    model_type: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_id: int  # -1: none

    def to_json_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        raise NotImplementedError

    @classmethod
    def from_json_dict(cls, d: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """The Qwen2 / Qwen2.5 dense decoder (``Qwen2ForCausalLM``)."""

    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    hidden_act: str = "silu"
    attention_bias: bool = True
    # Window of keys that layers >= max_window_layers attend to; 0 = every layer sees all keys.
    sliding_window: int = 0
    max_window_layers: int = 0
    torch_dtype: str = "bfloat16"

    @property
    def n_rep(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_json_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        archs = d.get("architectures") or []
        architecture = archs[0] if archs else "Qwen2ForCausalLM"
        model_type = d.get("model_type", "qwen2")
        heads = _need_int(d, "num_attention_heads")
        hidden = _need_int(d, "hidden_size")
        head_dim = _opt_int(d, "head_dim", None) or hidden // heads
        kv_heads = _opt_int(d, "num_key_value_heads", None) or heads

        # q/k/v bias: Qwen2 always has it; an explicit flag wins (nanoinfer/config.py:106-110).
        ab = d.get("attention_bias")
        attention_bias = bool(ab) if ab is not None else (model_type == "qwen2")

        # The window counts only when the model opts in (nanoinfer/config.py:112-116).
        sw = _opt_int(d, "sliding_window", None)
        use_sw = d.get("use_sliding_window")
        if use_sw is None:
            use_sw = False if model_type == "qwen2" else sw is not None
        window = int(sw) if (use_sw and sw) else 0
        max_window_layers = _opt_int(d, "max_window_layers", 0) or 0

        if read_rope_scaling(d) is not None:
            raise ConfigError(
                f"config.json: rope_scaling {read_rope_scaling(d)!r} is not supported by "
                f"{architecture} in this engine (only unscaled rotary positions)")

        eos = d.get("eos_token_id", -1)
        if isinstance(eos, list):
            eos = eos[0] if eos else -1
        if eos is None:
            eos = -1

        cfg = cls(
            architecture=architecture,
            model_type=model_type,
            vocab_size=_need_int(d, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_need_int(d, "num_hidden_layers"),
            max_position_embeddings=_opt_int(d, "max_position_embeddings", 4096),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_id=int(eos),
            intermediate_size=_need_int(d, "intermediate_size"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_opt_float(d, "rms_norm_eps", 1e-6),
            rope_theta=read_rope_theta(d),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=attention_bias,
            sliding_window=window,
            max_window_layers=max_window_layers if window else 0,
            torch_dtype=str(d.get("torch_dtype") or d.get("dtype") or "bfloat16"),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ConfigError(f"head_dim must be positive and even, got {self.head_dim}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if self.max_position_embeddings <= 0:
            raise ConfigError("max_position_embeddings must be > 0")
        if self.sliding_window < 0:
            raise ConfigError("sliding_window must be >= 0")

    def to_json_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.sliding_window > 0,
            "sliding_window": self.sliding_window if self.sliding_window else None,
            "max_window_layers": self.max_window_layers,
            "eos_token_id": self.eos_token_id if self.eos_token_id >= 0 else None,
            "torch_dtype": self.torch_dtype,
        }
        return d


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in '{model_dir}'")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def write_config_json(cfg: ModelConfig, model_dir: str) -> str:
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "config.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(cfg.to_json_dict(), f, indent=2)
        f.write("\n")
    return path
