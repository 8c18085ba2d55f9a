"""The registries: architecture name -> (configuration class, plan builder), and part kind -> class.

``config.json``'s ``architectures[0]`` chooses the model everywhere in the engine (loader,
entry points, trace replay). The reference keys its only registry by ``model_type``
(nanoinfer/weights.py:147-155); this one is keyed by the architecture name.

Adding an architecture: write a ``ModelConfig`` subclass that reads its config.json keys and a
function ``plan(config) -> ModelPlan``; call ``register_architecture``. Adding a part: write the
class (interfaces in ``parts/base.py``) and call ``register_part(kind, cls)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Type

from .config.model_config import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    plan: Callable  # (ModelConfig) -> ModelPlan


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, type] = {}
_ARRANGEMENTS: Dict[str, type] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], plan: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, plan)


def architecture_names():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}'; this engine knows {sorted(_ARCHITECTURES)}") from None


def config_from_json_dict(d: Mapping) -> ModelConfig:
    """Choose the architecture by ``architectures[0]`` and read its typed configuration."""
    archs = d.get("architectures")
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0]).config_cls.from_json_dict(d)


def plan_for(config: ModelConfig):
    plan = get_architecture(config.architecture).plan(config)
    plan.validate()
    return plan


def register_part(kind: str, cls: type) -> None:
    """Register a mixer, feed-forward, norm, position encoding, embedding or head class."""
    _PARTS[kind] = cls


def get_part(kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[kind]
    except KeyError:
        raise KeyError(f"unknown part kind '{kind}'; registered: {sorted(_PARTS)}") from None


def register_arrangement(name: str, cls: type) -> None:
    _ARRANGEMENTS[name] = cls


def get_arrangement(name: str) -> type:
    _ensure_builtin()
    try:
        return _ARRANGEMENTS[name]
    except KeyError:
        raise KeyError(f"unknown block arrangement '{name}'; registered: {sorted(_ARRANGEMENTS)}") from None


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    from . import parts as _parts  # noqa: F401  registers the built-in parts
    from .models import qwen2 as _qwen2  # noqa: F401  registers Qwen2ForCausalLM
