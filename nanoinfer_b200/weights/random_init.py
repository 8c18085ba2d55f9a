"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

Distributions: N(0, 0.02) for matrices, embeddings and biases, 1 + N(0, 0.1) for norm gains.
Each tensor has a generator of its own, seeded from (seed, tensor name), so a tensor's values do
not depend on which other tensors exist or in which order they are made. The reference has no
such mode in its C++ engine; its oracle tests build ``Model(cfg)`` with framework-default
initialisation (tests/test_cache.py:65-75).
"""
from __future__ import annotations

import os
import zlib
from typing import Dict

import torch

from ..config.model_config import ModelConfig, write_config_json
from ..parts.spec import ModelPlan, TensorSpec
from .safetensors_io import save_safetensors

_STD = {"matrix": 0.02, "embedding": 0.02, "bias": 0.02}


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1)


def random_tensor(ts: TensorSpec, seed: int, dtype: torch.dtype) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(_tensor_seed(seed, ts.name))
    x = torch.randn(ts.shape, generator=g, dtype=torch.float32)
    if ts.init == "gain":
        x = 1.0 + 0.1 * x
    elif ts.init in _STD:
        x = _STD[ts.init] * x
    else:
        raise ValueError(f"tensor '{ts.name}': unknown init rule '{ts.init}'")
    return x.to(dtype)


def random_tensors(plan: ModelPlan, seed: int, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    return {ts.name: random_tensor(ts, seed, dtype) for ts in plan.tensor_specs()}


def write_random_model(config: ModelConfig, model_dir: str, seed: int = 0,
                       dtype: str = "bfloat16") -> str:
    """Create ``model_dir`` with config.json and model.safetensors; returns ``model_dir``."""
    from ..registry import plan_for
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    plan = plan_for(config)
    os.makedirs(model_dir, exist_ok=True)
    write_config_json(config, model_dir)
    tensors = random_tensors(plan, seed, torch_dtype)
    save_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                     metadata={"format": "pt", "seed": str(seed)})
    return model_dir
