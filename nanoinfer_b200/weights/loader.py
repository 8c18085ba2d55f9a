"""Weights by tensor name: load a model folder into the tensors that a plan asks for.

Kept as stored: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 becomes
bfloat16 (the engine has no float16 kernels), integer tables become int32. The parts then take
what they need: matrix operands in the engine's compute dtype, gains and biases in 32-bit.

All problems of a checkpoint are reported together in ONE error: missing tensors, unexpected
tensors and wrong shapes. Reference: nanoinfer/weights.py:56-68 (missing / unexpected after
remap raise) and cpp/src/model.cpp:336-340 (``missing weight <name>``).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.spec import ModelPlan
from .safetensors_io import SafetensorsError, open_model_files


class WeightError(ValueError):
    """A checkpoint that does not fit the plan. ``missing``, ``unexpected`` and ``wrong_shape`` list why."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong_shape: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"weights in '{where}' do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        super().__init__("\n".join(lines))


def _as_kept(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.bfloat16 if t.dtype == torch.float16 else torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool, torch.int32):
        return t.to(torch.int32)
    raise SafetensorsError(f"unsupported tensor dtype {t.dtype}")


def load_tensors(model_dir: str, plan: ModelPlan) -> Dict[str, torch.Tensor]:
    """CPU tensors for every name in ``plan.tensor_specs()``; raises ``WeightError`` otherwise."""
    files = open_model_files(model_dir)
    where_is = {}
    for f in files:
        for name in f.names():
            where_is[name] = f
    specs = plan.tensor_specs()
    wanted = {ts.name: ts for ts in specs}
    missing = [n for n in wanted if n not in where_is]
    ignored = set(plan.ignored_tensors)
    unexpected = sorted(n for n in where_is if n not in wanted and n not in ignored)
    wrong = []
    for n, ts in wanted.items():
        if n in where_is and tuple(where_is[n].shape(n)) != tuple(ts.shape):
            wrong.append(f"{n}: file has {list(where_is[n].shape(n))}, model needs {list(ts.shape)}")
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)
    return {n: _as_kept(where_is[n].tensor(n)) for n in wanted}
