"""Weights by tensor name: load a model folder into the tensors that a plan asks for.

Kept as stored: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 and float64
become float32 (float16 -> float32 loses nothing; bfloat16 would drop three mantissa bits, which the
32-bit path must not), integer tables become int32. The parts then take what they need: matrix
operands in the engine's compute dtype, gains and biases in 32-bit.

All problems of a checkpoint are reported together in ONE error: missing tensors, unexpected
tensors, wrong shapes and wrong element types (a matrix, embedding, gain or bias stored as integers
or booleans; an integer table stored as floats). Reference: nanoinfer/weights.py:56-68 (missing /
unexpected after remap raise), cpp/src/model.cpp:336-340 (``missing weight <name>``) and
cpp/src/serialize.cpp:18-64 (a file whose element type is not the expected one is refused).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.spec import ModelPlan
from .safetensors_io import SafetensorsError, open_model_files


class WeightError(ValueError):
    """A checkpoint that does not fit the plan. ``missing``, ``unexpected``, ``wrong_shape`` and
    ``wrong_dtype`` list why."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong_shape: List[str],
                 wrong_dtype: List[str] = ()):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"weights in '{where}' do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong element types ({len(self.wrong_dtype)}): " + "; ".join(self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT_TAGS = ("F64", "F32", "F16", "BF16")


def _as_kept(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.float32)
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
    wrong_dtype = []
    for n, ts in wanted.items():
        if n not in where_is:
            continue
        tag = where_is[n].dtype_tag(n)
        floating = tag in _FLOAT_TAGS
        if ts.integer and floating:
            wrong_dtype.append(f"{n}: stored as {tag}, the model needs an integer table")
        elif not ts.integer and not floating:
            wrong_dtype.append(f"{n}: stored as {tag}, the model needs floating point ({ts.init})")
    if missing or unexpected or wrong or wrong_dtype:
        raise WeightError(model_dir, missing, unexpected, wrong, wrong_dtype)
    return {n: _as_kept(where_is[n].tensor(n)) for n in wanted}
