"""Built-in parts; importing this package registers them."""
from . import spec, base  # noqa: F401
from . import norm, position, attention, feedforward, embedding, block  # noqa: F401
from .spec import ModelPlan, LayerSpec, PartSpec, ScheduleEntry, TensorSpec
from .base import (CacheNeed, StateNeed, StepContext, HostBatch, LayerCache, Runtime, Part, Norm,
                   PositionEncoding, Mixer, FeedForward, Embedding, Head)

__all__ = ["ModelPlan", "LayerSpec", "PartSpec", "ScheduleEntry", "TensorSpec", "CacheNeed",
           "StateNeed", "StepContext", "HostBatch", "LayerCache", "Runtime", "Part", "Norm",
           "PositionEncoding", "Mixer", "FeedForward", "Embedding", "Head"]
