"""Built-in parts; importing this package registers them."""
from . import spec, base  # noqa: F401
from . import norm, position, attention, feedforward, embedding, block  # noqa: F401
from .spec import ModelPlan, LayerSpec, PartSpec, ScheduleEntry, TensorSpec
from .base import (CacheNeed, PagedTensor, FoldedNorm, LazyNorm, StateNeed, StepContext, HostBatch, LayerCache, Runtime, Part, Norm,
                   PositionEncoding, Mixer, FeedForward, Embedding, Head)

__all__ = ["ModelPlan", "LayerSpec", "PartSpec", "ScheduleEntry", "TensorSpec", "CacheNeed", "PagedTensor", "FoldedNorm", "LazyNorm",
           "StateNeed", "StepContext", "HostBatch", "LayerCache", "Runtime", "Part", "Norm",
           "PositionEncoding", "Mixer", "FeedForward", "Embedding", "Head"]
