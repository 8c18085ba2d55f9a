"""Engine options: everything that is a choice of the run, not a property of the model.

One typed object handed over at construction; there are no process-wide switches.
(The reference spreads such choices over a construction-time struct, a mutable global and
environment variables: cpp/src/backend.hpp:189-193, cpp/src/cuda/cuda_backend.hpp:43-95.)
"""
from __future__ import annotations

from dataclasses import dataclass

from .kernel_options import KernelOptions


_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"          # "bfloat16": serving kernels; "float32": true 32-bit everywhere
    page_size: int = 16              # tokens per cache page
    num_pages: int = 0               # pages per cache group; 0 = size from max_cache_tokens
    max_cache_tokens: int = 0        # used when num_pages == 0
    max_batch: int = 8               # most requests live at a time (also the number of state slots)
    max_tokens_per_step: int = 2048  # token budget of one step (scheduler)
    device: str = "cuda:0"
    cuda_graphs: bool = True         # replay captured graphs for pure-decode steps
    kernel_options: KernelOptions = KernelOptions()   # pins kernel paths; the defaults leave the choice to the library

    def __post_init__(self):
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(set(_DTYPES))}, got {self.dtype!r}")
        object.__setattr__(self, "dtype", _DTYPES[self.dtype])
        if self.page_size <= 0:
            raise ValueError("page_size must be > 0")
        if self.max_batch <= 0:
            raise ValueError("max_batch must be > 0")
        if self.max_tokens_per_step <= 0:
            raise ValueError("max_tokens_per_step must be > 0")

    def pages_needed(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def resolved_num_pages(self) -> int:
        if self.num_pages > 0:
            return self.num_pages
        if self.max_cache_tokens > 0:
            return self.pages_needed(self.max_cache_tokens)
        raise ValueError("EngineConfig needs num_pages or max_cache_tokens")
