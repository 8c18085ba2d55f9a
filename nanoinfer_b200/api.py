"""The Python entry points, in the reference's manner.

* ``load_model(model_dir, dtype=..., ...) -> Model`` (reference: ``nicpp.Model(weights_dir, mode, device)``,
  cpp/bindings/nicpp.cpp:207-217; ``nanoinfer.weights.load_model``, nanoinfer/weights.py:25-71).
* ``Model.generate(prompt_ids, max_tokens=20, params=SamplingParams(), seed=0, eos_id=-1) -> list[int]``
  (cpp/bindings/nicpp.cpp:296-316; loop: cpp/src/generate.cpp:10-42).
* ``generate(model, tokenizer, prompt, max_tokens=32, use_cache=True, sampling=None) -> str``
  (nanoinfer/generate.py:33-85).
* ``Request`` and ``Scheduler`` for many requests (cpp/python/ni/scheduler.py).
"""
from __future__ import annotations

from typing import List, Optional

from .config.engine_config import EngineConfig
from .config.kernel_options import KernelOptions
from .engine.engine import Engine
from .engine.scheduler import Request, Scheduler
from .sampling.params import SamplingParams
from .sampling.sampler import Sampler


class Model:
    """A loaded model with its cache and sampler: what requests are run on."""

    def __init__(self, model_dir: str, engine_config: EngineConfig, ops=None):
        self.engine = Engine(model_dir, engine_config, ops=ops)
        self.config = self.engine.config
        self.sampler = Sampler(self.engine.rt.ops, self.engine.device)
        self.eos_token_id = self.engine.plan.eos_token_id

    def generate(self, prompt_ids: List[int], max_tokens: int = 20, params: Optional[SamplingParams] = None,
                 seed: int = 0, eos_id: int = -1, use_cache: bool = True) -> List[int]:
        """Continue ``prompt_ids`` by up to ``max_tokens`` tokens; EOS ends generation and is not returned.

        ``use_cache=False`` is the reference's ``--no-cache`` (nanoinfer/generate.py:44-60, 94-98): every
        token is computed from the whole sequence so far with nothing kept between tokens. It is slow and
        exists to check the cache: both ways give the same tokens."""
        params = params or SamplingParams()
        if params.seed is not None:
            seed = params.seed
        if not use_cache:
            return self._generate_recomputing(list(prompt_ids), max_tokens, params, seed, eos_id)
        sched = Scheduler(self, lookahead=True)      # run() to the end: the one-step lag of the host is not seen
        sched.add(Request("generate", list(prompt_ids), max_tokens=max_tokens, temperature=params.temperature,
                          top_k=params.k, top_p=params.p, repetition_penalty=params.repetition_penalty,
                          seed=seed, eos_id=eos_id))
        return sched.run()["generate"]      # run() gives back what the request holds if a step raises

    def weight_bytes(self):
        """(bytes the weights take on the device, the same with every element in 32-bit), as the reference's
        ``Model.weight_bytes`` (cpp/bindings/nicpp.cpp:317)."""
        return self.engine.model.weight_bytes()

    def weight_breakdown(self):
        """dtype name -> (tensors, bytes) (the reference lists its storage formats: cpp/src/model.cpp:320-334)."""
        return self.engine.model.weight_breakdown()

    def _generate_recomputing(self, ids: List[int], max_tokens: int, params: SamplingParams, seed: int,
                              eos_id: int) -> List[int]:
        from .engine.engine import StepEntry
        from .sampling.sampler import SampleRow
        eos = eos_id if eos_id >= 0 else self.eos_token_id
        out: List[int] = []
        if not ids:
            return out
        budget = self.engine.engine_config.max_tokens_per_step
        while len(out) < max_tokens:
            rc = self.engine.open("generate-no-cache")
            try:
                for start in range(0, len(ids), budget):        # the whole sequence again, in portions
                    part = ids[start:start + budget]
                    last = start + len(part) == len(ids)
                    logits = self.engine.step([StepEntry(rc, part, [len(part) - 1] if last else [])])
            finally:
                self.engine.close(rc)
            context = ids if params.repetition_penalty != 1.0 else None
            token = self.sampler.sample(logits, [SampleRow(params, context, len(out), seed)])[0]
            if token == eos:
                break
            out.append(token)
            ids = ids + [token]
            if len(ids) >= self.engine.max_positions:
                break       # the cached way's stop rule (Scheduler._accept): no position is left for another token
        self.engine.check_device()
        return out


def load_model(model_dir: str, dtype: str = "bfloat16", page_size: int = 16, num_pages: int = 0,
               max_cache_tokens: int = 0, max_batch: int = 8, max_tokens_per_step: int = 2048,
               device: str = "cuda:0", cuda_graphs: bool = True,
               kernel_options: Optional[KernelOptions] = None) -> Model:
    if num_pages <= 0 and max_cache_tokens <= 0:
        max_cache_tokens = 16384
    cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=num_pages, max_cache_tokens=max_cache_tokens,
                       max_batch=max_batch, max_tokens_per_step=max_tokens_per_step, device=device,
                       cuda_graphs=cuda_graphs, kernel_options=kernel_options or KernelOptions())
    return Model(model_dir, cfg)


def generate(model: Model, tokenizer, prompt: str, max_tokens: int = 32, use_cache: bool = True,
             sampling: Optional[SamplingParams] = None) -> str:
    """Text in, text out. ``tokenizer`` needs ``encode(str) -> ids`` and ``decode(ids) -> str``.
    ``use_cache=False`` recomputes the whole sequence for every token (see ``Model.generate``)."""
    enc = tokenizer.encode(prompt)
    ids = list(getattr(enc, "ids", enc))
    eos = getattr(tokenizer, "eos_token_id", None)
    out = model.generate(ids, max_tokens=max_tokens, params=sampling or SamplingParams(),
                         eos_id=eos if eos is not None else -1, use_cache=use_cache)
    return tokenizer.decode(out)
