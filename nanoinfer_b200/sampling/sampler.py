"""Token selection for a batch of logit rows, on the device.

Order (nanoinfer/sampling.py:126-151): repetition penalty -> greedy when temperature is 0 ->
temperature -> top-k -> top-p -> softmax -> draw. The uniform number of a draw is a function of
(seed, number of tokens the request has generated), so what a request samples does not depend on
the batch it is in, nor on whether it was preempted and recomputed. The reference draws from a
stateful generator per sequence (cpp/python/ni/scheduler.py:69), so its sampled tokens are
reproducible only within one engine; so are these.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .params import SamplingParams

_M64 = (1 << 64) - 1


def uniform_for(seed: int, counter: int) -> float:
    """A number in [0, 1) with 24 random bits from (seed, counter): splitmix64 finaliser."""
    x = ((int(seed) & _M64) * 0x9E3779B97F4A7C15 + (int(counter) + 1) * 0xD1B54A32D192ED03) & _M64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


@dataclass
class SampleRow:
    params: SamplingParams
    context: Optional[Sequence[int]]   # prompt + generated so far (read only with a penalty)
    generated: int                     # tokens generated so far: the draw counter
    seed: int = 0


class Sampler:
    def __init__(self, ops, device):
        self.ops, self.device = ops, torch.device(device)

    def sample(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> List[int]:
        """One token per row of ``logits [len(rows), vocab]`` (float32, on the device; penalised in place)."""
        n = len(rows)
        if n == 0:
            return []
        assert logits.shape[0] == n
        dev = logits.device
        if any(r.params.repetition_penalty != 1.0 for r in rows):
            seen, start = [], [0]
            for r in rows:
                if r.params.repetition_penalty != 1.0:
                    if r.context is None:
                        raise ValueError("repetition_penalty != 1 needs the request's context")
                    seen.append(np.unique(np.asarray(r.context, dtype=np.int64)).astype(np.int32))
                else:
                    seen.append(np.zeros(0, np.int32))
                start.append(start[-1] + seen[-1].size)
            flat = np.concatenate(seen) if start[-1] else np.zeros(1, np.int32)
            self.ops.repetition_penalty(
                logits, torch.from_numpy(flat).to(dev), torch.tensor(start, dtype=torch.int32, device=dev),
                torch.tensor([r.params.repetition_penalty for r in rows], dtype=torch.float32, device=dev))
        out = torch.empty(n, dtype=torch.int32, device=dev)
        if all(r.params.greedy for r in rows):
            self.ops.argmax(logits, out)
            return out.tolist()
        greedy = torch.empty(n, dtype=torch.int32, device=dev)
        self.ops.argmax(logits, greedy)
        temp = torch.tensor([r.params.temperature if not r.params.greedy else 1.0 for r in rows],
                            dtype=torch.float32, device=dev)
        top_k = torch.tensor([r.params.k for r in rows], dtype=torch.int32, device=dev)
        top_p = torch.tensor([r.params.p for r in rows], dtype=torch.float32, device=dev)
        uni = torch.tensor([uniform_for(r.seed, r.generated) for r in rows], dtype=torch.float32, device=dev)
        self.ops.sample(logits, temp, top_k, top_p, uni, out)
        g, s = greedy.tolist(), out.tolist()
        return [g[i] if rows[i].params.greedy else s[i] for i in range(n)]
