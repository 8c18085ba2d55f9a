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


class PendingTokens:
    """Tokens sampled on the device whose copy to the host is under way: ``device`` can feed the next
    step at once, ``wait()`` returns the ids."""

    def __init__(self, device: torch.Tensor, host: torch.Tensor, event, n: int):
        self.device, self._host, self._event, self._n = device, host, event, n

    def wait(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host[:self._n].tolist()


class Sampler:
    def __init__(self, ops, device):
        self.ops, self.device = ops, torch.device(device)
        self._pinned: List[torch.Tensor] = []       # host buffers of the asynchronous reads, used in turn
        self._pinned_par: List[torch.Tensor] = []   # and of the sampling parameters on their way to the device
        self._turn = 0

    @staticmethod
    def can_sample_async(rows: Sequence[SampleRow]) -> bool:
        """Rows without a penalty that are all greedy or all sampled: nothing the host must wait for."""
        if not rows or any(r.params.repetition_penalty != 1.0 for r in rows):
            return False
        greedy = [r.params.greedy for r in rows]
        return all(greedy) or not any(greedy)

    _RING = 4       # pinned buffers in rotation: one is reused only after three more steps have been launched

    def _pinned_pair(self, n: int):
        """This call's pinned buffers (tokens out, sampling parameters in), large enough for ``n`` rows."""
        if not self._pinned or self._pinned[0].numel() < n:
            size = max(256, 2 * n)
            self._pinned = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(self._RING)]
            self._pinned_par = [torch.empty(4 * size, dtype=torch.float32).pin_memory() for _ in range(self._RING)]
        self._turn = (self._turn + 1) % self._RING
        return self._pinned[self._turn], self._pinned_par[self._turn]

    def sample_async(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> PendingTokens:
        """As ``sample`` for rows that ``can_sample_async`` accepts, without waiting for the device."""
        n = len(rows)
        assert logits.shape[0] == n and self.can_sample_async(rows)
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        on_gpu = out.device.type == "cuda"
        host, stage = self._pinned_pair(n) if on_gpu else (None, None)
        if rows[0].params.greedy:
            self.ops.argmax(logits, out)
        else:
            self.ops.sample(logits, *self._device_parameters(rows, out.device, stage), out)
        if not on_gpu:       # a host backend (tests): nothing is asynchronous
            return PendingTokens(out, out, None, n)
        host[:n].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(out, host, event, n)

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
        any_greedy = any(r.params.greedy for r in rows)
        greedy = None
        if any_greedy:
            greedy = torch.empty(n, dtype=torch.int32, device=dev)
            self.ops.argmax(logits, greedy)
        self.ops.sample(logits, *self._device_parameters(rows, dev), out)
        s = out.tolist()
        if not any_greedy:
            return s
        g = greedy.tolist()
        return [g[i] if rows[i].params.greedy else s[i] for i in range(n)]

    def _device_parameters(self, rows: Sequence[SampleRow], dev, stage=None):
        """Temperature, top-k, top-p and the uniform numbers of the rows on the device: one array (top-k as integer
        bits), one copy from pinned memory. A greedy row's temperature is 1 (its sample is not used)."""
        n = len(rows)
        par = np.empty((4, n), dtype=np.float32)
        par[0] = [r.params.temperature if not r.params.greedy else 1.0 for r in rows]
        par[1].view(np.int32)[:] = [r.params.k for r in rows]
        par[2] = [r.params.p for r in rows]
        par[3] = [uniform_for(r.seed, r.generated) for r in rows]
        if torch.device(dev).type == "cuda":
            if stage is None:
                _, stage = self._pinned_pair(n)
            stage[:4 * n].numpy()[:] = par.reshape(-1)
            d = torch.empty(4 * n, dtype=torch.float32, device=dev)
            d.copy_(stage[:4 * n], non_blocking=True)
        else:
            d = torch.from_numpy(par.reshape(-1).copy())
        return d[:n], d[n:2 * n].view(torch.int32), d[2 * n:3 * n], d[3 * n:]
