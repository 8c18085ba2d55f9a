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
    distinct: bool = False             # ``context`` lists every id once already (an int32 array): nothing to sort out


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
        self._pinned_ids: List[torch.Tensor] = []   # and of the ids that a repetition penalty applies to
        self._seen_turn = 0

    @staticmethod
    def can_sample_async(rows: Sequence[SampleRow]) -> bool:
        """Any rows: greedy and sampled ones in any mix; a row with a repetition penalty brings its context, and the
        one id that the host may not know yet (the token of the step in flight) is read on the device."""
        return bool(rows)

    _RING = 4       # pinned buffers in rotation: one is reused only after three more steps have been launched

    def _pinned_pair(self, n: int):
        """This call's pinned buffers (tokens out, sampling parameters in), large enough for ``n`` rows."""
        if not self._pinned or self._pinned[0].numel() < n:
            size = max(256, 2 * n)
            self._pinned = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(self._RING)]
            self._pinned_par = [torch.empty(4 * size, dtype=torch.float32).pin_memory() for _ in range(self._RING)]
        self._turn = (self._turn + 1) % self._RING
        return self._pinned[self._turn], self._pinned_par[self._turn]

    def sample_async(self, logits: torch.Tensor, rows: Sequence[SampleRow],
                     pending: Optional[torch.Tensor] = None) -> PendingTokens:
        """As ``sample``, without waiting for the device. ``pending`` [rows] int32 on the device: each row's newest
        token where the host has not read it yet, so that it is missing from the row's context; a penalty takes it
        from there."""
        n = len(rows)
        assert logits.shape[0] == n and self.can_sample_async(rows)
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        on_gpu = out.device.type == "cuda"
        host, stage = self._pinned_pair(n) if on_gpu else (None, None)
        self._penalise(logits, rows, pending)
        if all(r.params.greedy for r in rows):
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
        self._penalise(logits, rows, None)
        out = torch.empty(n, dtype=torch.int32, device=dev)
        if all(r.params.greedy for r in rows):
            self.ops.argmax(logits, out)
            return out.tolist()
        self.ops.sample(logits, *self._device_parameters(rows, dev), out)
        return out.tolist()

    def _penalise(self, logits: torch.Tensor, rows: Sequence[SampleRow], pending: Optional[torch.Tensor]) -> None:
        """The repetition penalty of the rows that have one, on the raw logits, in place. The distinct ids of all rows
        go to the device with the penalties and the rows' offsets as one array from pinned memory (one copy in stream
        order; nothing waits)."""
        if not any(r.params.repetition_penalty != 1.0 for r in rows):
            return
        dev = logits.device
        seen, start = [], [0]
        for r in rows:
            if r.params.repetition_penalty != 1.0:
                if r.context is None:
                    raise ValueError("repetition_penalty != 1 needs the request's context")
                ids = np.asarray(r.context, dtype=np.int32) if r.distinct else \
                    np.unique(np.asarray(r.context, dtype=np.int64)).astype(np.int32)
                seen.append(ids)
            else:
                seen.append(np.zeros(0, np.int32))
            start.append(start[-1] + seen[-1].size)
        n = len(rows)
        packed = np.empty(2 * n + 1 + max(start[-1], 1), dtype=np.int32)       # [penalties as bits | starts | ids]
        packed[:n].view(np.float32)[:] = [r.params.repetition_penalty for r in rows]
        packed[n:2 * n + 1] = start
        packed[2 * n + 1:] = 0
        if start[-1]:
            packed[2 * n + 1:2 * n + 1 + start[-1]] = np.concatenate(seen)
        if dev.type == "cuda":
            stage = self._pinned_seen(packed.size)
            stage[:packed.size].numpy()[:] = packed
            d = torch.empty(packed.size, dtype=torch.int32, device=dev)
            d.copy_(stage[:packed.size], non_blocking=True)
        else:
            d = torch.from_numpy(packed)
        self.ops.repetition_penalty(logits, d[2 * n + 1:], d[n:2 * n + 1], d[:n].view(torch.float32), pending)

    def _pinned_seen(self, size: int) -> torch.Tensor:
        """Pinned staging for the ids of the penalty, in the same rotation as the other two buffers."""
        if len(self._pinned_ids) != self._RING or self._pinned_ids[0].numel() < size:
            self._pinned_ids = [torch.empty(max(4096, 2 * size), dtype=torch.int32).pin_memory() for _ in range(self._RING)]
        self._seen_turn = (self._seen_turn + 1) % self._RING
        return self._pinned_ids[self._seen_turn]

    def _device_parameters(self, rows: Sequence[SampleRow], dev, stage=None):
        """Temperature, top-k, top-p and the uniform numbers of the rows on the device: one array (top-k as integer
        bits), one copy from pinned memory. A greedy row beside sampled ones is the draw at 0 from the one largest
        logit at temperature 1: of the elements that are kept (the maxima) the first in vocabulary order is taken,
        which is what the argmax kernel gives."""
        n = len(rows)
        par = np.empty((4, n), dtype=np.float32)
        par[0] = [1.0 if r.params.greedy else r.params.temperature for r in rows]
        par[1].view(np.int32)[:] = [1 if r.params.greedy else r.params.k for r in rows]
        par[2] = [1.0 if r.params.greedy else r.params.p for r in rows]
        par[3] = [0.0 if r.params.greedy else uniform_for(r.seed, r.generated) for r in rows]
        if torch.device(dev).type == "cuda":
            if stage is None:
                _, stage = self._pinned_pair(n)
            stage[:4 * n].numpy()[:] = par.reshape(-1)
            d = torch.empty(4 * n, dtype=torch.float32, device=dev)
            d.copy_(stage[:4 * n], non_blocking=True)
        else:
            d = torch.from_numpy(par.reshape(-1).copy())
        return d[:n], d[n:2 * n].view(torch.int32), d[2 * n:3 * n], d[3 * n:]
