"""Continuous batching above the step function.

Every step takes, under a token budget, one token from each request that is decoding and a
portion of the prompt of each request that is still being prefilled, admits waiting requests
into free places, runs them all as ONE batch, samples where a request's last known token was in
the batch, and finishes and frees what is done.

The reference's scheduler (cpp/python/ni/scheduler.py:200-375) has the same queues, stop rules and
counters, but prefills each admitted prompt whole and alone and reserves the worst case of pages up
front. Here pages are taken step by step. When the pool cannot hold a step's new tokens, the request
admitted last is preempted: its pages are given back, it returns to the head of the waiting queue
and is later recomputed from its prompt and the tokens it had generated.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, List, Optional

import numpy as np

from ..cache.pages import OutOfPages
from ..sampling.params import SamplingParams
from ..sampling.sampler import SampleRow
from .engine import StepEntry


@dataclass
class Request:
    """A generation request; the reference's names and defaults (cpp/python/ni/scheduler.py:37-51)."""
    request_id: str
    prompt_ids: List[int]
    max_tokens: int = 32
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 0
    eos_id: int = -1      # -1: the model's eos_token_id

    def sampling(self) -> SamplingParams:
        return SamplingParams(temperature=self.temperature, top_k=self.top_k, top_p=self.top_p,
                              repetition_penalty=self.repetition_penalty, seed=self.seed)


class State(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class Sequence:
    """A request at run time: what it has generated, what of it is in the cache."""

    def __init__(self, req: Request, order: int):
        self.req = req
        self.params = req.sampling()
        self.ids: List[int] = list(req.prompt_ids)   # prompt + output, grown in place
        self.output_ids: List[int] = []
        self.state = State.WAITING
        self.cache = None          # RequestCache while running
        self.fed = 0               # tokens of (prompt + output) that the cache holds
        self.order = order         # admission order; the largest is preempted first
        self.preemptions = 0
        self._distinct = np.empty(64, dtype=np.int32)      # the distinct ids of ``ids`` in order of first appearance
        self._distinct_set: set = set()
        self._distinct_upto = 0                             # how many of ``ids`` they cover
        self._prompt_array = None                           # the prompt as an int32 array, once a portion of it is run

    @property
    def all_ids(self) -> List[int]:
        return self.ids

    def distinct_ids(self) -> np.ndarray:
        """Every id of prompt + output once (what a repetition penalty applies to), kept up to date token by token."""
        have = self._distinct_set
        for tok in self.ids[self._distinct_upto:]:
            if tok not in have:
                if len(have) == self._distinct.size:
                    self._distinct = np.concatenate([self._distinct, np.empty_like(self._distinct)])
                self._distinct[len(have)] = tok
                have.add(tok)
        self._distinct_upto = len(self.ids)
        return self._distinct[:len(have)]

    def tokens(self, start: int, count: int):
        """``ids[start:start + count]`` as a step takes them. A portion that lies in the prompt is a view of the prompt as
        an int32 array, made once (turning two thousand Python integers into an array for every portion is the dearest
        thing the host does before a prompt step's first launch); anything else, and a prompt that holds something
        other than integers of 32 bits (the step refuses it by name), is the list's slice."""
        if count > 1 and start + count <= len(self.req.prompt_ids):
            if self._prompt_array is None:
                try:
                    a = np.asarray(self.req.prompt_ids)
                    whole = a.ndim == 1 and a.dtype.kind in "iu" and -2 ** 31 <= int(a.min()) and int(a.max()) < 2 ** 31
                    self._prompt_array = a.astype(np.int32) if whole else False
                except (OverflowError, TypeError, ValueError):
                    self._prompt_array = False
            if self._prompt_array is not False:
                return self._prompt_array[start:start + count]
        return self.ids[start:start + count]

    def sample_row(self, generated: int) -> SampleRow:
        """The row that draws this request's token number ``generated``."""
        if self.params.repetition_penalty != 1.0:
            return SampleRow(self.params, self.distinct_ids(), generated, self.req.seed, distinct=True)
        return SampleRow(self.params, None, generated, self.req.seed)

    @property
    def pending(self) -> int:
        return len(self.ids) - self.fed

    def emit(self, tok: int) -> None:
        self.output_ids.append(tok)
        self.ids.append(tok)


@dataclass
class PlannedEntry:
    seq: Sequence
    start: int          # first token (index into all_ids) of the portion
    count: int
    samples: bool       # the portion ends at the last known token: a token is sampled from its last row


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    admitted: List[Sequence] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    """``add()`` requests, then ``run()``; or call ``step()`` yourself.

    ``model`` offers ``engine`` (with ``cache``, ``open``, ``close``, ``step``), ``sampler`` and
    ``eos_token_id``."""

    def __init__(self, model, max_batch: Optional[int] = None, max_tokens_per_step: Optional[int] = None,
                 lookahead: bool = False):
        """``lookahead``: decoding steps (greedy and sampled rows in any mix, with or without a repetition penalty) are launched with the previous step's tokens still on the
        device; the host reads them while the new step runs, so ``finished`` and the sequences' outputs lag
        one step behind the device, and a request that stops at EOS has run one step too many (its result is
        dropped). What is generated is the same."""
        self.model = model
        self.lookahead = lookahead
        self._inflight = None      # (sequences, PendingTokens) of a step whose tokens the host has not read yet
        self.steps_ahead = 0       # steps launched before the host had read the previous one's tokens
        self.engine = model.engine
        ec = self.engine.engine_config
        self.max_batch = min(max_batch or ec.max_batch, ec.max_batch)
        self.max_tokens_per_step = max_tokens_per_step or ec.max_tokens_per_step
        if self.max_tokens_per_step < self.max_batch:
            raise ValueError("max_tokens_per_step must be at least max_batch (one token for each decoding request)")
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.finished: Dict[str, List[int]] = {}
        self._eos_default = model.eos_token_id
        self._order = 0
        self.steps = 0
        self.peak_batch = 0
        self.tokens_run = 0
        self.peak_step_tokens = 0       # the most tokens that one step carried
        self.prompt_steps = 0           # steps that carried a portion of a prompt ...
        self.prompt_step_tokens = 0     # ... and the tokens of those steps (against the budget: stats())
        self.preemptions = 0

    # ---- queue ----------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        cache = self.engine.cache
        worst = len(req.prompt_ids) + max(req.max_tokens, 1)
        need = -(-worst // cache.page_size)
        if cache.groups and need > cache.num_pages:
            raise ValueError(f"request {req.request_id} needs {need} pages; the pool has {cache.num_pages} "
                             f"(raise num_pages or page_size)")
        if len(req.prompt_ids) > self.engine.max_positions:
            raise ValueError(f"request {req.request_id}: prompt of {len(req.prompt_ids)} tokens exceeds the "
                             f"model's context length {self.engine.max_positions}")
        req.sampling()  # validates
        self._order += 1
        self.waiting.append(Sequence(req, self._order))

    def has_work(self) -> bool:
        return bool(self.running or self.waiting)

    def _finish(self, seq: Sequence) -> None:
        seq.state = State.FINISHED
        self.finished[seq.req.request_id] = seq.output_ids
        if seq.cache is not None:
            self.engine.close(seq.cache)
            seq.cache = None
        self.engine.check_device()      # what is handed out as finished was computed by kernels that all completed

    def _accept(self, seq: Sequence, tok: int) -> bool:
        """Stop rules, in the reference's order (cpp/python/ni/scheduler.py:250-259): EOS is checked before
        the token is emitted, so it is not part of the output; then max_tokens."""
        eos = seq.req.eos_id if seq.req.eos_id >= 0 else self._eos_default
        if eos >= 0 and tok == eos:
            return True
        seq.emit(tok)
        if len(seq.ids) >= self.engine.max_positions:
            return True            # no position left for another token
        return len(seq.output_ids) >= seq.req.max_tokens

    # ---- planning: decisions only, nothing runs -------------------------------------------
    def _pages_for_new(self, tokens: int) -> int:
        return -(-tokens // self.engine.cache.page_size)

    def plan(self) -> StepPlan:
        cache = self.engine.cache
        plan = StepPlan()
        budget = self.max_tokens_per_step

        # 1. running requests: decoding ones first (one token each), then prompts in admission order
        order = sorted(self.running, key=lambda s: (s.pending > 1, s.order))
        for seq in order:
            if budget <= 0:
                break
            n = min(seq.pending, budget)
            plan.entries.append(PlannedEntry(seq, seq.fed, n, samples=(n == seq.pending)))
            budget -= n

        # 2. pages for them; preempt the request admitted last until the step fits
        free = [cache.num_free(g) for g in range(len(cache.groups))]
        while plan.entries:
            need = cache.demand([(e.seq.cache, e.count) for e in plan.entries])
            if all(k <= f for k, f in zip(need, free)):
                free = [f - k for f, k in zip(free, need)]
                break
            victim = max((e.seq for e in plan.entries), key=lambda s: s.order)
            if len(self.running) == 1:
                raise OutOfPages(f"request {victim.req.request_id} alone does not fit the cache pool")
            plan.entries = [e for e in plan.entries if e.seq is not victim]
            plan.preempted.append(victim)
            self._preempt(victim)
            free = [cache.num_free(g) for g in range(len(cache.groups))]     # the victim's pages came back

        # 3. admit waiting requests, first come first served, while places, budget and pages last
        while self.waiting and len(self.running) < self.max_batch and budget > 0 and not plan.preempted:
            seq = self.waiting[0]
            if not seq.req.prompt_ids:
                self.waiting.popleft()
                self.finished[seq.req.request_id] = []
                seq.state = State.FINISHED
                continue
            # the whole of what is known of the request, and one more token, must fit what is free now
            need = self._pages_for_new(len(seq.all_ids) + 1)
            if any(need > f for f in free):
                break       # head of the line waits; nobody skips ahead
            self.waiting.popleft()
            seq.cache = self.engine.open(seq.req.request_id)
            seq.state = State.RUNNING
            seq.fed = 0
            self.running.append(seq)
            plan.admitted.append(seq)
            n = min(seq.pending, budget)
            plan.entries.append(PlannedEntry(seq, 0, n, samples=(n == seq.pending)))
            budget -= n
            free = [f - need for f in free]
        return plan

    def _preempt(self, seq: Sequence) -> None:
        self.engine.close(seq.cache)
        seq.cache = None
        seq.fed = 0
        seq.state = State.WAITING
        seq.preemptions += 1
        self.preemptions += 1
        self.running.remove(seq)
        self.waiting.appendleft(seq)

    # ---- one step -------------------------------------------------------------------------
    def _resolve_inflight(self) -> None:
        """Read the tokens of the step in flight and apply the stop rules."""
        if self._inflight is None:
            return
        seqs, pending = self._inflight
        self._inflight = None
        for seq, tok in zip(seqs, pending.wait()):
            if seq.state is not State.RUNNING:
                continue            # stopped meanwhile (EOS one step earlier, cancelled): the extra token is dropped
            if self._accept(seq, int(tok)):
                self._finish(seq)
        self.running = [s for s in self.running if s.state is State.RUNNING]

    def _continuation(self):
        """The sequences of the step in flight, if the next step is exactly one more token for each of them:
        nobody waits to be admitted, nobody's token in flight is its last by count, and the pages for one more token
        each are there. Greedy and sampled rows may stand in one batch (the sampling kernel takes both), and so may
        rows with a repetition penalty (the id that the host has not read yet is penalised from the device's copy)."""
        if self._inflight is None or self.waiting:
            return None
        seqs, _ = self._inflight
        if len(seqs) != len(self.running) or len(seqs) > self.max_tokens_per_step:
            return None
        for a, b in zip(seqs, sorted(self.running, key=lambda s: s.order)):
            if a is not b or a.state is not State.RUNNING:
                return None
            if len(a.output_ids) + 1 >= a.req.max_tokens or len(a.ids) + 2 >= self.engine.max_positions:
                return None
        if not self.engine.cache.fits([(s.cache, 1) for s in seqs]):
            return None
        return seqs

    def _step_ahead(self, seqs) -> StepPlan:
        """Launch the next decode step from the device's copy of the tokens in flight, then read those."""
        _, pending = self._inflight
        entries = [StepEntry(s.cache, [0], [0]) for s in seqs]       # the ids are placeholders
        rows = [s.sample_row(len(s.output_ids) + 1) for s in seqs]      # the host's ids lack the token in flight:
        logits = self.engine.step(entries, borrow_logits=True, device_tokens=pending.device)
        nxt = self.model.sampler.sample_async(logits, rows, pending=pending.device)   # a penalty reads it there
        plan = StepPlan(entries=[PlannedEntry(s, s.fed, 1, True) for s in seqs])
        for s in seqs:
            s.fed += 1              # the token in flight is in the cache now; ``ids`` gets it below
        self._resolve_inflight()
        self._inflight = (list(seqs), nxt)
        self.tokens_run += len(seqs)
        self.peak_step_tokens = max(self.peak_step_tokens, len(seqs))
        self.peak_batch = max(self.peak_batch, len(seqs))
        self.steps += 1
        self.steps_ahead += 1
        return plan

    def step(self) -> StepPlan:
        if self.lookahead:
            seqs = self._continuation()
            if seqs is not None:
                return self._step_ahead(seqs)
            self._resolve_inflight()
        plan = self.plan()
        if plan.entries:
            entries, rows, samplers = [], [], []
            for e in plan.entries:
                ids = e.seq.tokens(e.start, e.count)
                wants = e.samples and e.seq.req.max_tokens > 0
                entries.append(StepEntry(e.seq.cache, ids, [e.count - 1] if wants else []))
                if wants:
                    samplers.append(e.seq)
                    rows.append(e.seq.sample_row(len(e.seq.output_ids)))
            logits = self.engine.step(entries, borrow_logits=True)
            for e in plan.entries:
                e.seq.fed += e.count
            if self.lookahead and rows and len(samplers) == len(plan.entries) and \
                    all(e.count == 1 for e in plan.entries) and self.model.sampler.can_sample_async(rows):
                # a pure decode step without penalties: leave its tokens on the device for the next step to start from
                self._inflight = (samplers, self.model.sampler.sample_async(logits, rows))
                toks = []
            else:
                toks = self.model.sampler.sample(logits, rows) if rows else []
            for seq, tok in zip(samplers, toks):
                if self._accept(seq, int(tok)):
                    self._finish(seq)
            for e in plan.entries:      # prompts that wanted no token at all
                if e.samples and e.seq.req.max_tokens <= 0 and e.seq.state is State.RUNNING:
                    self._finish(e.seq)
            self.tokens_run += plan.num_tokens
            self.peak_step_tokens = max(self.peak_step_tokens, plan.num_tokens)
            if any(e.count > 1 or not e.samples for e in plan.entries):
                self.prompt_steps += 1
                self.prompt_step_tokens += plan.num_tokens
        self.running = [s for s in self.running if s.state is State.RUNNING]
        self.peak_batch = max(self.peak_batch, len(plan.entries))
        self.steps += 1
        return plan

    def stats(self) -> Dict[str, float]:
        """Counters of what ran so far. ``budget_use`` is the mean share of ``max_tokens_per_step`` that the steps
        with a portion of a prompt carried (1.0 = every such step was full); the reference's scheduler keeps
        ``peak_batch`` alone (cpp/src/scheduler.cpp)."""
        use = self.prompt_step_tokens / (self.prompt_steps * self.max_tokens_per_step) if self.prompt_steps else 0.0
        return {"steps": self.steps, "tokens_run": self.tokens_run, "peak_batch": self.peak_batch,
                "peak_step_tokens": self.peak_step_tokens, "prompt_steps": self.prompt_steps,
                "tokens_per_step": self.tokens_run / self.steps if self.steps else 0.0, "budget_use": use,
                "steps_ahead": self.steps_ahead, "preemptions": self.preemptions}

    def cancel(self, request_id: str) -> bool:
        """Queued: dropped with an empty output. Running: finished with what it has; pages are freed."""
        self._resolve_inflight()
        for seq in self.waiting:
            if seq.req.request_id == request_id:
                self.waiting.remove(seq)
                self.finished[request_id] = seq.output_ids
                seq.state = State.FINISHED
                return True
        for seq in self.running:
            if seq.req.request_id == request_id:
                self._finish(seq)
                self.running = [s for s in self.running if s.state is State.RUNNING]
                return True
        return False

    def run(self) -> Dict[str, List[int]]:
        try:
            while self.has_work():
                self.step()
        except BaseException:
            self.abort()
            raise
        self.engine.check_device()
        return self.finished

    def abort(self) -> None:
        """Give back what running requests hold (after an error in a step): the engine stays usable."""
        self._inflight = None
        for seq in list(self.running):
            if seq.cache is not None and not seq.cache.closed:
                self.engine.close(seq.cache)
            seq.cache = None
            seq.state = State.FINISHED
        self.running = []
