"""CUDA graphs for the two kinds of step whose launches repeat: pure decode, and prompt portions of a recurring shape.

DecodeGraphs: steps in which every request brings exactly one token.

Such a step launches a fixed sequence of kernels whose sizes depend only on the number of requests
and, for the split of long contexts, on the context length. The sequence is captured once per
(request bucket, context bucket) and replayed; the step's inputs (token ids, positions, block
tables, ...) live in a device buffer of fixed address that one host-to-device copy refreshes before
each replay. A batch smaller than its bucket is padded with rows that own no pages: kernels write
nothing for them and their attention is empty.

The reference captures a graph for ONE sequence and feeds position and token through device
scalars (cpp/src/cuda/cuda_backend.cu:1047-1119); the idea is the same, for any batch.
"""
from __future__ import annotations

import gc
import weakref
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


@dataclass
class _Captured:
    graph: "torch.cuda.CUDAGraph"
    inputs: torch.Tensor
    logits: torch.Tensor
    launches: int
    mirror: "_InputMirror" = None


class _InputMirror:
    """Pinned host copy of a captured graph's input buffer, kept up to date row by row.

    Between two decode steps of the same requests only the token, the position and the context length
    of a row change, and now and then one block-table entry; the mirror rewrites a row's block table
    only when the request in that row, or the version of its tables, differs from what the row holds.
    The layout is the one ``Engine.build_context`` produces for a padded batch of one-token requests."""

    def __init__(self, rb: int, widths: List[int], device: torch.device, pad_slot: int = 0):
        sizes = [rb, rb, rb, rb + 1, rb, rb, rb] + [rb * w for w in widths]
        self.size = sum(sizes)
        on_gpu = torch.device(device).type == "cuda"
        self.host = torch.empty(self.size, dtype=torch.int32)
        self.event = None                   # on a host backend (tests of the layout) nothing is asynchronous
        if on_gpu:
            self.host = self.host.pin_memory()
            self.event = torch.cuda.Event()
            self.event.record()
        h = self.host.numpy()
        offs = np.concatenate([[0], np.cumsum(sizes)])
        cut = [h[offs[i]:offs[i + 1]] for i in range(len(sizes))]
        self.tok, self.pos, req_index, q_start, self.ctx, self.slots, want = cut[:7]
        self.tables = [cut[7 + g].reshape(rb, w) for g, w in enumerate(widths)]
        h[:] = 0
        req_index[:] = np.arange(rb)
        q_start[:] = np.arange(rb + 1)
        want[:] = np.arange(rb)
        for t in self.tables:
            t[:] = -1
        self.pad_slot = pad_slot            # the state slot of rows without a request
        self.slots[:] = pad_slot
        self.rb = rb
        self.row_req = [None] * rb          # the request whose pages a row's block tables list
        self.row_ver = [-1] * rb

    def fill(self, entries) -> None:
        if self.event is not None:
            self.event.synchronize()        # the previous copy has left the buffer
        n = len(entries)
        self.tok[:n] = [e.tokens[0] for e in entries]
        lens = np.fromiter((e.request.length for e in entries), dtype=np.int32, count=n)
        self.pos[:n] = lens
        self.ctx[:n] = lens + 1
        row_req, row_ver = self.row_req, self.row_ver
        for i, e in enumerate(entries):
            rc = e.request
            if row_req[i] is not rc or row_ver[i] != rc.version:
                for t, held in zip(self.tables, rc.tables):
                    t[i, :len(held)] = held
                    t[i, len(held):] = -1
                self.slots[i] = rc.slot
                row_req[i], row_ver[i] = rc, rc.version
        for i in range(n, self.rb):         # rows that a request has left become padding again
            if row_req[i] is None:
                continue
            self.tok[i] = self.pos[i] = self.ctx[i] = 0
            self.slots[i] = self.pad_slot
            for t in self.tables:
                t[i, :] = -1
            row_req[i], row_ver[i] = None, -1

    def send(self, device_buffer: torch.Tensor) -> int:
        device_buffer.copy_(self.host, non_blocking=True)
        if self.event is not None:
            self.event.record()
        return self.size * 4


class DecodeGraphs:
    max_batch = 256

    def __init__(self, engine):
        self._engine = weakref.ref(engine)      # no reference cycle: an engine that is dropped dies at once
        self.captured: Dict[Tuple[int, int], _Captured] = {}
        self.seen = set()
        self.pool = None
        self.stream = None         # the side stream that captures

    @property
    def engine(self):
        return self._engine()

    def _key(self, entries) -> Tuple[int, int, List[int]]:
        eng = self.engine
        rb = _bucket(len(entries))
        max_ctx = max(e.request.length + 1 for e in entries)
        cb = max(256, _bucket(max_ctx))
        return rb, cb, eng.cache.table_widths(cb)

    def step(self, entries, borrow: bool = False, device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        eng = self.engine
        rb, cb, widths = self._key(entries)
        key = (rb, cb)
        cap = self.captured.get(key)
        if cap is None:
            if key not in self.seen:
                # the first step of a shape runs eagerly: it sets up whatever the kernels set up on first use
                self.seen.add(key)
                ctx, want_rows, _ = eng.build_context(entries)
                if device_tokens is not None:
                    ctx.token_ids[:len(entries)].copy_(device_tokens[:len(entries)], non_blocking=True)
                return eng.model.forward(ctx, eng.storage.layer_caches(ctx.block_tables), want_rows)
            cap = self._capture(key, entries, rb, cb, widths)
        cap.mirror.fill(entries)
        eng.last_h2d_bytes = cap.mirror.send(cap.inputs)
        if device_tokens is not None:       # the ids sampled on the device replace the placeholders (after the copy above, in stream order)
            cap.inputs[:len(entries)].copy_(device_tokens[:len(entries)], non_blocking=True)
        want_list = [i for i, e in enumerate(entries) for _ in e.want]
        cap.graph.replay()
        eng.graph_launches += cap.launches
        if not want_list:
            return None
        n = len(want_list)
        if want_list == list(range(n)):
            out = cap.logits[:n]
        else:
            out = cap.logits[torch.tensor(want_list, dtype=torch.long, device=cap.logits.device)]
            borrow = True
        return out if borrow else out.clone()

    def _capture(self, key, entries, rb: int, cb: int, widths: List[int]) -> _Captured:
        eng = self.engine
        probe, _, _ = eng.build_context(entries, pad_to=rb, widths=widths)
        size = sum(v.numel() for v in (probe.token_ids, probe.positions, probe.req_index, probe.q_start,
                                       probe.ctx_lens, probe.state_slots)) + rb \
            + sum(t.numel() for t in probe.block_tables.values())
        static = torch.empty(size, dtype=torch.int32, device=eng.device)
        ctx, want_rows, _ = eng.build_context(entries, pad_to=rb, widths=widths, static=static)
        ctx.host.ctx_lens = [cb] * rb           # launch shapes are chosen for the whole bucket
        caches = eng.storage.layer_caches(ctx.block_tables)
        ops = eng.rt.ops
        torch.cuda.synchronize()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        # Freeing device memory or another graph while a stream captures invalidates the capture, and the
        # cyclic collector may free such objects at any allocation: keep it off until the capture ends.
        # The capture is begun and ended by hand on a side stream: the ``torch.cuda.graph`` context would
        # collect garbage and empty the allocator's cache first, ~0.1 s per capture, which a short run with
        # a dozen (batch, context) buckets notices.
        gc_was_on = gc.isenabled()
        gc.disable()
        if self.stream is None:
            self.stream = torch.cuda.Stream()
        self.stream.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(self.stream):
                graph.capture_begin(pool=self.pool)
                try:
                    logits = eng.model.forward(ctx, caches, want_rows)
                finally:
                    graph.capture_end()
        finally:
            if gc_was_on:
                gc.enable()
        torch.cuda.current_stream().wait_stream(self.stream)
        cap = _Captured(graph, static, logits, ops.launches - before, _InputMirror(rb, widths, eng.device, eng.storage.pad_slot))
        assert cap.mirror.size == size
        self.captured[key] = cap
        return cap


class PortionGraphs:
    """CUDA graphs for steps that hold a prompt portion (alone, beside other portions, or beside decoded tokens).

    A long prompt is cut into portions of the scheduler's token budget, so the same shape (the entries' token
    counts, the number of wanted rows, the block tables' widths rounded up to a power of two) comes again and
    again. Such a step is some two hundred launches whose host side costs about as much as a tenth of the
    device's work; captured once, the third time its shape is seen, it is one launch. Everything a kernel
    reads of the step (ids, positions, lengths, wanted rows, block tables) lies in a device buffer of fixed
    address that one copy refreshes; the launch geometry depends on the shape alone (for the decoded tokens of
    a mixed step: on the power of two that bounds their contexts, as in DecodeGraphs). A shape seen once is
    never captured, and at most ``capacity`` shapes are kept. A request that decodes while a long prompt is
    fed in portions of the token budget repeats one shape step after step: n ones and a portion of budget - n."""

    def __init__(self, engine, min_tokens: int = 256, capacity: int = 8, sightings: int = 3):
        self._engine = weakref.ref(engine)
        self.min_tokens, self.capacity = min_tokens, capacity
        # A capture costs about ten eager steps' host time: a shape is captured when it is seen for the third time (a
        # prompt cut by the budget, or decoding beside one, comes dozens of times; a batch of prompts of odd lengths
        # that happens to recur once does not pay for a capture).
        self.sightings = sightings
        self.captured: Dict[tuple, _Captured] = {}
        self.seen: Dict[tuple, int] = {}
        self.refused = set()        # shapes whose capture failed
        self.pool = None
        self.stream = None

    def _key(self, entries):
        eng = self._engine()
        q_lens = tuple(len(e.tokens) for e in entries)
        if max(q_lens) < 2 or sum(q_lens) < self.min_tokens:
            return None
        widths = tuple(_bucket(max(1, max(len(e.request.tables[g]) for e in entries))) for g in range(len(eng.cache.groups)))
        n_want = sum(len(e.want) for e in entries)
        all_rows = n_want == sum(q_lens) and all(list(e.want) == list(range(len(e.tokens))) for e in entries)
        # decoded tokens: how their keys are split over CTAs is chosen for the power of two that bounds their contexts
        decode_ctx = [e.request.length + 1 for e, n in zip(entries, q_lens) if n == 1]
        cb = max(256, _bucket(max(decode_ctx))) if decode_ctx else 0
        return q_lens, widths, n_want, all_rows, cb

    def step(self, entries, token_arrays, borrow: bool):
        """(True, logits) if the step ran from a graph, (False, None) if the caller has to run it."""
        eng = self._engine()
        key = self._key(entries)
        if key is None or getattr(eng.rt.ops, "_op_events", None) is not None:     # (launches that are being timed one by one run eagerly)
            return False, None
        cap = self.captured.get(key)
        if cap is None:
            if len(self.seen) > 4096:
                self.seen.clear()
            self.seen[key] = self.seen.get(key, 0) + 1
            if self.seen[key] < self.sightings or len(self.captured) >= self.capacity or key in self.refused:
                return False, None          # the first step of a shape runs eagerly (and sets up what kernels set up on first use)
            try:
                cap = self._capture(key, entries, token_arrays)
            except RuntimeError:
                # a step that cannot be captured (memory for its pool, a part that turns out to need the host) runs
                # eagerly from now on; the caller builds the step's inputs anew
                self.refused.add(key)
                torch.cuda.synchronize()
                return False, None
        else:
            eng.build_context(entries, widths=list(key[1]), static=cap.inputs, token_arrays=token_arrays)
        cap.graph.replay()
        eng.graph_launches += cap.launches
        if cap.logits is None:
            return True, None
        return True, (cap.logits if borrow else cap.logits.clone())

    def _capture(self, key, entries, token_arrays) -> _Captured:
        eng = self._engine()
        widths = list(key[1])
        probe, _, _ = eng.build_context(entries, widths=widths, token_arrays=token_arrays)
        size = sum(v.numel() for v in (probe.token_ids, probe.positions, probe.req_index, probe.q_start,
                                       probe.ctx_lens, probe.state_slots)) + key[2] \
            + sum(t.numel() for t in probe.block_tables.values())
        static = torch.empty(size, dtype=torch.int32, device=eng.device)
        ctx, want_rows, _ = eng.build_context(entries, widths=widths, static=static, token_arrays=token_arrays)
        n_dec = sum(1 for n in key[0] if n == 1)
        ctx.host.ctx_lens[:n_dec] = [key[4]] * n_dec        # (the rows of one token come first: build_context)
        caches = eng.storage.layer_caches(ctx.block_tables)
        ops = eng.rt.ops
        torch.cuda.synchronize()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        gc_was_on = gc.isenabled()      # see DecodeGraphs._capture: nothing may be freed while a stream captures
        gc.disable()
        if self.stream is None:
            self.stream = torch.cuda.Stream()
        self.stream.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(self.stream):
                graph.capture_begin(pool=self.pool)
                try:
                    logits = eng.model.forward(ctx, caches, want_rows)
                finally:
                    graph.capture_end()
        finally:
            if gc_was_on:
                gc.enable()
        torch.cuda.current_stream().wait_stream(self.stream)
        cap = _Captured(graph, static, logits, ops.launches - before)
        self.captured[key] = cap
        return cap
