"""CUDA graphs for steps in which every request brings exactly one token (pure decode).

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
from typing import Dict, List, Optional, Sequence, Tuple

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


class DecodeGraphs:
    max_batch = 256

    def __init__(self, engine):
        self._engine = weakref.ref(engine)      # no reference cycle: an engine that is dropped dies at once
        self.captured: Dict[Tuple[int, int], _Captured] = {}
        self.seen = set()
        self.pool = None

    @property
    def engine(self):
        return self._engine()

    def _key(self, entries) -> Tuple[int, int, List[int]]:
        eng = self.engine
        rb = _bucket(len(entries))
        max_ctx = max(e.request.length + 1 for e in entries)
        cb = max(256, _bucket(max_ctx))
        page = eng.cache.page_size
        widths = [max(1, -(-cb // page)) for _ in eng.cache.groups]
        return rb, cb, widths

    def step(self, entries, borrow: bool = False) -> Optional[torch.Tensor]:
        eng = self.engine
        rb, cb, widths = self._key(entries)
        key = (rb, cb)
        cap = self.captured.get(key)
        if cap is None:
            if key not in self.seen:
                # the first step of a shape runs eagerly: it sets up whatever the kernels set up on first use
                self.seen.add(key)
                ctx, want_rows, _ = eng.build_context(entries)
                return eng.model.forward(ctx, eng.storage.layer_caches(ctx.block_tables), want_rows)
            cap = self._capture(key, entries, rb, cb, widths)
        _, _, want_list = eng.build_context(entries, pad_to=rb, widths=widths, static=cap.inputs)
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
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self.pool):
                logits = eng.model.forward(ctx, caches, want_rows)
        finally:
            if gc_was_on:
                gc.enable()
        cap = _Captured(graph, static, logits, ops.launches - before)
        self.captured[key] = cap
        return cap
