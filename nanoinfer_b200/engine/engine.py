"""The engine: a model, its cache, and ONE step function.

``step(entries)`` takes a batch of (request, its next tokens, which of them want logits): portions
of prompts beside single decoded tokens, cut anywhere. It runs only the tokens it is given, as one
flat batch, from the cache that earlier steps left, appends their keys and values, and returns the
32-bit logits at the wanted places. Everything above it (scheduler, generation, trace replay) goes
through this one function.

The reference has three forwards instead (one request with t tokens; N requests with one token;
a ragged batch: cpp/src/model.cpp:347-561); the ragged one is the shape generalised here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.pages import CacheManager, OutOfPages, RequestCache
from ..cache.storage import CacheStorage
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig, read_config_json
from ..models.decoder import DecoderModel
from ..parts.base import HostBatch, Runtime, StepContext
from ..registry import config_from_json_dict, plan_for
from ..weights.loader import load_tensors

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class StepEntry:
    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()     # places among ``tokens`` whose logits are wanted


class Engine:
    def __init__(self, model_dir: str, engine_config: EngineConfig, ops=None):
        self.engine_config = engine_config
        self.config: ModelConfig = config_from_json_dict(read_config_json(model_dir))
        self.plan = plan_for(self.config)
        tensors = load_tensors(model_dir, self.plan)
        if ops is None:
            from ..csrc.lib import load_kernels  # fails loudly when the CUDA library cannot be had
            ops = load_kernels(engine_config.kernel_options)
        self.device = torch.device(engine_config.device)
        self.dtype = _TORCH_DTYPE[engine_config.dtype]
        self.rt = Runtime(self.device, self.dtype, ops)
        self.model = DecoderModel(self.plan, tensors, self.rt)
        self.storage = CacheStorage(self.model.cache_needs(), engine_config.resolved_num_pages(),
                                    engine_config.page_size, engine_config.max_batch, self.dtype, self.device)
        self.cache: CacheManager = self.storage.make_manager(engine_config.max_batch)
        self.vocab_size = self.plan.vocab_size
        self.max_positions = self.plan.max_position_embeddings
        self.steps_run = 0
        self.tokens_run = 0
        self.last_h2d_bytes = 0
        self.graph_launches = 0     # kernel launches replayed from captured graphs
        self._stage = None          # pinned host buffer of the step's int32 inputs
        self._stage_event = None
        self._graphs = None
        self._portion_graphs = None
        if engine_config.cuda_graphs and self.device.type == "cuda" and self.model.graph_safe():
            from .graphs import DecodeGraphs, PortionGraphs
            self._graphs = DecodeGraphs(self)
            self._portion_graphs = PortionGraphs(self)

    # ---- requests -------------------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        return self.cache.open(request_id)

    def close(self, rc: RequestCache) -> None:
        self.cache.close(rc)

    def truncate(self, rc: RequestCache, new_length: int) -> None:
        """The request forgets its positions from ``new_length`` on (to recompute them, or to decode from the same
        context again). A model whose mixers keep per-request state cannot go back."""
        if self.storage.state:
            raise ValueError("a model with per-request state cannot be truncated: the state has no history")
        self.cache.truncate(rc, new_length)

    def reset_graphs(self) -> None:
        """Forget the captured graphs; steps capture them anew (after a change of what kernels do at launch)."""
        if self._graphs is not None:
            from .graphs import DecodeGraphs, PortionGraphs
            self._old_graphs = getattr(self, "_old_graphs", []) + [self._graphs, self._portion_graphs]     # their memory pools stay alive
            self._graphs = DecodeGraphs(self)
            self._portion_graphs = PortionGraphs(self)

    def check_device(self) -> None:
        """Raises if a kernel's bounded wait ran out since the last check (the kernel then returned without
        finishing its work, and the run's results are wrong). Waits for the device: the scheduler calls it
        when a request finishes and when a run ends, trace replay before it writes logits out."""
        check = getattr(self.rt.ops, "check_device_errors", None)
        if check is not None:
            check()

    # ---- the step -------------------------------------------------------------------------
    def _check(self, entries: Sequence[StepEntry]) -> List[np.ndarray]:
        """Refuses what a step cannot run; returns every entry's token ids as an int32 array (made once: a prompt
        portion has thousands of ids, and turning a Python list into an array is the dearest thing the host does
        before the first launch; an entry whose ``tokens`` already are an int32 array costs nothing)."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        arrays = []
        for e in entries:
            if e.request.closed:
                raise ValueError(f"request {e.request.request_id!r} is closed")
            if id(e.request) in seen:
                raise ValueError(f"request {e.request.request_id!r} appears twice in one step")
            seen.add(id(e.request))
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request.request_id!r}: an entry needs at least one token")
            if e.request.length + n > self.max_positions:
                raise ValueError(
                    f"request {e.request.request_id!r}: position {e.request.length + n} exceeds the "
                    f"model's context length {self.max_positions} (max_position_embeddings)")
            first = e.tokens[0]
            if n == 1 and type(first) is int:       # a decoded token: no array arithmetic for one comparison
                in_range = 0 <= first < self.vocab_size
                ids = np.array((first,), dtype=np.int32) if in_range else None
            else:
                try:        # integers only: a float or a string is not quietly turned into an id
                    ids = np.asarray(e.tokens)
                    in_range = ids.ndim == 1 and ids.dtype.kind in "iu" and int(ids.min()) >= 0 and int(ids.max()) < self.vocab_size
                    if in_range and ids.dtype != np.int32:
                        ids = ids.astype(np.int32)
                except (OverflowError, TypeError, ValueError):      # ids of mixed kinds that no array holds
                    in_range = False
            if not in_range:
                bad = next((t for t in e.tokens if not (isinstance(t, (int, np.integer)) and 0 <= int(t) < self.vocab_size)), None)
                raise ValueError(f"token id {bad!r} outside the vocabulary 0..{self.vocab_size - 1}")
            arrays.append(ids)
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise ValueError(f"wanted place {w} outside the entry's {n} tokens")
        return arrays

    def build_context(self, entries: Sequence[StepEntry], pad_to: int = 0, widths: Optional[List[int]] = None,
                      static: Optional[torch.Tensor] = None, token_arrays: Optional[List[np.ndarray]] = None):
        """Host arrays -> one int32 device buffer -> the views a step needs.

        With ``pad_to`` the batch is padded to that many requests of one token each; a padding row holds
        no pages (its block-table row is -1, its context length 0), so kernels write nothing for it and
        its attention is empty; its state slot is the spare one that no request is ever given. ``widths`` fixes the block-table widths; ``static`` is a device buffer of
        the right size that is reused (a captured graph reads its inputs there)."""
        # Rows are laid out with the one-token entries first, whatever the caller's order: the attention sends the
        # LEADING one-token requests to the decode kernel, and a decoded token behind a prompt portion would otherwise
        # take the prefill kernel's path (right, but a tile of 128 rows for one token). The wanted rows keep the
        # caller's order, so the logits come back as asked.
        caller = list(entries)
        order = sorted(range(len(caller)), key=lambda i: len(caller[i].tokens) != 1)        # stable
        entries = [caller[i] for i in order]
        if token_arrays is not None:
            token_arrays = [token_arrays[i] for i in order]
        q_lens = [len(e.tokens) for e in entries]
        r_real = len(entries)
        r = max(r_real, pad_to)
        pad = r - r_real
        m = sum(q_lens) + pad
        ctx_lens = [e.request.length + n for e, n in zip(entries, q_lens)] + [0] * pad
        q_lens_p = q_lens + [1] * pad
        q_start = np.zeros(r + 1, dtype=np.int32)
        np.cumsum(q_lens_p, out=q_start[1:])
        if token_arrays is None:
            token_arrays = [np.asarray(e.tokens, dtype=np.int32) for e in entries]
        token_ids = np.concatenate(list(token_arrays) + [np.zeros(pad, np.int32)])
        positions = np.concatenate([np.arange(e.request.length, e.request.length + n, dtype=np.int32)
                                    for e, n in zip(entries, q_lens)] + [np.zeros(pad, np.int32)])
        req_index = np.repeat(np.arange(r, dtype=np.int32), q_lens_p)
        slots = np.asarray([e.request.slot for e in entries] + [self.storage.pad_slot] * pad, dtype=np.int32)
        row_of = {id(e): int(q_start[i]) for i, e in enumerate(entries)}
        want_list = [row_of[id(e)] + int(w) for e in caller for w in e.want]
        want = np.asarray(want_list, dtype=np.int32)
        if pad_to:      # a graph computes the logits of every row
            want = np.arange(r, dtype=np.int32)
        tables = []
        for g in range(len(self.cache.groups)):
            width = widths[g] if widths is not None else max(1, max(len(e.request.tables[g]) for e in entries))
            t = np.full((r, width), -1, dtype=np.int32)
            for i, e in enumerate(entries):
                row = e.request.tables[g]
                t[i, :len(row)] = row
            tables.append(t)
        parts = [token_ids, positions, req_index, q_start, np.asarray(ctx_lens, dtype=np.int32), slots, want]
        parts += [t.reshape(-1) for t in tables]
        flat = np.concatenate(parts) if parts else np.zeros(0, np.int32)
        dev = self._to_device(flat, static)
        views, off = [], 0
        for p in parts:
            views.append(dev[off:off + p.size])
            off += p.size
        block_tables = {g: views[7 + g].view(r, tables[g].shape[1]) for g in range(len(tables))}
        ctx = StepContext(
            num_tokens=m, token_ids=views[0], positions=views[1], req_index=views[2], q_start=views[3],
            ctx_lens=views[4], state_slots=views[5],
            host=HostBatch(q_lens=q_lens_p, ctx_lens=ctx_lens, slots=slots.tolist()),
            block_tables=block_tables, rt=self.rt,
            all_rows_wanted=(want.size == m and bool((want == np.arange(m, dtype=np.int32)).all())))
        return ctx, (views[6] if want.size else None), want_list

    def _to_device(self, flat: np.ndarray, static: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One host-to-device copy of the step's inputs, from pinned memory when the device is a GPU."""
        self.last_h2d_bytes = int(flat.nbytes)
        if self.device.type != "cuda":
            if static is not None:
                static.copy_(torch.from_numpy(flat))
                return static
            return torch.from_numpy(flat).to(self.device)
        if self._stage is None or self._stage.numel() < flat.size:
            self._stage = torch.empty(max(4096, 2 * flat.size), dtype=torch.int32).pin_memory()
            self._stage_event = torch.cuda.Event()
        else:
            self._stage_event.synchronize()      # the previous step's copy has left the buffer
        self._stage[:flat.size].numpy()[:] = flat
        dev = static if static is not None else torch.empty(flat.size, dtype=torch.int32, device=self.device)
        assert dev.numel() == flat.size
        dev.copy_(self._stage[:flat.size], non_blocking=True)
        self._stage_event.record()
        return dev

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], borrow_logits: bool = False,
             device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch. Returns logits ``[wanted, vocab]`` (float32, on the device) in the order of the
        entries and of each entry's ``want``; None if nothing is wanted. Raises ``OutOfPages`` before
        changing anything if the pools cannot hold the new tokens. With ``borrow_logits`` the result may be
        a view of a buffer that the next step overwrites (for callers that consume it at once).

        ``device_tokens`` (int32 on the device, one per entry, every entry of one token): the token ids are
        taken from there instead of from the entries, whose ids are placeholders. A caller that has sampled
        the previous step's tokens on the device can so launch the next step before it has read them."""
        token_arrays = self._check(entries)
        if device_tokens is not None:
            if any(len(e.tokens) != 1 for e in entries) or device_tokens.numel() < len(entries) \
                    or device_tokens.dtype != torch.int32 or device_tokens.device != self.device:
                raise ValueError("device_tokens: one int32 token on the engine's device per entry of one token")
        demands = [(e.request, len(e.tokens)) for e in entries]
        if not self.cache.fits(demands):
            raise OutOfPages("the step's new tokens do not fit the free cache pages")
        for rc, n in demands:
            self.cache.extend(rc, n)
        self.storage.zero_slots(self.cache.take_fresh_slots())
        if self._graphs is not None and all(n == 1 for _, n in demands) and len(entries) <= self._graphs.max_batch:
            logits = self._graphs.step(entries, borrow=borrow_logits, device_tokens=device_tokens)
            m_tokens = len(entries)
        else:
            replayed = False
            if self._portion_graphs is not None and device_tokens is None:
                replayed, logits = self._portion_graphs.step(entries, token_arrays, borrow_logits)
            if not replayed:
                ctx, want_rows, _ = self.build_context(entries, token_arrays=token_arrays)
                if device_tokens is not None:
                    ctx.token_ids[:len(entries)].copy_(device_tokens[:len(entries)], non_blocking=True)
                caches = self.storage.layer_caches(ctx.block_tables)
                logits = self.model.forward(ctx, caches, want_rows)
            m_tokens = sum(n for _, n in demands)
        for rc, n in demands:
            self.cache.commit(rc, n)
        self.steps_run += 1
        self.tokens_run += m_tokens
        return logits
