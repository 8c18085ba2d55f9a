"""Device memory of the cache: the paged tensors of every entry, group by group, and the state slots.

What an entry keeps per token is a list of tensors (``CacheNeed.tensors``: keys and values for attention; a mixer
may keep keys alone, one latent, or tensors of different widths and dtypes). Layout of one of them:
``[num_pages, heads, page_size, width]``, so that the ``page_size x width`` tile of one head of one page is
contiguous. The reference keeps
``[layers, blocks, n_kv, block_size, head_dim]`` in 32-bit (cpp/src/cuda/cuda_backend.cu:852-871);
here the element type is the engine's compute dtype.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, LayerCache, StateNeed
from .pages import CacheManager, GroupSpec


def plan_groups(needs: Sequence[Tuple[Optional[CacheNeed], Optional[StateNeed], Optional[int]]]):
    """Cache groups from the per-entry needs: entries that keep the same tensors with the same window
    share a group. Returns (groups, group index of each entry or -1)."""
    keys: list = []
    members: List[List[int]] = []
    entry_group = []
    for i, (need, _state, reads) in enumerate(needs):
        if need is None:
            entry_group.append(-1)
            continue
        k = need.group_key()
        if k not in keys:
            keys.append(k)
            members.append([])
        g = keys.index(k)
        members[g].append(i)
        entry_group.append(g)
    # An entry that reads another entry's cache is in that entry's group.
    for i, (need, _state, reads) in enumerate(needs):
        if reads is not None:
            entry_group[i] = entry_group[reads]
    groups = [GroupSpec(k[1], tuple(m), k[0]) for k, m in zip(keys, members)]
    return groups, entry_group


class CacheStorage:
    def __init__(self, needs, num_pages: int, page_size: int, max_requests: int,
                 dtype: torch.dtype, device):
        self.needs = list(needs)
        self.groups, self.entry_group = plan_groups(self.needs)
        self.page_size, self.num_pages = page_size, num_pages
        self.pages: Dict[int, Dict[str, torch.Tensor]] = {}     # entry -> tensor name -> pages
        self.state: Dict[int, torch.Tensor] = {}
        for g in self.groups:
            if len({t.name for t in g.tensors}) != len(g.tensors):
                raise ValueError(f"a cache need names a tensor twice: {[t.name for t in g.tensors]}")
            for e in g.entries:
                self.pages[e] = {t.name: torch.zeros((num_pages, t.heads, page_size, t.width),
                                                     dtype=t.dtype if t.dtype is not None else dtype, device=device)
                                 for t in g.tensors}
        # One slot more than there can be requests: the padding rows of a captured decode step read and write
        # the spare slot, never a live request's state.
        self.pad_slot = max_requests
        for i, (_need, state, _reads) in enumerate(self.needs):
            if state is not None:
                self.state[i] = torch.zeros((max_requests + 1,) + tuple(state.shape), dtype=state.dtype, device=device)

    def make_manager(self, max_requests: int) -> CacheManager:
        return CacheManager(self.groups, self.num_pages, self.page_size, max_requests)

    def zero_slots(self, slots: Sequence[int]) -> None:
        """State starts at zero for a request that has just been given a slot."""
        if not slots or not self.state:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=next(iter(self.state.values())).device)
        for t in self.state.values():
            t.index_fill_(0, idx, 0)

    def layer_caches(self, block_tables: Dict[int, torch.Tensor]) -> List[LayerCache]:
        out = []
        for i, (need, _state, reads) in enumerate(self.needs):
            g = self.entry_group[i]
            owner = reads if reads is not None else i
            out.append(LayerCache(
                pages=self.pages.get(owner, {}),
                block_table=block_tables.get(g) if g >= 0 else None,
                page_size=self.page_size, writes=reads is None and need is not None,
                state=self.state.get(i)))
        return out

    def bytes_per_token(self) -> int:
        total = 0
        for per_entry in self.pages.values():
            for t in per_entry.values():
                total += t.shape[1] * t.shape[3] * t.element_size()
        return total
