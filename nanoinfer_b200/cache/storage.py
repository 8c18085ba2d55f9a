"""Device memory of the cache: key and value pages per group and entry, and the state slots.

Layout of one entry's keys (values likewise): ``[num_pages, kv_heads, page_size, head_dim]``, so that
the ``page_size x head_dim`` tile of one kv head of one page is contiguous. The reference keeps
``[layers, blocks, n_kv, block_size, head_dim]`` in 32-bit (cpp/src/cuda/cuda_backend.cu:852-871);
here the element type is the engine's compute dtype.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, LayerCache, StateNeed
from .pages import CacheManager, GroupSpec


def plan_groups(needs: Sequence[Tuple[Optional[CacheNeed], Optional[StateNeed], Optional[int]]]):
    """Cache groups from the per-entry needs: entries with the same (kv_heads, head_dim, window)
    share a group. Returns (groups, group index of each entry or -1)."""
    keys: List[Tuple[int, int, int]] = []
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
    groups = [GroupSpec(k[0], k[1], k[2], tuple(m)) for k, m in zip(keys, members)]
    return groups, entry_group


class CacheStorage:
    def __init__(self, needs, num_pages: int, page_size: int, max_requests: int,
                 dtype: torch.dtype, device):
        self.needs = list(needs)
        self.groups, self.entry_group = plan_groups(self.needs)
        self.page_size, self.num_pages = page_size, num_pages
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        for g in self.groups:
            for e in g.entries:
                shape = (num_pages, g.kv_heads, page_size, g.head_dim)
                self.k[e] = torch.zeros(shape, dtype=dtype, device=device)
                self.v[e] = torch.zeros(shape, dtype=dtype, device=device)
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
                k_pages=self.k.get(owner), v_pages=self.v.get(owner),
                block_table=block_tables.get(g) if g >= 0 else None,
                page_size=self.page_size, writes=reads is None and need is not None,
                state=self.state.get(i)))
        return out

    def bytes_per_token(self) -> int:
        total = 0
        for g in self.groups:
            for e in g.entries:
                total += 2 * g.kv_heads * g.head_dim * self.k[e].element_size()
        return total
