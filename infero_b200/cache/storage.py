"""Device arrays behind the cache manager's bookkeeping.

Per group two arrays, keys [slots_in_group, pages, kv_heads, page_size, key width] and values
[slots_in_group, pages, kv_heads, page_size, value width], in the engine's precision (bf16, or
float32 on the 32-bit path); a page id addresses the same page in every layer of its group.
(The reference stores [kv_heads, n_slots, head_dim] f16 per layer, crates/model/src/cache.rs:171-189.)
Every group has a pool of its own, and the pools differ in size: a group that keeps every key gets
the pages the engine was given, a group that keeps a window of W keys only what its live requests can
ever hold at once (``plan_group_pages``), so the pages a window has passed are memory that was never
allocated.  Each array holds one page more than its pool: the page that the entries padding a captured
step read and write.  Per state slot one array [max_requests, *shape], allocated once so addresses never
change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KvCacheSpec, StateSpec
from .manager import GroupSpec


@dataclass
class LayerKv:
    k: torch.Tensor            # [pages, kv_heads, page_size, key width]
    v: torch.Tensor            # [pages, kv_heads, page_size, value width]
    group: int
    page_size: int


def group_cache_slots(kv_specs: Dict[int, KvCacheSpec]) -> Tuple[List[KvCacheSpec], Dict[int, Tuple[int, int]]]:
    """Group cache slots by spec.  Returns the group specs and slot -> (group, index in group)."""
    groups: List[KvCacheSpec] = []
    where: Dict[int, Tuple[int, int]] = {}
    counts: List[int] = []
    for slot in sorted(kv_specs):
        spec = kv_specs[slot]
        if spec not in groups:
            groups.append(spec)
            counts.append(0)
        g = groups.index(spec)
        where[slot] = (g, counts[g])
        counts[g] += 1
    return groups, where


def window_pool_pages(window: int, page_size: int, max_requests: int, max_batch_tokens: int) -> int:
    """Pages that a group with a window of ``window`` keys can ever hold at once.  A request at length L
    that brings n tokens holds the pages covering positions L - W + 1 .. L + n - 1 (everything before
    went back when the step before was committed): at most ceil(W / P) + ceil(n / P) + 2 pages.  Over
    ``max_requests`` live requests whose portions add up to at most ``max_batch_tokens``:"""
    P = page_size
    return max_requests * (-(-window // P) + 3) + -(-max_batch_tokens // P)


def plan_group_pages(group_specs: Sequence[KvCacheSpec], num_pages: int, page_size: int, max_requests: int,
                     max_batch_tokens: int) -> List[int]:
    """Pool size per group: ``num_pages`` where every key is kept, the window bound (if smaller) elsewhere."""
    out = []
    for s in group_specs:
        if s.window:
            out.append(min(num_pages, window_pool_pages(int(s.window), page_size, max_requests, max_batch_tokens)))
        else:
            out.append(num_pages)
    return out


class CacheStorage:
    def __init__(self, kv_specs: Dict[int, KvCacheSpec], state_specs: Dict[int, StateSpec],
                 pages_per_group, page_size: int, max_requests: int, dtype: torch.dtype, device):
        """``pages_per_group``: one count per group (or one int for all), the pad page included."""
        self.page_size = page_size
        self.group_specs, self._where = group_cache_slots(kv_specs)
        if isinstance(pages_per_group, int):
            pages_per_group = [pages_per_group] * len(self.group_specs)
        self.pages_per_group = [int(n) for n in pages_per_group]
        assert len(self.pages_per_group) == len(self.group_specs)
        self.k_arrays: List[torch.Tensor] = []
        self.v_arrays: List[torch.Tensor] = []
        for g, spec in enumerate(self.group_specs):
            n = sum(1 for s in self._where.values() if s[0] == g)
            shape = (n, self.pages_per_group[g], spec.num_kv_heads, page_size)
            self.k_arrays.append(torch.zeros(shape + (spec.head_dim,), dtype=dtype, device=device))
            self.v_arrays.append(torch.zeros(shape + (spec.value_dim,), dtype=dtype, device=device))
        # one object per cache slot for the life of the pool: what points into a pool (a descriptor kept
        # by native code) is valid exactly as long as it meets the same object
        self._layer_kv: Dict[int, LayerKv] = {
            slot: LayerKv(k=self.k_arrays[g][i], v=self.v_arrays[g][i], group=g, page_size=page_size)
            for slot, (g, i) in self._where.items()}
        self.states: Dict[int, torch.Tensor] = {
            slot: torch.zeros((max_requests,) + tuple(s.shape), dtype=s.dtype, device=device)
            for slot, s in state_specs.items()}

    @property
    def arrays(self) -> List[torch.Tensor]:
        """Every device array of keys and values (keys of group 0, values of group 0, keys of group 1, ...)."""
        return [a for pair in zip(self.k_arrays, self.v_arrays) for a in pair]

    def bookkeeping_groups(self) -> List[GroupSpec]:
        return [GroupSpec(window=s.window) for s in self.group_specs]

    def layer_kv(self, slot: int) -> LayerKv:
        return self._layer_kv[slot]

    def state(self, slot: int) -> torch.Tensor:
        return self.states[slot]

    def zero_state(self, request_slot: int) -> None:
        for t in self.states.values():
            t[request_slot].zero_()

    def bytes(self) -> int:
        return sum(a.numel() * a.element_size() for a in self.arrays) + \
            sum(a.numel() * a.element_size() for a in self.states.values())

    def bytes_per_token(self, group: Optional[int] = None) -> int:
        """Bytes of keys and values one token takes in all layers (of one group, or of all)."""
        return sum(a.shape[0] * a.shape[2] * a.shape[4] * a.element_size()
                   for g, (k, v) in enumerate(zip(self.k_arrays, self.v_arrays)) if group in (None, g)
                   for a in (k, v))
