"""Device arrays behind the cache manager's bookkeeping.

Per group one array [slots_in_group, 2 (k, v), num_pages, kv_heads, page_size, head_dim] in
the engine's precision (bf16, or float32 on the 32-bit path); a page id addresses the same
page in every layer of its group.  (The reference stores [kv_heads, n_slots, head_dim] f16
per layer, crates/model/src/cache.rs:171-189.)  Per state slot one array
[max_requests, *shape], allocated once so addresses never change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from ..parts.base import KvCacheSpec, StateSpec
from .manager import GroupSpec


@dataclass
class LayerKv:
    k: torch.Tensor            # [num_pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
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


class CacheStorage:
    def __init__(self, kv_specs: Dict[int, KvCacheSpec], state_specs: Dict[int, StateSpec],
                 num_pages: int, page_size: int, max_requests: int, dtype: torch.dtype, device):
        self.page_size = page_size
        self.num_pages = num_pages
        self.group_specs, self._where = group_cache_slots(kv_specs)
        self.arrays: List[torch.Tensor] = []
        for g, spec in enumerate(self.group_specs):
            n = sum(1 for s in self._where.values() if s[0] == g)
            self.arrays.append(torch.zeros((n, 2, num_pages, spec.num_kv_heads, page_size, spec.head_dim),
                                           dtype=dtype, device=device))
        # one object per cache slot for the life of the pool: what points into a pool (a descriptor kept
        # by native code) is valid exactly as long as it meets the same object
        self._layer_kv: Dict[int, LayerKv] = {
            slot: LayerKv(k=self.arrays[g][i, 0], v=self.arrays[g][i, 1], group=g, page_size=page_size)
            for slot, (g, i) in self._where.items()}
        self.states: Dict[int, torch.Tensor] = {
            slot: torch.zeros((max_requests,) + tuple(s.shape), dtype=s.dtype, device=device)
            for slot, s in state_specs.items()}

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

    def bytes_per_token(self) -> int:
        return sum(a.shape[0] * 2 * a.shape[3] * a.shape[5] * a.element_size() for a in self.arrays)
