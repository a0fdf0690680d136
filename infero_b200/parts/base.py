"""Interfaces every part of a layer has to meet.

A part is built from its spec alone (sizes and constants are parameters), declares the
tensors it wants by name, is bound to loaded tensors, and then runs on a ``StepContext``.
No part knows which model it is in.  A part defined outside this package plugs in through
``infero_b200.registry.register_part``.

    Norm.forward(ctx, x, delta, rows=None) -> h      x float32 residual stream [T, d];
                                                     delta (or None) is added to x first
    Mixer.forward(ctx, h, slot) -> delta             h [T, d] in ctx.act_dtype; delta is a tensor or
                                                     kernels.Partials (a product left as split-K sums;
                                                     .materialize(dtype) gives the tensor)
    FeedForward.forward(ctx, h) -> delta
    PositionEncoding                                 a rotary table or an in-place rewrite of q and k
                                                     (see the class)
    Block.forward(ctx, x, delta, slot) -> delta      x updated in place; the returned delta
                                                     is added by whoever normalises next

Mixers say what they keep between steps: ``cache_spec()`` (paged keys and values) and/or
``state_spec()`` (a fixed-size array per request).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"          # matrix | embedding | norm | bias
    init: str = "normal"          # normal | ones  (random-weights mode)
    optional: bool = False


@dataclass(frozen=True)
class KvCacheSpec:
    """Paged keys and values of one cache slot.  Slots with equal specs form a group that
    shares a page allocator and block tables.  Keys and values may have different widths (a mixer
    whose values are narrower or wider than its keys, or that caches one latent vector as the
    "key" and a value of another size): the storage keeps them in two arrays."""
    num_kv_heads: int
    head_dim: int                     # width of a key
    window: Optional[int] = None      # None: every key is kept
    v_head_dim: Optional[int] = None  # width of a value; None: the same as the key's

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of one cache slot, zeroed when a request starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    def declare(self) -> List[TensorDecl]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass


class Norm(Part):
    def forward(self, ctx, x, delta, rows=None):
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> Optional[KvCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, ctx, h, slot):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h):
        raise NotImplementedError


class PositionEncoding(Part):
    """Built from a ``PositionSpec``.  One of two forms, which the mixer tells apart by the method:

    ``inv_freq(device) -> float32 [rotary_dim / 2]``: a rotary table; the mixer's fused kernel turns
    pairs (i, i + rotary_dim/2) of every head of q and k by position * inv_freq[i].

    ``apply(ctx, q, k)``: anything else; q ``[T, heads, head]`` and k ``[T, kv heads, head]`` are views
    to be rewritten in place, with ``ctx.positions`` (int32 ``[T]``) the tokens' positions."""
