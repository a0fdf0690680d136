"""Grouped-query attention over the paged cache."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config.spec import MixerSpec
from ..registry import part_class
from .base import KvCacheSpec, Mixer, TensorDecl
from .linear import Linear


class GqaAttention(Mixer):
    """q,k,v = h Wq^T + bq, ...; rotary on q and k; append k,v to the cache; causal (and
    windowed) softmax attention with kv head = head // group; delta = attn Wo^T
    (crates/model/src/lib.rs:5628-5663, :5895-5913, :5979-5993, :6996-7047).

    q, k and v are one stacked product [H*D + 2*Hkv*D, d] with a stacked bias; the reference
    stacks them only for its quantised formats (crates/model/src/weights.rs:2704-2735).  Where the
    tensors live under the block's prefix is data of the spec (``MixerSpec.names``): separate q, k, v
    or one stored [q; k; v] tensor.
    """

    def __init__(self, spec: MixerSpec, prefix: str):
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.head_dim % 2 or not (2 <= spec.head_dim <= 256):
            raise ValueError(f"head_dim {spec.head_dim} must be even and at most 256")
        self.spec = spec
        self.prefix = prefix
        self.rope = None
        if spec.position is not None:
            self.rope = part_class("position", spec.position.kind)(spec.position)
        self.qkv: Linear = None
        self.out: Linear = None
        self.names = spec.tensor_names()
        self.stored_stacked = "qkv" in self.names       # the checkpoint holds one [q; k; v] tensor

    def _n(self, role: str, what: str = "weight") -> str:
        return f"{self.prefix}.{self.names[role]}.{what}"

    def cache_spec(self) -> Optional[KvCacheSpec]:
        return KvCacheSpec(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def declare(self) -> List[TensorDecl]:
        s = self.spec
        da, dkv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        widths = {"q": da, "k": dkv, "v": dkv, "qkv": da + 2 * dkv}
        roles = ("qkv",) if self.stored_stacked else ("q", "k", "v")
        out = [TensorDecl(self._n(r), (widths[r], s.hidden)) for r in roles]
        out.append(TensorDecl(self._n("o"), (s.hidden, da)))
        if s.qkv_bias:
            out += [TensorDecl(self._n(r, "bias"), (widths[r],), role="bias") for r in roles]
        if s.out_bias:
            out.append(TensorDecl(self._n("o", "bias"), (s.hidden,), role="bias"))
        return out

    @staticmethod
    def _stack(ts):
        if len({t.dtype for t in ts}) > 1:
            ts = [t.float() for t in ts]
        return torch.cat(ts, dim=0)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        roles = ("qkv",) if self.stored_stacked else ("q", "k", "v")
        w = self._stack([tensors[self._n(r)] for r in roles])
        b = self._stack([tensors[self._n(r, "bias")] for r in roles]) if s.qkv_bias else None
        self.qkv = Linear(w, b, f"{self.prefix}.qkv")
        ob = tensors[self._n("o", "bias")] if s.out_bias else None
        self.out = Linear(tensors[self._n("o")], ob, self._n("o", "product"))

    def forward(self, ctx, h, slot):
        s = self.spec
        T = h.shape[0]
        H, Hkv, D = s.num_heads, s.num_kv_heads, s.head_dim
        qkv = self.qkv.forward(h, defer=True)                  # [T, (H + 2 Hkv) D]
        kv = ctx.kv_cache(slot.cache)                          # keys, values, group
        table = ctx.block_table(kv.group)
        rotary = self.rope is None or hasattr(self.rope, "inv_freq")
        if rotary:
            inv = self.rope.inv_freq(h.device) if self.rope is not None else ctx.zero_inv_freq(h.device)
        else:
            # a position encoding that is no rotary table: it rewrites q and k itself, and the
            # cache append runs with zero angles
            inv = ctx.zero_inv_freq(h.device)
            if isinstance(qkv, K.Partials):
                qkv = qkv.materialize(h.dtype)
            self.rope.apply(ctx, qkv[:, :H * D].unflatten(1, (H, D)),
                            qkv[:, H * D:(H + Hkv) * D].unflatten(1, (Hkv, D)))
        if isinstance(qkv, K.Partials):
            q = torch.empty((T, H * D), dtype=h.dtype, device=h.device)
            K.rope_cache_partials(qkv, q, ctx.positions, ctx.tok_entry, table, inv, kv.k, kv.v, H, Hkv, D,
                                  kv.page_size, write_cache=slot.write_cache)
        else:
            q = qkv
            K.rope_cache(qkv, ctx.positions, ctx.tok_entry, table, inv, kv.k, kv.v, H, Hkv, D,
                         kv.page_size, write_cache=slot.write_cache)
        attn = torch.empty((T, H * D), dtype=h.dtype, device=h.device)
        from ..kernels import attention as A
        A.paged_attention(ctx, q, attn, kv, table, H, Hkv, D, s.window, s.scale)
        return self.out.forward(attn, defer=True, residual=True)
