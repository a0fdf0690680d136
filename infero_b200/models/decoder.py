"""A decoder assembled from a ``ModelSpec``: embedding, a schedule of blocks, final norm, head.

Nothing here is specific to one architecture.  The order in which layers run is the
spec's ``schedule`` (a block may appear twice; an entry may read the cache another entry
fills).  The reference's fixed loop is crates/model/src/lib.rs:3899-3949; the final norm
runs only on the rows whose logits are wanted (:4044-4058) and the head product always
returns 32-bit logits (:4075-4214).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config.spec import ModelSpec
from ..parts.base import KvCacheSpec, StateSpec, TensorDecl
from ..parts.linear import Linear
from ..registry import part_class


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
        self.spec = spec
        self.blocks = [part_class("block", b.kind)(b) for b in spec.blocks]
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, spec.final_norm_name)
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None
        self._native = None                  # the native launcher of a whole step, made at first use
        for e in spec.schedule:
            if not (0 <= e.block < len(self.blocks)):
                raise ValueError(f"schedule names block {e.block}, model has {len(self.blocks)}")
        self._check_cache_slots()

    # ---- what each cache slot holds ----------------------------------------------------
    def _check_cache_slots(self) -> None:
        self.kv_specs: Dict[int, KvCacheSpec] = {}
        self.state_specs: Dict[int, StateSpec] = {}
        writers = set()
        for e in self.spec.schedule:
            mixer = self.blocks[e.block].mixer
            cs, ss = mixer.cache_spec(), mixer.state_spec()
            if cs is not None:
                if e.cache in self.kv_specs and self.kv_specs[e.cache] != cs:
                    raise ValueError(f"cache slot {e.cache} is used with two different layouts")
                self.kv_specs[e.cache] = cs
                if e.write_cache:
                    if e.cache in writers:
                        raise ValueError(f"cache slot {e.cache} is written by two schedule entries")
                    writers.add(e.cache)
            if ss is not None:
                if e.cache in self.state_specs and self.state_specs[e.cache] != ss:
                    raise ValueError(f"state slot {e.cache} is used with two different shapes")
                self.state_specs[e.cache] = ss
        for c in self.kv_specs:
            if c not in writers:
                raise ValueError(f"cache slot {c} is read but never written")

    # ---- weights ---------------------------------------------------------------------------
    def declare(self) -> List[TensorDecl]:
        s = self.spec
        out = [TensorDecl(s.embed_name, (s.vocab_size, s.hidden), role="embedding")]
        for b in self.blocks:
            out += b.declare()
        out += self.final_norm.declare()
        if not s.tie_embeddings:
            out.append(TensorDecl(s.head_name, (s.vocab_size, s.hidden)))
        seen = set()
        for d in out:
            if d.name in seen:
                raise ValueError(f"tensor '{d.name}' is declared twice")
            seen.add(d.name)
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed = tensors[s.embed_name].contiguous()
        for b in self.blocks:
            b.bind(tensors)
        self.final_norm.bind(tensors)
        # a tied head aliases the embedding (crates/model/src/weights.rs:2835-2849)
        self.head = Linear(self.embed if s.tie_embeddings else tensors[s.head_name], None, "lm_head")

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embed)
        add(self.head.weight)
        for b in self.blocks:
            for part in b.parts():
                for v in vars(part).values():
                    if isinstance(v, Linear):
                        add(v.weight)
                        add(v.bias)
                    elif isinstance(v, torch.Tensor):
                        add(v)
        add(self.final_norm.weight)
        return total

    # ---- one pass over the tokens of a step -------------------------------------------------
    def forward(self, ctx, token_ids: torch.Tensor, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """token_ids int32 [T] on the device; logit_rows int32 [R] (indices into the T tokens)
        or None.  Returns float32 logits [R, vocab], or None when no row is wanted."""
        s = self.spec
        native = self._native
        if native is None:
            from .native_decoder import NativeDecoder
            native = self._native = NativeDecoder(self)
        out = native.run(ctx, token_ids, logit_rows)      # the whole step in one native call, where it applies
        if out is not NotImplemented:
            return out
        T = token_ids.numel()
        x = torch.empty((T, s.hidden), dtype=torch.float32, device=token_ids.device)
        K.embed_gather(self.embed, token_ids, x, s.embed_scale, getattr(ctx, "device_tokens", None))
        delta = None
        for i, entry in enumerate(s.schedule):
            # a block may look at what runs after it (the built-in block folds the next block's first norm
            # into its own last product when that block is of its kind)
            nxt = s.schedule[i + 1] if i + 1 < len(s.schedule) else None
            ctx.upcoming = (self.blocks[nxt.block], nxt) if nxt is not None else None
            delta = self.blocks[entry.block].forward(ctx, x, delta, entry)
        ctx.upcoming = None
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        h = self.final_norm.forward(ctx, x, delta, rows=logit_rows)
        logits = self.head.forward(h, out_dtype=torch.float32)
        if s.logit_scale != 1.0:
            logits.mul_(s.logit_scale)
        return logits
