"""Arrangement of the parts in one layer."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.spec import BlockSpec
from ..registry import part_class
from .base import Part, TensorDecl


class PreNormBlock(Part):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (crates/metal/examples/qwen2_f16.rs:863-935).

    The adds are done by the norm that follows: ``forward`` receives the delta the layer
    before left pending and returns its own feed-forward delta the same way, so each
    residual add shares one pass over x with a normalisation.
    """

    def __init__(self, spec: BlockSpec):
        self.spec = spec
        p = spec.prefix
        self.mixer_norm = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = part_class("mixer", spec.mixer.kind)(spec.mixer, p)
        self.ffn_norm = part_class("norm", spec.ffn_norm.kind)(spec.ffn_norm, f"{p}.{spec.ffn_norm_name}")
        self.ffn = part_class("feed_forward", spec.ffn.kind)(spec.ffn, p)
        self._native = None                  # the native launcher of this block, made at first use

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def declare(self) -> List[TensorDecl]:
        out: List[TensorDecl] = []
        for part in self.parts():
            out += part.declare()
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.bind(tensors)

    def _native_for(self, ctx):
        """This block's native launcher if the step ``ctx`` goes that way, else None."""
        native = self._native
        if native is None:
            from .native_block import NativeBlock
            native = self._native = NativeBlock(self)
        return native if native.wants(ctx) else None

    def forward(self, ctx, x, delta, slot):
        native = self._native_for(ctx)
        if native is not None:
            # the package's own parts in a bf16 step: the whole layer in one native call (same kernels,
            # same arguments, same order as below)
            out = native.run(ctx, x, delta, slot)
            if out is not None:
                return out
        if hasattr(delta, "as_partials"):
            delta = delta.as_partials()
        h = self.mixer_norm.forward(ctx, x, delta)
        a = self.mixer.forward(ctx, h, slot)
        h = self.ffn_norm.forward(ctx, x, a)
        return self.ffn.forward(ctx, h)
