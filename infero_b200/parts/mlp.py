"""SwiGLU feed-forward."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..config.spec import FeedForwardSpec
from .base import FeedForward, TensorDecl
from .linear import Linear


class SwiGluMlp(FeedForward):
    """delta = down(silu(gate(h)) * up(h)) (crates/model/src/lib.rs:7391-7451, :7506-7531;
    crates/kernels/src/cu/ops.cu:111-133).  gate and up are stacked into one [2*ff, d]
    matrix at bind time, rows alternating gate_j, up_j, so that one product yields each pair
    side by side: the tensor-core kernel applies the activation in its epilogue, and where it
    cannot (32-bit path, a product cut into several splits) the SwiGLU kernel takes the same
    alternating layout."""

    def __init__(self, spec: FeedForwardSpec, prefix: str):
        self.spec = spec
        self.prefix = prefix
        self.gate_up: Linear = None
        self.down: Linear = None

    def _n(self, leaf: str) -> str:
        return f"{self.prefix}.mlp.{leaf}"

    def declare(self) -> List[TensorDecl]:
        d, ff = self.spec.hidden, self.spec.intermediate
        return [TensorDecl(self._n("gate_proj.weight"), (ff, d)),
                TensorDecl(self._n("up_proj.weight"), (ff, d)),
                TensorDecl(self._n("down_proj.weight"), (d, ff))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self._n("gate_proj.weight")], tensors[self._n("up_proj.weight")]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.gate_up = Linear(torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]), None,
                              self._n("gate_up"))
        self.down = Linear(tensors[self._n("down_proj.weight")], None, self._n("down_proj"))

    def forward(self, ctx, h):
        T = h.shape[0]
        act = torch.empty((T, self.spec.intermediate), dtype=h.dtype, device=h.device)
        if not self.gate_up.forward_swiglu(h, act):
            K.swiglu(self.gate_up.forward(h, defer=True), act)
        return self.down.forward(act, defer=True)
