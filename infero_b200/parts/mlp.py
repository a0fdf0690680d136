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
    alternating layout.  Where the tensors live under the block's prefix is data of the spec
    (``FeedForwardSpec.names``): separate gate and up, or one stored [gate; up] tensor."""

    def __init__(self, spec: FeedForwardSpec, prefix: str):
        self.spec = spec
        self.prefix = prefix
        self.gate_up: Linear = None
        self.down: Linear = None
        self.names = spec.tensor_names()
        self.stored_stacked = "gate_up" in self.names    # the checkpoint holds one [gate; up] tensor

    def _n(self, role: str) -> str:
        return f"{self.prefix}.{self.names[role]}.weight"

    def declare(self) -> List[TensorDecl]:
        d, ff = self.spec.hidden, self.spec.intermediate
        if self.stored_stacked:
            return [TensorDecl(self._n("gate_up"), (2 * ff, d)), TensorDecl(self._n("down"), (d, ff))]
        return [TensorDecl(self._n("gate"), (ff, d)), TensorDecl(self._n("up"), (ff, d)),
                TensorDecl(self._n("down"), (d, ff))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.stored_stacked:
            g, u = tensors[self._n("gate_up")].chunk(2, dim=0)
        else:
            g, u = tensors[self._n("gate")], tensors[self._n("up")]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.gate_up = Linear(torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]), None,
                              f"{self.prefix}.gate_up")
        self.down = Linear(tensors[self._n("down")], None, self._n("down"))

    def forward(self, ctx, h):
        T = h.shape[0]
        act = torch.empty((T, self.spec.intermediate), dtype=h.dtype, device=h.device)
        if not self.gate_up.forward_swiglu(h, act):
            K.swiglu(self.gate_up.forward(h, defer=True), act)
        return self.down.forward(act, defer=True, residual=True)
