"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config.spec import NormSpec
from .base import Norm, TensorDecl


class RmsNorm(Norm):
    """h = v * rsqrt(mean(v^2) + eps) * w with v = x (+ delta), all in 32-bit
    (crates/kernels/src/cu/ops.cu:44-62; fused add as in cu/mmvq.cu:761)."""

    def __init__(self, spec: NormSpec, weight_name: str):
        self.spec = spec
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.weight_name, (self.spec.dim,), role="norm", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, ctx, x, delta, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.dim), dtype=ctx.act_dtype, device=x.device)
        K.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows)
        return out
