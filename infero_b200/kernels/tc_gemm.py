"""Tensor-core (tcgen05 / TMEM / TMA) matrix product for bf16 operands."""
from __future__ import annotations

import torch


def supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return False


def gemm(a, w, bias, out) -> None:
    raise NotImplementedError
