"""Rotary position encoding, NeoX pairing."""
from __future__ import annotations

import numpy as np
import torch

from ..config.spec import PositionSpec
from .base import PositionEncoding


class RopeNeox(PositionEncoding):
    """inv_freq[i] = theta^(-2i / rotary_dim), i < rotary_dim/2; angle = pos * inv_freq[i]
    (crates/kernels/src/cu/ops.cu:488-523).  The table is made on the host in 64-bit and
    rounded once to 32-bit; the kernel multiplies by the position and takes sincosf."""

    def __init__(self, spec: PositionSpec):
        self.spec = spec
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        half = spec.rotary_dim // 2
        inv = np.float64(spec.theta) ** (-2.0 * np.arange(half, dtype=np.float64) / spec.rotary_dim)
        self._inv_host = torch.from_numpy(inv.astype(np.float32))
        self._inv_dev = {}

    def inv_freq(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._inv_dev:
            self._inv_dev[key] = self._inv_host.to(device)
        return self._inv_dev[key]
