"""out = a @ W^T (+ bias): the one place that picks a matrix-product kernel.

Weights stay [out_features, in_features] as stored (crates/model/src/weights.rs:2276-2277).
Choice, in the spirit of the reference's ``matmul_pre`` (crates/model/src/lib.rs:8462-8505):

  float32 weights or activations -> gemm_tiled (true 32-bit, order-fixed accumulation)
  bf16 x bf16                    -> the tcgen05 kernel when the shape allows it,
                                    gemm_skinny for 1..4 rows otherwise,
                                    gemm_tiled as the any-shape fallback.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, name: str = ""):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.bias = bias
        self.name = name
        self.out_features, self.in_features = weight.shape

    def forward(self, a: torch.Tensor, out: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, defer: bool = False, residual: bool = False):
        """``defer``: the caller's next kernel can add up partial sums itself, so for few rows on
        the tensor-core path return ``Partials`` (32-bit split-K products + bias) instead of a
        finished tensor.  ``residual``: the result is an update of the 32-bit residual stream; a
        finished bf16-path product is then written in 32-bit too, so that what a token's residual
        receives does not lose 16 bits in steps of many rows that it keeps in steps of few."""
        M = a.shape[0]
        if defer and out is None and 0 < M <= 256 and a.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            from ..kernels import tc_gemm
            if tc_gemm.supported(a, self.weight):
                return K.Partials(tc_gemm.partials(a, self.weight), self.bias)
        if out is None:
            if residual and out_dtype is None and a.dtype == torch.bfloat16:
                out_dtype = torch.float32
            out = torch.empty((M, self.out_features), dtype=out_dtype or a.dtype, device=a.device)
        if M == 0:
            return out
        w = self.weight
        if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            from ..kernels import tc_gemm
            if tc_gemm.supported(a, w, out):
                tc_gemm.gemm(a, w, self.bias, out)
                return out
            if (M <= 16 and self.in_features % 8 == 0 and a.stride(0) % 8 == 0
                    and a.data_ptr() % 16 == 0):
                for m0 in range(0, M, 4):
                    K.gemm_skinny(a[m0:m0 + 4], w, self.bias, out[m0:m0 + 4])
                return out
        K.gemm_tiled(a, w, self.bias, out)
        return out

    def forward_swiglu(self, a: torch.Tensor, out: torch.Tensor) -> bool:
        """For a weight whose rows alternate gate_j, up_j: out[:, j] = silu(a @ gate_j) * (a @ up_j)
        inside the product kernel's epilogue.  False when that kernel cannot take it (then nothing
        was launched and the caller does product and activation separately)."""
        if a.dtype != torch.bfloat16 or self.weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            return False
        from ..kernels import tc_gemm
        if a.shape[0] == 0 or not tc_gemm.supported(a, self.weight):
            return False
        return tc_gemm.gemm_swiglu(a, self.weight, out)
