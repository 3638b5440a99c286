"""y = x · Wᵀ with W stored [out, in] (crates/spissa-runtime/src/ops.rs:62-105).

``Linear`` holds one weight matrix and picks the kernel for a call by the operands'
storage types and sizes. The 32-bit path always uses the FFMA kernel.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is a matrix [out, in]")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype=None,
                 accumulate: bool = False) -> torch.Tensor:
        """``accumulate`` adds the product into ``out`` (float32) instead of overwriting it."""
        if out is None:
            if accumulate:
                raise ValueError("accumulation needs the tensor to add into")
            out = torch.empty(x.shape[0], self.out_features, dtype=out_dtype or x.dtype, device=x.device)
        K.gemm_generic(x, self.weight, out, accumulate=accumulate)
        return out
