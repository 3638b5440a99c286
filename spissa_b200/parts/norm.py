"""RMS norm: y = x / sqrt(mean(x²) + eps) · w, statistics in 32-bit.

crates/spissa-runtime/src/ops.rs:159-179 (eps inside the root, the weight multiplies
directly, no ``1 + w``).
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Norm, WeightSpec
from .registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, prefix: str = "", weight_name: str = "weight"):
        super().__init__(prefix)
        self.size = int(size)
        self.eps = float(eps)
        self.weight_name = prefix + weight_name
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.size,), init="ones")]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.weight_name].contiguous()

    def fused_fields(self):
        if self.weight is None or self.weight.dtype != torch.bfloat16:
            return None
        return dict(kind="rmsnorm", weight=self.weight, eps=self.eps, size=self.size)

    def forward(self, h: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty(n, self.size, dtype=self.rt.act_dtype, device=h.device)
        K.rmsnorm(h, self.weight, out, self.eps, rows)
        return out
