"""SwiGLU feed-forward: down( silu(x·Wgᵀ) ⊙ (x·Wuᵀ) ), silu(z) = z / (1 + e^{-z}).

crates/spissa-runtime/src/models/llama/generate.rs:590-637 (gate, up), :642-763 (down);
crates/spissa-runtime/src/ops.rs:192-194 (silu). Gate and up run as one matrix product
over the stacked weight [Wg; Wu]; the down projection adds into the residual stream.
"""
from __future__ import annotations

import torch

from .base import FeedForward, WeightSpec
from .linear import GatedLinear, Linear
from .registry import register_part
from ..phases import phase


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.gate_up = self.down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["gate"], (I, H)), WeightSpec(self.names["up"], (I, H)),
                WeightSpec(self.names["down"], (H, I))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        if g.dtype != u.dtype:
            raise ValueError(f"{self.prefix}: gate and up projections must share a storage type")
        self.gate_up = GatedLinear(g, u)
        self.down = Linear(tensors[self.names["down"]])

    def fused_fields(self):
        gu = self.gate_up
        if gu is None or not gu.block or gu.weight.dtype != torch.bfloat16 or self.down.weight.dtype != torch.bfloat16:
            return None
        return dict(kind="swiglu", gate_up=gu.weight, pair=gu.block, down=self.down.weight,
                    hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    def forward(self, x, step, residual):
        with phase("gate_projection+up_projection+activation_multiply_ms"):
            act = self.gate_up(x, self.rt.act_dtype)
        with phase("down_projection+mlp_residual_ms"):
            self.down(act, out=residual, accumulate=True)
