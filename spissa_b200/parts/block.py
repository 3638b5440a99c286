"""The pre-norm arrangement of a layer: h += mixer(norm(h)); h += ffn(norm(h)).

crates/spissa-runtime/src/models/llama/generate.rs:190-199 (norm before attention),
:459 (first residual sum), :465-471 (norm before the feed-forward), :773 (second sum).
The residual stream ``h`` is 32-bit in every mode; mixer and feed-forward add into it.
"""
from __future__ import annotations

from .base import Block
from .registry import build_part, register_part
from ..phases import phase


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, mixer, ffn, norms: dict, prefix: str = ""):
        super().__init__(prefix)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn)
        self.mixer_norm = build_part("norm", norms["mixer"])
        self.ffn_norm = build_part("norm", norms["ffn"])

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_request(self):
        return self.mixer.cache_request()

    def fused_fields(self):
        f = dict(kind="prenorm", mixer_norm=self.mixer_norm.fused_fields(), mixer=self.mixer.fused_fields(),
                 ffn_norm=self.ffn_norm.fused_fields(), ffn=self.ffn.fused_fields())
        return None if any(v is None for v in f.values()) else f

    def forward(self, h, step, cache):
        with phase("attention_norm_ms"):
            x = self.mixer_norm.forward(h)
        self.mixer.forward(x, step, cache, h)
        with phase("mlp_norm_ms"):
            x = self.ffn_norm.forward(h)
        self.ffn.forward(x, step, h)
