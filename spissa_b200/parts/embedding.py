"""Token embedding and output head.

Embedding: h[t,:] = E[id_t,:], no scale (crates/spissa-runtime/src/ops.rs:6-30); the
rows enter the 32-bit residual stream. Head: logits = x · Wᵀ with W either its own
tensor or the embedding table when the model ties them
(crates/spissa-runtime/src/models/llama/api.rs:176-181, :336-346); logits are 32-bit.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from .base import Part, WeightSpec
from .linear import Linear
from .registry import register_part


@register_part("embedding", "embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, prefix: str = "", weight_name: str = "weight"):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight_name = prefix + weight_name
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.weight_name].contiguous()

    def fused_fields(self):
        """What a runner that gathers the rows itself needs: the table [vocab, hidden] (bfloat16)."""
        if self.weight is None or self.weight.dtype != torch.bfloat16 or type(self) is not TokenEmbedding:
            return None
        return dict(kind="token_embedding", weight=self.weight, vocab_size=self.vocab_size, hidden_size=self.hidden_size)

    def forward(self, step) -> torch.Tensor:
        """The residual stream [T, H] (float32) of the step's tokens. An embedding that needs more than the token ids
        (positions, for a learned position table) finds it in ``step``. A token id outside the table gives a zero row
        and a fault code in the device's status word (ids that come from the host are checked there already)."""
        ids = step.tokens
        out = torch.empty(ids.shape[0], self.hidden_size, dtype=torch.float32, device=ids.device)
        K.embed_gather(self.weight, ids, out, K.status_word(ids.device))
        return out


@register_part("head", "lm_head")
class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str | None = None, prefix: str = "",
                 weight_name: str = "weight"):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tied_to = tied_to
        self.weight_name = prefix + weight_name
        self.proj = None

    def weight_specs(self):
        return [] if self.tied_to else [WeightSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.proj = Linear(tensors[self.tied_to or self.weight_name])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x, out_dtype=torch.float32)

    def fused_fields(self):
        """What a runner that computes the head itself needs: the weight [vocab, hidden] (bfloat16, contiguous)."""
        w = self.proj.weight if self.proj is not None else None
        if w is None or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.data_ptr() % 16:
            return None
        return dict(kind="linear_head", weight=w, vocab_size=self.vocab_size, hidden_size=self.hidden_size)

    def greedy(self, x: torch.Tensor, note=None):
        """The index of the largest logit of every row (int32 [rows]) without the logits, as the reference's greedy
        head keeps only (best index, best value) while it streams the rows
        (crates/spissa-runtime/src/streaming/linear_argmax.rs:13, streaming/argmax.rs:30-51): the lowest index wins
        among equal logits. None when no kernel takes these operands (the caller then asks for the logits).
        ``note``: the tokens also go into the per-slot headers (an engine's ``step_note()``)."""
        w = self.proj.weight
        if not K.head_argmax_supported(x, w):
            return None
        rows = x.shape[0]
        n_cand = K.head_argmax_candidates(rows, w.shape[0])
        cand = torch.empty(rows, n_cand, 2, dtype=torch.float32, device=x.device)
        out = torch.empty(rows, dtype=torch.int32, device=x.device)
        K.head_argmax(x, w, cand, out, note)
        return out
