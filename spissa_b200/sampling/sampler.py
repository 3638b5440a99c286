"""Choosing the next token from logits: greedy, or temperature with top-k and top-p.

Meanings follow the reference (crates/spissa-runtime/src/ops.rs:309-324 greedy, first
maximum wins; :377-430 temperature → top-k → top-p → one draw; :446-457 the uniform
number is one xorshift64* step of a seed, its top 24 bits / 2^24). Temperature ≤ 0
means greedy (ops.rs:389-391).

The reference's Llama session passes the same seed at every step
(crates/spissa-runtime/src/models/llama/session/mod.rs:686) while its Qwen session
adds the step index (crates/spissa-runtime/src/models/qwen/session.rs:189). Here the
seed of a draw is derived from (seed, request index, step), so a request draws the
same numbers alone and inside any batch.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0        # 0 = greedy
    top_k: int = 0                  # 0 = no cap
    top_p: float = 0.95             # used only when temperature > 0
    seed: int = 0

    def __post_init__(self):
        if self.temperature > 0 and not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must not be negative, got {self.top_k}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


def seeded_unit(seed: int) -> float:
    """The reference's ``seeded_unit_f32``: one xorshift64* step, top 24 bits / 2^24."""
    x = _GOLDEN if (seed & _MASK) == 0 else seed & _MASK
    x ^= x >> 12
    x ^= (x << 25) & _MASK
    x ^= x >> 27
    x = (x * 0x2545F4914F6CDD1D) & _MASK
    return float(x >> 40) / float(1 << 24)


def draw_seed(seed: int, request: int, step: int) -> int:
    """The seed of one draw: depends on the run's seed, the request's index and the step only."""
    return (seed + _GOLDEN * (request + 1) + 0xD1B54A32D192ED03 * (step + 1)) & _MASK


def uniforms(params: SamplingParams, requests, step: int) -> list:
    return [seeded_unit(draw_seed(params.seed, r, step)) for r in requests]


class Sampler:
    """Runs the sampling kernels on rows of logits that live on the device."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._scratch = None

    def sample(self, logits: torch.Tensor, params: SamplingParams, requests, step: int, note=None) -> torch.Tensor:
        """One token per row (int32 on the device). ``requests`` are the rows' request indices.

        ``note`` (an engine's ``step_note()``): the tokens are also written into the per-slot headers of the step's
        sequences on the device (last token, draw counter, position), where the next decode step can take them."""
        from ..csrc import lib as K
        rows, V = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if rows == 0:
            return out
        if params.greedy:
            K.argmax_rows(logits, out)
        else:
            need = K.sample_scratch_keys(rows, V)
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.int64, device=logits.device)
            u = torch.tensor(uniforms(params, requests, step), dtype=torch.float32).to(logits.device)
            K.sample_rows(logits, params.temperature, params.top_k, params.top_p, u, self._scratch, out)
        if note is not None:
            self.note(out, note)
        return out

    @staticmethod
    def note(tokens: torch.Tensor, note) -> None:
        from ..csrc import lib as K
        if tokens.numel() != len(note.slots):
            raise ValueError(f"{tokens.numel()} tokens cannot be noted for the {len(note.slots)} sequences of the step")
        K.header_note(note.header, note.seq_slot, note.seq_len, tokens)
        note.done()
