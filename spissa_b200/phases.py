"""Per-phase timings of a step, behind a flag: CUDA events around named groups of kernels.

The reference times every phase of its block with a wall clock into ``RamaTransformerPhaseTimings``
(crates/spissa-runtime/src/session.rs:14-78, filled in crates/spissa-runtime/src/models/llama/generate.rs:187-776)
and the step's other parts into ``RamaSessionPhaseTimings`` (session.rs:80-101: embedding, transformer, final norm,
head); its ``llama-test --profile-phases`` prints them (crates/spissa-cli/src/bin/llama-test.rs:25-69). Here the
phases are the launches that belong together: where one kernel does what the reference does in several phases the
names are joined (``qkv_projection+rotary+kv_append``). Off by default; a step that is profiled runs kernel by
kernel and part by part (no CUDA graph, no one-kernel decode path), because only there do the phases exist as
separate launches. Parts mark their phases with ``with phase("name"):``, which costs one comparison when nothing
is being profiled.
"""
from __future__ import annotations

from contextlib import contextmanager

import torch

_active = None


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NULL = _Null()


class PhaseTimer:
    def __init__(self):
        self.spans = []                     # (name, start event, end event) in launch order
        self.stack = []

    def totals(self) -> dict:
        """name -> milliseconds over all layers, in order of first appearance (waits for the device)."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.spans:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    def counts(self) -> dict:
        out = {}
        for name, _, _ in self.spans:
            out[name] = out.get(name, 0) + 1
        return out


class _Span:
    __slots__ = ("timer", "name", "start")

    def __init__(self, timer, name):
        self.timer, self.name = timer, name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self.timer.spans.append((self.name, self.start, end))
        return False


def phase(name: str):
    """``with phase("attention"):`` around the launches of one phase; nothing happens unless a step is being profiled."""
    if _active is None:
        return _NULL
    return _Span(_active, name)


def profiling() -> bool:
    return _active is not None


@contextmanager
def profile():
    """Collect the phases of the steps run inside: ``with profile() as t: ...; t.totals()``."""
    global _active
    before = _active
    timer = PhaseTimer()
    _active = timer
    try:
        yield timer
    finally:
        _active = before


def summary(totals: dict, layers: int) -> dict:
    """The step's phases in milliseconds with the sums the reference reports: ``transformer_ms`` (all layers),
    ``total_ms``, and ``profiled_layers``."""
    outer = ("embedding_ms", "final_norm_ms", "lm_head_ms", "sample_ms")
    inner = {k: round(v, 4) for k, v in totals.items() if k not in outer}
    out = {"embedding_ms": round(totals.get("embedding_ms", 0.0), 4),
           "transformer_ms": round(sum(inner.values()), 4),
           "transformer_detail": inner,
           "final_norm_ms": round(totals.get("final_norm_ms", 0.0), 4),
           "lm_head_ms": round(totals.get("lm_head_ms", 0.0), 4)}
    if "sample_ms" in totals:
        out["sample_ms"] = round(totals["sample_ms"], 4)
    out["total_ms"] = round(sum(totals.values()), 4)
    out["profiled_layers"] = layers
    return out
