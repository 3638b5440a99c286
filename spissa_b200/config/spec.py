"""The architecture-neutral description of a model that the engine builds from.

An architecture (``config/llama.py`` is one) turns its typed configuration into a
``ModelSpec``: which part stands where, with which sizes, under which checkpoint
names, and in which order the layers run. Nothing below knows an architecture's
name; parts are looked up by the ``kind`` strings in ``parts/registry.py``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: registry key, constructor parameters, checkpoint-name prefix."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""

    def with_params(self, **kw) -> "PartSpec":
        p = dict(self.params)
        p.update(kw)
        return PartSpec(self.kind, p, self.prefix)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of a mixer, a feed-forward and norms.

    ``norms`` maps the arrangement's norm places (for the pre-norm block:
    ``"mixer"`` and ``"ffn"``) to norm parts.
    """
    block: str
    mixer: PartSpec
    ffn: PartSpec
    norms: dict


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer within a step.

    ``layer`` indexes ``ModelSpec.layers``; a layer may appear in several entries.
    ``cache`` names the cache this run uses: entries with the same ``cache`` share
    it. ``writes_cache`` is False for a run that only reads a cache that an earlier
    entry of the same step has written.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    extras: dict = field(default_factory=dict)

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("a model needs a non-empty layer schedule")
        writers = {}
        for pos, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {pos} names layer {e.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"schedule entries {writers[e.cache]} and {pos} both write cache {e.cache}")
                writers[e.cache] = pos
            elif e.cache not in writers:
                raise ValueError(f"schedule entry {pos} reads cache {e.cache} before any entry writes it")


def default_schedule(n_layers: int) -> tuple:
    """Every layer once, in order, each with a cache of its own."""
    return tuple(ScheduleEntry(i, i, True) for i in range(n_layers))
