"""Interfaces of the parts a model is put together from.

A part knows its own sizes and constants (constructor parameters), the checkpoint
names and shapes of its weights (``weight_specs``) and how to run on the tokens of
one step (``forward``). It does not know which model it is in, which layer it is,
or how the step was batched beyond what ``StepBatch`` tells every part.

Interfaces (duck-typed; the base classes hold the shared plumbing only):

* ``Norm.forward(h, rows=None) -> x``: ``h`` is the 32-bit residual stream [T, H];
  returns the normed rows in the activation dtype. ``rows`` (int32 device tensor)
  selects rows.
* ``PositionEncoding``: either exposes ``rotary()`` -> (inv_freq tensor, rotary_dim)
  so that the attention mixer can rotate while it writes the cache, or implements
  ``apply(qkv, step, num_heads, num_kv_heads, head_dim)`` which changes q and k in
  place.
* ``Mixer.cache_request()`` -> ``KVCacheRequest`` | ``StateRequest`` | None, and
  ``Mixer.forward(x, step, cache, residual)``: reads the normed ``x`` [T, H], ADDS its
  result into ``residual`` (32-bit, [T, H]) in place. ``cache`` is the view of this
  run's cache (``cache.views.KVLayerView`` / ``StateLayerView``) or None.
* ``FeedForward.forward(x, step, residual)``: same contract without a cache.
* ``Block.forward(h, step, cache)``: runs one layer on the residual stream in place.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part expects in the checkpoint."""
    name: str                 # full checkpoint name
    shape: tuple
    kind: str = "float"       # "float" (bfloat16 / float32 storage) or "int" (kept as int32)
    init: str = "normal"      # random-weights mode: "normal" = N(0, std), "ones" = norm weight


@dataclass(frozen=True)
class KVCacheRequest:
    """Keys and values of every visible position; ``window`` None means all of them."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A fixed-size state per sequence, zeroed when a sequence starts."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What the engine tells every part once: where and in which precision it runs.

    ``act_dtype`` is the storage type of activations between kernels and of the
    cache: bfloat16 in the serving mode, float32 in the true 32-bit mode.
    """
    device: torch.device
    act_dtype: torch.dtype
    page_size: int = 64

    @property
    def full_precision(self) -> bool:
        return self.act_dtype == torch.float32


class Part:
    """Shared plumbing: the weight list, and taking bound tensors.

    ``graph_safe``: the part's ``forward`` only launches work whose arguments live on the
    device (nothing is read from ``step.host``), so a decode step may be captured in a CUDA
    graph. The built-in parts say True; a part that does not say so makes its model run
    kernel by kernel.
    """
    graph_safe = False

    def fused_fields(self):
        """What a kernel that runs several parts at once needs of this part (tensors, sizes, constants), as a
        dict with a ``kind`` entry, or None when this part must run by its own ``forward`` (the default).
        Called after ``bind``. A part never has to offer this; offering it changes no result."""
        return None

    def __init__(self, prefix: str = ""):
        self.prefix = prefix
        self.rt: Optional[Runtime] = None

    def weight_specs(self) -> list:
        return []

    def bind(self, tensors: dict, rt: Runtime) -> None:
        """Take this part's tensors (already on the device, in their storage dtype)."""
        self.rt = rt

    def children(self) -> list:
        return []

    def all_weight_specs(self) -> list:
        out = list(self.weight_specs())
        for c in self.children():
            out.extend(c.all_weight_specs())
        return out

    def bind_all(self, tensors: dict, rt: Runtime) -> None:
        self.bind(tensors, rt)
        for c in self.children():
            c.bind_all(tensors, rt)


class Norm(Part):
    pass


class PositionEncoding(Part):
    pass


class Mixer(Part):
    def cache_request(self):
        return None


class FeedForward(Part):
    pass


class Block(Part):
    pass
