"""What a mixer sees of the cache during one run of its layer."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class KVLayerView:
    """Paged keys and values of one cache: pools [pages, kv heads, page_size, head_dim].

    ``page_table`` [B, P] lists, per sequence of the step, the pages that hold its
    positions 0.., in order; ``seq_row`` maps a sequence of the step to its row.
    ``token_seq`` / ``positions`` are the step's arrays, repeated here so that the
    kernels' bindings need this one object.
    """
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    page_table: torch.Tensor
    page_size: int
    token_seq: torch.Tensor
    positions: torch.Tensor
    seq_slot: torch.Tensor          # row index into page_table (the step's seq_row)
    window: Optional[int]
    writes: bool                    # False: this run only reads what another run wrote


@dataclass
class StateLayerView:
    """Fixed-size per-sequence state of one cache: ``state`` [slots, *shape].

    Row ``step.seq_slot[b]`` belongs to sequence b of the step; it is zero when the
    sequence starts.
    """
    state: torch.Tensor
    writes: bool
