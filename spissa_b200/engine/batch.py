"""The tokens of one step, flattened, with what every kernel needs to place them.

A step carries, for each of its sequences, the next tokens of that sequence (a whole
prompt, a slice of one, or a single token). All sequences' tokens lie one after
another in ``tokens``; ``token_seq`` and ``positions`` say whose they are and where
they stand. The arrays travel to the device as ONE int32 buffer and one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor            # int32 [T]
    positions: torch.Tensor         # int32 [T]   absolute position of each token
    token_seq: torch.Tensor         # int32 [T]   index of the token's sequence within the step
    seq_start: torch.Tensor         # int32 [B+1] first token of each sequence in the flat arrays
    seq_slot: torch.Tensor          # int32 [B]   slot of each sequence (row of the state areas)
    seq_row: torch.Tensor           # int32 [B]   row of each sequence in the step's page tables
    seq_len: torch.Tensor           # int32 [B]   length of each sequence after this step
    want_rows: torch.Tensor         # int32 [W]   flat indices of the tokens whose logits are wanted
    n_want: int
    max_new: int                    # most tokens any sequence brings
    max_len: int                    # longest sequence after this step
    all_single: bool                # every sequence brings exactly one token (a decode step)
    page_tables: dict = field(default_factory=dict)   # kv group name -> int32 [B, P] device tensor
    host: dict = field(default_factory=dict)          # the same arrays as Python lists, for host logic
    h2d_bytes: int = 0              # bytes this step's arrays took on their way to the device
    scratch: dict = field(default_factory=dict)       # what parts make once per step and share between layers
    key_split: Optional[torch.Tensor] = None   # int32 [2] on the device: how the one-kernel decode path splits the keys
                                               # (pages per chunk, chunks); set by a captured step, refreshed per replay


def pack_step(entries, lengths_before, kv_tables: dict, device, pinned: bool = True) -> StepBatch:
    """Build the device arrays of a step.

    ``entries``: list of (slot, tokens, want) with ``want`` positions among these tokens.
    ``lengths_before``: cached length of each entry's sequence before this step.
    ``kv_tables``: kv group name -> list (per entry) of page lists covering the new length.
    """
    B = len(entries)
    # long token lists are handled as tensors, not element by element: a prompt of thousands of tokens is packed in
    # tens of microseconds instead of a millisecond of interpreter time in front of the first kernel
    seq_start, want_rows, seq_slot, seq_len = [0], [], [], []
    tok_parts, pos_parts, seq_parts = [], [], []
    for b, ((slot, toks, want), before) in enumerate(zip(entries, lengths_before)):
        n = len(toks)
        base = seq_start[-1]
        tok_parts.append(toks if isinstance(toks, torch.Tensor) else torch.tensor(toks, dtype=torch.int32))
        pos_parts.append(torch.arange(before, before + n, dtype=torch.int32))
        seq_parts.append(torch.full((n,), b, dtype=torch.int32))
        seq_start.append(base + n)
        seq_slot.append(int(slot))
        seq_len.append(before + n)
        for w in want:
            want_rows.append(base + int(w))
    T, W = seq_start[-1], len(want_rows)
    widths = {g: max(1, max(len(p) for p in rows)) for g, rows in kv_tables.items()}
    sizes = [T, T, T, B + 1, B, B, B, W] + [B * widths[g] for g in kv_tables]
    total = sum(sizes)
    flat = torch.empty(total, dtype=torch.int32, pin_memory=pinned and torch.cuda.is_available())
    small = seq_start + seq_slot + list(range(B)) + seq_len + want_rows
    for g, rows in kv_tables.items():
        w = widths[g]
        for r in rows:
            small.extend(r)
            small.extend([0] * (w - len(r)))
    torch.cat(tok_parts + pos_parts + seq_parts + [torch.tensor(small, dtype=torch.int32)], out=flat)
    dev = flat.to(device, non_blocking=True)
    views, off = [], 0
    for s in sizes:
        views.append(dev[off:off + s])
        off += s
    page_tables = {}
    for i, g in enumerate(kv_tables):
        page_tables[g] = views[8 + i].view(B, widths[g])
    new_counts = [len(e[1]) for e in entries]
    return StepBatch(
        n_tokens=T, n_seqs=B, tokens=views[0], positions=views[1], token_seq=views[2], seq_start=views[3],
        seq_slot=views[4], seq_row=views[5], seq_len=views[6], want_rows=views[7], n_want=W,
        max_new=max(new_counts), max_len=max(seq_len), all_single=all(c == 1 for c in new_counts),
        page_tables=page_tables, h2d_bytes=total * 4,
        host=dict(seq_start=seq_start, seq_len=seq_len, new_counts=new_counts, seq_slot=seq_slot,
                  want_rows=want_rows),
    )
