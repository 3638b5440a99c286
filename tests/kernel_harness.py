"""Helpers for kernel tests: a paged cache laid out by hand and plain references."""
import math
import random
from types import SimpleNamespace

import torch

from plain import llama_plain as P

PAGE = 64


def paged_meta(new_counts, lengths_before, device, seed=0, page=PAGE, spare_pages=3):
    """Step arrays and a page table with shuffled pages for sequences that bring ``new_counts`` tokens."""
    rng = random.Random(seed)
    B = len(new_counts)
    total_len = [b + n for b, n in zip(lengths_before, new_counts)]
    n_pages = sum((t + page - 1) // page for t in total_len) + spare_pages
    order = list(range(n_pages))
    rng.shuffle(order)
    rows, it = [], iter(order)
    for t in total_len:
        rows.append([next(it) for _ in range((t + page - 1) // page)])
    width = max(len(r) for r in rows)
    table = torch.tensor([r + [0] * (width - len(r)) for r in rows], dtype=torch.int32, device=device)
    token_seq, positions = [], []
    for b, (before, n) in enumerate(zip(lengths_before, new_counts)):
        token_seq += [b] * n
        positions += list(range(before, before + n))
    meta = SimpleNamespace(
        token_seq=torch.tensor(token_seq, dtype=torch.int32, device=device),
        positions=torch.tensor(positions, dtype=torch.int32, device=device),
        seq_slot=torch.arange(B, dtype=torch.int32, device=device),
        page_table=table, page_size=page, n_pages=n_pages, rows=rows, total_len=total_len, new_counts=list(new_counts),
        seq_len=torch.tensor(total_len, dtype=torch.int32, device=device),
        seq_start=torch.tensor([0] + list(torch.tensor(new_counts).cumsum(0)), dtype=torch.int32, device=device))
    return meta


def fill_cache(meta, k_seqs, v_seqs, nkv, hd, dtype, device, junk=1e4):
    """Pools [pages, nkv, page, hd] holding each sequence's keys/values [len, nkv, hd]; the rest is junk."""
    k_pool = torch.full((meta.n_pages, nkv, meta.page_size, hd), junk, dtype=dtype, device=device)
    v_pool = torch.full((meta.n_pages, nkv, meta.page_size, hd), -junk, dtype=dtype, device=device)
    for b, (k, v) in enumerate(zip(k_seqs, v_seqs)):
        for pos in range(k.shape[0]):
            pg, off = meta.rows[b][pos // meta.page_size], pos % meta.page_size
            k_pool[pg, :, off, :] = k[pos].to(dtype)
            v_pool[pg, :, off, :] = v[pos].to(dtype)
    return k_pool, v_pool


def plain_attention_rows(q_seqs, k_seqs, v_seqs, new_counts, window=None):
    """For each sequence the attention rows of its last ``new_counts[b]`` positions, concatenated."""
    out = []
    for q, k, v, n in zip(q_seqs, k_seqs, v_seqs, new_counts):
        full = P.causal_attention(q.double(), k.double(), v.double(), window=window)
        out.append(full[-n:])
    return torch.cat(out, 0)
