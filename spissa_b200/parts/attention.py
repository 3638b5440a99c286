"""Causal grouped-query attention over the cache, as a mixer.

q = x·Wqᵀ, k = x·Wkᵀ, v = x·Wvᵀ (no bias); positions are applied to q and k; k and v
go to the cache at the token's position; each query head h attends, through kv head
h // (heads / kv_heads), to the visible keys of its own sequence with scores scaled by
1/√head_dim and a 32-bit softmax; the heads are projected back with Wo.
crates/spissa-runtime/src/models/llama/generate.rs:274-450,
crates/spissa-runtime/src/rotary.rs:335-415.

The three projections run as one matrix product over the stacked weight
[Wq; Wk; Wv]. With ``window`` = w a query at position p sees keys p−w+1 … p.
A run that shares another run's cache (``cache.writes`` False) computes q only and
reads the keys the other run stored; a layer built with ``shares_kv`` has no k/v
projections at all and can only run that way.
"""
from __future__ import annotations

import math

import torch

from ..csrc import lib as K
from .base import KVCacheRequest, Mixer, WeightSpec
from .linear import GEMV_TOKENS, Linear
from .registry import build_part, register_part
from ..phases import phase


def length_bucket(max_len: int, page_size: int) -> int:
    """Powers of two up to 8 pages, then steps of 8 pages, steps that double while they are under a sixteenth of
    the length: the bucket fixes how the keys are split, and a split made for a much longer bucket leaves most
    chunks empty; a capture costs tens of milliseconds, so it should not come more often than every few hundred
    steps either."""
    b = 4 * page_size
    while b < max_len and b < 8 * page_size:
        b *= 2
    if max_len <= b:
        return b
    step = 8 * page_size
    while step * 16 < max_len:
        step *= 2
    return -(-max_len // step) * step


@register_part("mixer", "attention")
class GQAAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position=None, window=None, shares_kv: bool = False, prefix: str = "", names: dict | None = None):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.shares_kv = bool(shares_kv)         # this layer has no k/v projections: it reads another run's cache
        self.scale = 1.0 / math.sqrt(self.head_dim)
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight")
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.position = build_part("position", position) if position is not None else None
        self.qkv = self.o = None

    def children(self):
        return [self.position] if self.position is not None else []

    def weight_specs(self):
        H, nh, nkv, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        own = [WeightSpec(self.names["q"], (nh * hd, H)), WeightSpec(self.names["o"], (H, nh * hd))]
        if self.shares_kv:
            return own
        return own + [WeightSpec(self.names["k"], (nkv * hd, H)), WeightSpec(self.names["v"], (nkv * hd, H))]

    def cache_request(self):
        return KVCacheRequest(self.num_kv_heads, self.head_dim, self.window)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        q = tensors[self.names["q"]]
        self.q_only = Linear(q)
        if not self.shares_kv:
            k, v = tensors[self.names["k"]], tensors[self.names["v"]]
            if not (q.dtype == k.dtype == v.dtype):
                raise ValueError(f"{self.prefix}: q, k and v projections must share a storage type")
            self.qkv = Linear(torch.cat([q, k, v], dim=0))
        self.o = Linear(tensors[self.names["o"]])
        # arrival counters of the split-key decode attention; the kernel returns them to zero
        self.counters = torch.zeros(4096, dtype=torch.int32, device=rt.device)

    def fused_fields(self):
        rotary = self.position is not None and hasattr(self.position, "rotary")
        if self.shares_kv or self.window or not rotary or self.qkv is None:
            return None
        inv_freq, rd = self.position.rotary()
        if rd != self.head_dim or self.qkv.weight.dtype != torch.bfloat16 or self.o.weight.dtype != torch.bfloat16:
            return None
        return dict(kind="gqa_rotary", qkv=self.qkv.weight, o=self.o.weight, inv_freq=inv_freq, scale=self.scale,
                    hidden_size=self.hidden_size, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                    head_dim=self.head_dim)

    def forward(self, x, step, cache, residual):
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = x.shape[0]
        writes = cache.writes
        if writes and self.shares_kv:
            raise ValueError(f"{self.prefix}: a layer without k/v projections cannot be the writer of a cache")
        rd, inv_freq = 0, None
        rotary = self.position is not None and hasattr(self.position, "rotary")
        if rotary:
            inv_freq, rd = self.position.rotary()
        q = torch.empty(T, nh * hd, dtype=self.rt.act_dtype, device=x.device)
        w = self.qkv.weight if writes else None
        if (writes and rotary and rd == hd and hd % 16 == 0 and T <= GEMV_TOKENS and q.dtype == torch.bfloat16
                and cache.k_pool.dtype == torch.bfloat16 and K.gemv_supported(x, w)):
            # a few tokens: one kernel does the QKV product, the rotation and the cache write
            with phase("qkv_projection+rotary+kv_append_ms"):
                K.gemv_qkv_rope(x, w, q, cache.k_pool, cache.v_pool, cache, inv_freq, nh, nkv, hd)
        else:
            with phase("qkv_projection_ms"):
                proj = self.qkv if writes else self.q_only
                qkv = proj(x, out_dtype=torch.float32)             # rotation reads unrounded products
                if not writes:
                    pad = torch.empty(T, (nh + 2 * nkv) * hd, dtype=torch.float32, device=x.device)
                    pad[:, :nh * hd] = qkv
                    qkv = pad
            with phase("rotary+kv_append_ms"):
                if self.position is not None and not rotary:
                    self.position.apply(qkv, step, nh, nkv, hd)
                K.rope_kv_write(qkv, q, cache.k_pool, cache.v_pool, cache, inv_freq, nh, nkv, hd, rd, write_kv=writes)
        with phase("attention_ms"):
            ctx = self.attend(q, step, cache)
        with phase("o_projection+attention_residual_ms"):
            self.o(ctx, out=residual, accumulate=True)

    def attend(self, q, step, cache):
        """The heads' outputs [T, heads·head_dim] for queries ``q`` (positions applied) over the keys and values that
        the cache holds for each token's sequence, the step's own tokens included."""
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = q.shape[0]
        ctx = torch.empty_like(q)
        if K.flash_supported(q, cache.k_pool, nh, nkv, hd, cache.page_size):
            if step.all_single:
                # the split is made for the length's bucket, not the length: a step run directly and the same step
                # replayed from a graph (captured for the bucket) then add up in the same order, bit for bit
                chunk_tiles, n_chunks = K.flash_decode_plan(T, nkv, length_bucket(step.max_len, cache.page_size),
                                                            cache.page_size)
                need = K.flash_decode_scratch_floats(T, nh, hd, n_chunks)
                scratch = torch.empty(need, dtype=torch.float32, device=q.device)
                K.flash_decode(q, cache.k_pool, cache.v_pool, ctx, cache, step.seq_len, nh, nkv, hd, self.window,
                               self.scale, chunk_tiles, n_chunks, scratch,
                               self.counters if T * nkv <= self.counters.numel() else None)
            elif T >= 256 and K.flash_tc_supported(q, cache.k_pool, nh, nkv, hd, cache.page_size, self.window):
                # long prompts: 128-token tiles on the tcgen05 tensor cores (S, P and O in tensor memory)
                tiles = K.query_tiles(step.host["new_counts"], K.flash_tc_query_tile())
                K.flash_prefill_tc(q, cache.k_pool, cache.v_pool, ctx, cache, step.seq_start, step.n_seqs, tiles,
                                   nh, nkv, hd, self.window, self.scale)
            else:
                tiles = K.query_tiles(step.host["new_counts"], K.flash_query_tile())
                K.flash_prefill(q, cache.k_pool, cache.v_pool, ctx, cache, step.seq_start, step.n_seqs,
                                tiles, nh, nkv, hd, self.window, self.scale)
        else:
            K.attention_generic(q, cache.k_pool, cache.v_pool, ctx, cache, nh, nkv, hd, self.window, self.scale)
        return ctx
