"""CUDA graphs for decode steps: one token per sequence, launch-bound when run kernel by kernel.

A graph is captured per (batch size, length bucket): the bucket (steps of 512 tokens, wider for long sequences)
fixes the width of the page tables and the way the decode attention splits the keys, so that
every launch in the graph has fixed arguments. The step's varying data (tokens, positions,
slots, lengths, page tables) live in static device buffers that are refreshed with one small
copy before each replay; page tables are copied only when they changed.

Where all layers of the step run as one kernel, that kernel reads its split of the keys from two words
among the varying data, so nothing in the graph depends on the length but the width of the page tables:
such graphs are keyed by powers of two (``wide_bucket``) and a sequence that grows from 2,000 to 4,000
tokens replays one graph all the way instead of capturing a new one every 512 tokens.
"""
from __future__ import annotations

import gc
import weakref

import torch

from .batch import StepBatch
from ..parts.attention import length_bucket  # noqa: F401  (the attention part splits the keys by it; graphs are keyed by it)


def wide_bucket(max_len: int, page_size: int) -> int:
    """The power of two (at least 4 pages) that holds ``max_len`` tokens."""
    b = 4 * page_size
    while b < max_len:
        b *= 2
    return b


class GraphTable:
    """Captured graphs by key, with a cap: when it is reached, the graph replayed longest ago makes room for the new
    one, so that a kind of step that keeps coming is never left to run kernel by kernel for the rest of the engine's
    life. A key is captured the second time it is seen (the first step of a kind warms its kernels up)."""

    def __init__(self, cap: int):
        self.cap = int(cap)
        self.graphs: dict = {}
        self.seen: dict = {}
        self.clock = 0
        self.evictions = 0

    def __len__(self):
        return len(self.graphs)

    def __iter__(self):
        return iter(self.graphs)

    def clear(self):
        self.graphs.clear()
        self.seen.clear()

    def get(self, key):
        g = self.graphs.get(key)
        if g is not None:
            self.clock += 1
            g.last_used = self.clock
        return g

    def wants_capture(self, key) -> bool:
        """Count one more sighting of ``key``; True from the second on."""
        if len(self.seen) > 8 * max(1, self.cap):
            self.seen.clear()                    # the counts are a hint only: they must not grow without bound
        n = self.seen[key] = self.seen.get(key, 0) + 1
        return n >= 2

    def put(self, key, graph, before_evict=None):
        while self.cap > 0 and len(self.graphs) >= self.cap:
            oldest = min(self.graphs, key=lambda k: getattr(self.graphs[k], "last_used", 0))
            if before_evict is not None:
                before_evict(self.graphs[oldest])
            del self.graphs[oldest]
            self.evictions += 1
        self.clock += 1
        graph.last_used = self.clock
        self.graphs[key] = graph
        return graph


class DecodeGraph:
    RING = 4

    def __init__(self, engine, n_seqs: int, bucket: int, fused=None, greedy: bool = False):
        """``fused``: the one-kernel decode runner when it takes these steps (the split of the keys is then data).
        ``greedy``: the captured step ends in the head's argmax and notes its tokens in the sequences' headers; what
        ``run`` returns is then the tokens (int32 [B]), not logits."""
        self.engine, self.B, self.bucket = weakref.proxy(engine), n_seqs, bucket      # no cycle: engines free at once
        self.fused = fused
        self.greedy = greedy
        self.noted = greedy and engine.cache.header is not None
        dev = engine.device
        B = n_seqs
        self.P = bucket // engine.page_size
        self.groups = list(engine.cache.kv_groups)
        # tokens, positions, slots, lengths, where a step's tokens lie in a device tensor, and the split of the keys
        self.n_dyn = 5 * B + 2
        self.n_tab = B * self.P
        total = self.n_dyn + self.n_tab * len(self.groups)
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.pinned = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        tables = {g: self.dev[self.n_dyn + i * self.n_tab:self.n_dyn + (i + 1) * self.n_tab].view(B, self.P)
                  for i, g in enumerate(self.groups)}
        self.batch = StepBatch(
            n_tokens=B, n_seqs=B, tokens=self.dev[0:B], positions=self.dev[B:2 * B], token_seq=ar[:B],
            seq_start=ar, seq_slot=self.dev[2 * B:3 * B], seq_row=ar[:B], seq_len=self.dev[3 * B:4 * B],
            want_rows=ar[:B], n_want=B, max_new=1, max_len=bucket, all_single=True,
            page_tables=tables, host={}, key_split=self.dev[5 * B:5 * B + 2] if fused is not None else None)
        self.last_tables = None
        self.graph = None
        self.logits = None
        self.kernels = 0

    def _upload(self, tokens, positions, slots, tables: dict, rows=None) -> None:
        """``tokens`` None: the tokens are on the device already; ``rows`` says where (see ``run``)."""
        B = self.B
        i = self.turn % self.RING
        self.turn += 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.pinned[i]
        split = self.fused.key_split(B, max(positions) + 1, self.engine.page_size) if self.fused is not None else (0, 0)
        dyn = (list(tokens) if tokens is not None else [0] * B) + list(positions) + list(slots) + \
            [p + 1 for p in positions] + (list(rows) if rows is not None else [0] * B) + list(split)
        buf[:self.n_dyn] = torch.tensor(dyn, dtype=torch.int32)
        first = 0 if tokens is not None else B      # leave the token block alone when the device fills it
        flat_tables = [tables[g] for g in self.groups]
        if flat_tables != self.last_tables:
            flat = []
            for t in flat_tables:
                for r in t:
                    flat.extend(r)
                    flat.extend([0] * (self.P - len(r)))
            buf[self.n_dyn:] = torch.tensor(flat, dtype=torch.int32)
            self.dev[first:].copy_(buf[first:], non_blocking=True)
            self.engine.h2d_bytes += (buf.numel() - first) * 4
            self.last_tables = [[list(r) for r in t] for t in flat_tables]
        else:
            self.dev[first:self.n_dyn].copy_(buf[first:self.n_dyn], non_blocking=True)
            self.engine.h2d_bytes += (self.n_dyn - first) * 4
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev

    def run(self, tokens, positions, slots, tables: dict, token_source=None, rows=None) -> torch.Tensor:
        """Logits [B, vocab] of the step; the tensor is reused by the next replay.

        With ``token_source`` (int32 on the device) the step's tokens are ``token_source[rows]`` and never
        visit the host: the sampler's output of one step feeds the next."""
        from ..csrc import lib
        if token_source is None:
            self._upload(tokens, positions, slots, tables)
        else:
            self._upload(None, positions, slots, tables, rows)
            lib.gather_i32(token_source, self.dev[4 * self.B:5 * self.B], self.dev[0:self.B])
        if self.graph is None:
            eng = self.engine
            graph = torch.cuda.CUDAGraph()
            before = lib.launches
            # Nothing but kernel launches and pool allocations happens in the captured region. The relaxed
            # mode keeps a stray runtime call of some finaliser (a pinned buffer of an old engine being
            # returned, say) from invalidating the capture; the collector is held off meanwhile as well.
            was_enabled = gc.isenabled()
            gc.collect()
            gc.disable()
            try:
                note = None
                if self.noted:
                    from .engine import StepNote
                    note = StepNote(eng.cache, eng.cache.header, [], self.batch.seq_slot, self.batch.seq_len)
                with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                    self.logits = eng.model.forward(self.batch, eng.cache, self.greedy, note)
            finally:
                if was_enabled:
                    gc.enable()
            self.kernels = lib.launches - before         # kernels the graph holds
            lib.launches = before
            self.graph = graph
        self.graph.replay()
        lib.launches += self.kernels
        return self.logits
