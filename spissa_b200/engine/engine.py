"""The engine: a model with its weights on one GPU, its cache, and ONE step function.

``Engine.step`` takes, for each sequence of a batch, the next tokens of that sequence
and the places among them whose logits are wanted; it runs only those tokens, as one
batch, against what earlier steps left in the cache, and returns the wanted logits.
The reference's step is ``append_tokens`` for its single sequence
(crates/spissa-runtime/src/models/llama/session/mod.rs:314-716: guard, embed, layers,
final norm, last row, head; position offset = cached length, :326).
"""
from __future__ import annotations

import json
import sys
from dataclasses import dataclass
from pathlib import Path

import torch

from ..cache import CacheManager
from ..cache.manager import HEADER_LAST_TOKEN, HEADER_WORDS
from ..config import load_config
from ..csrc import build as kernel_build
from ..csrc import lib as K
from ..csrc.lib import KernelError
from ..parts.base import Runtime
from ..weights import load_tensors, random_tensors
from .batch import pack_step
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class StepError(ValueError):
    """A step was refused before anything ran; the cache is unchanged."""


@dataclass
class StepEntry:
    slot: int
    tokens: list
    want: list


@dataclass
class StepNote:
    """What a sampler needs to note its tokens in the headers of the last step's sequences: ``header`` [slots, 4]
    int32 on the device, and the step's own arrays ``seq_slot`` / ``seq_len`` [B] (row b of the logits is sequence
    b). ``done()`` keeps the host's draw counters in step."""
    cache: object
    header: torch.Tensor
    slots: list
    seq_slot: torch.Tensor
    seq_len: torch.Tensor

    def done(self) -> None:
        self.cache.note_sampled(self.slots)


def _require_gpu(device) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("spissa_b200 runs on a CUDA device (B200, sm_100a) only; none is visible. "
                           "There is no CPU path.")
    return torch.device(device)


class Engine:
    """``Engine.from_folder(dir, dtype=..., max_tokens=...)`` or ``Engine.from_config(cfg, seed=...)``."""

    PAGE_SIZE = 64
    greedy_steps = True            # ``step`` and ``step_device`` take ``greedy=True`` and return tokens instead of logits

    def __init__(self, config, tensors: dict, dtype, max_tokens: int, max_seqs: int | None = None,
                 device="cuda:0", use_graphs: bool = True, fuse_decode: bool = True, fuse_prefill: bool = True):
        self.device = _require_gpu(device)
        self.config = config
        self.dtype = _DTYPES[dtype]
        self.rt = Runtime(self.device, self.dtype, self.PAGE_SIZE)
        self.model = Model(config.to_spec())
        kernel_build.prefetch(self.model.kernel_modules(self.dtype))      # in the background, while the weights go up
        self.model.fuse_decode = fuse_decode
        self.model.fuse_prefill = fuse_prefill
        with torch.cuda.device(self.device):
            self.model.bind(tensors, self.rt)
            n_pages = (max_tokens + self.PAGE_SIZE - 1) // self.PAGE_SIZE
            if max_seqs is None:
                max_seqs = max(1, min(n_pages, 256))
            self.cache = CacheManager(self.model.cache_requests(), max_tokens, max_seqs, self.PAGE_SIZE,
                                      self.dtype, self.device)
        self.vocab_size = self.model.spec.vocab_size
        self.max_position = self.model.spec.max_position
        self.steps_run = 0
        self.h2d_bytes = 0            # bytes of step arrays copied to the device so far
        # decode steps replay CUDA graphs once a (batch size, length bucket) has been seen before
        self.use_graphs = use_graphs and self.model.graph_safe()
        from .graph import GraphTable
        self.max_graphs = 24
        self._graphs = GraphTable(self.max_graphs)
        # steps launched but not yet confirmed: [(reservation, pinned copy of the status word, event)] oldest first
        self._pending: list = []
        self._status_host: list = []
        self._last_step = None
        # per-phase timings (CUDA events around kernel groups): steps then run kernel by kernel and part by part and
        # leave their phases in ``last_phases``; ``phase_totals`` adds them up until it is cleared
        self.profile_phases = False
        self.last_phases = None
        self.phase_totals: dict = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", max_tokens: int = 4096, max_seqs: int | None = None,
                    device="cuda:0", use_graphs: bool = True, fuse_decode: bool = True,
                    fuse_prefill: bool = True) -> "Engine":
        dev = _require_gpu(device)
        config = load_config(folder)
        model = Model(config.to_spec())
        kernel_build.prefetch(model.kernel_modules(_DTYPES[dtype]))       # in the background, while the weights are read
        tensors = load_tensors(folder, model.weight_specs(), dev, _DTYPES[dtype] == torch.float32)
        return cls(config, tensors, dtype, max_tokens, max_seqs, device, use_graphs, fuse_decode, fuse_prefill)

    @classmethod
    def from_config(cls, config, seed: int = 0, dtype="bfloat16", max_tokens: int = 4096,
                    max_seqs: int | None = None, device="cuda:0", std: float = 0.02,
                    norm_std: float = 0.0, use_graphs: bool = True, fuse_decode: bool = True,
                    fuse_prefill: bool = True) -> "Engine":
        """Random weights drawn on the device (no file); the same generator rule as the folder writer."""
        dev = _require_gpu(device)
        model = Model(config.to_spec())
        tensors = random_tensors(model.weight_specs(), seed, std, norm_std, torch.bfloat16, device=dev)
        if _DTYPES[dtype] == torch.float32:
            tensors = {k: (v.float() if v.is_floating_point() else v) for k, v in tensors.items()}
        return cls(config, tensors, dtype, max_tokens, max_seqs, device, use_graphs, fuse_decode, fuse_prefill)

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    @property
    def page_size(self) -> int:
        return self.cache.page_size

    @property
    def max_seqs(self) -> int:
        return self.cache.max_seqs

    def free_tokens(self) -> int:
        return self.cache.free_tokens()

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, max_new_tokens: int, sampling=None, stop_ids=None, max_batch=None,
                 on_token=None, return_logits: bool = False):
        """Generate for a list of token-id prompts; see ``engine.generate.generate``."""
        from ..sampling import Sampler, SamplingParams
        from .generate import generate as run
        if getattr(self, "_sampler", None) is None:
            self._sampler = Sampler(self.device)
        if stop_ids is None:
            stop_ids = self.config.stop_token_ids() if hasattr(self.config, "stop_token_ids") else []
        with torch.cuda.device(self.device):
            try:
                out = run(self, self._sampler, [list(p) for p in prompts], max_new_tokens,
                          sampling or SamplingParams(), stop_ids, max_batch, on_token, return_logits)
            except BaseException:
                self._abandon()
                raise
            self.check()
            return out

    # ------------------------------------------------------------------ the step as a transaction
    def _validate(self, ents) -> tuple:
        """Everything that can be refused is refused here, before anything runs. Returns (lengths, packed tokens)."""
        if not ents:
            raise StepError("a step needs at least one sequence")
        lengths = []
        packed = {}                                  # entry index -> its tokens as an int32 tensor
        for slot, toks, want in ents:
            if not toks:
                raise StepError(f"slot {slot}: a sequence of a step brings at least one token")
            if len(toks) > 32:
                # a prompt: checked as a tensor (which the packing below takes as it is)
                try:
                    as_tensor = torch.tensor(toks, dtype=torch.int64)
                except (TypeError, ValueError, RuntimeError, OverflowError):
                    raise StepError(f"slot {slot}: token ids must be integers") from None
                bad = (as_tensor < 0) | (as_tensor >= self.vocab_size)
                if bool(bad.any()):
                    t = int(as_tensor[bad][0])
                    raise StepError(f"slot {slot}: token id {t} is outside the vocabulary of {self.vocab_size}")
                packed[len(lengths)] = as_tensor.to(torch.int32)
            else:
                for t in toks:
                    if not (0 <= int(t) < self.vocab_size):
                        raise StepError(f"slot {slot}: token id {t} is outside the vocabulary of {self.vocab_size}")
            for w in want:
                if not (0 <= int(w) < len(toks)):
                    raise StepError(f"slot {slot}: wanted place {w} is outside the {len(toks)} tokens given")
            before = self.cache.length(slot)
            self._check_position(slot, before, len(toks))
            lengths.append(before)
        return lengths, packed

    def _check_position(self, slot: int, before: int, new: int) -> None:
        # the reference refuses a turn that would pass max_seq_len before anything runs
        # (crates/spissa-runtime/src/session.rs:307-320)
        if self.max_position and before + new > self.max_position:
            raise StepError(f"slot {slot}: {before} cached + {new} new tokens pass the model's "
                            f"{self.max_position} positions")

    def _begin(self, counts):
        """Reserve the step's pages (all or nothing). Models with fixed-size state keep one step in flight at most:
        its rows are copied aside first, so that a fault can put them back."""
        self._settle(wait=False)
        if self.cache.has_state():
            self._settle(wait=True)
        res = self.cache.reserve(counts)
        if self.cache.has_state():
            self.cache.checkpoint(res)
        return res

    def _launched(self, res, step_arrays) -> None:
        """The step's kernels are queued: lengths move on, and the status word is asked for behind them."""
        self.cache.advance(res)
        self._last_step = ([s for s, _ in res.counts], step_arrays[0], step_arrays[1])
        host = self._status_host.pop() if self._status_host else torch.zeros(1, dtype=torch.int32, pin_memory=True)
        host.copy_(K.status_word(self.device), non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._pending.append((res, host, event))
        self.steps_run += 1

    def _settle(self, wait: bool) -> None:
        """Confirm the steps in flight whose status has arrived (``wait``: all of them), oldest first. The first one
        whose status word is not zero ends it: that step and every later one are rolled back and ``KernelError`` is
        raised; the engine goes on from the last confirmed state."""
        while self._pending:
            res, host, event = self._pending[0]
            if not wait and not event.query():
                return
            event.synchronize()
            code = int(host[0])
            if code:
                self._fail(code)
            self.cache.confirm(res)
            self._pending.pop(0)
            self._status_host.append(host)

    def _fail(self, code: int) -> None:
        torch.cuda.synchronize(self.device)
        for res, host, _ in reversed(self._pending):
            self.cache.rollback(res)
            self._status_host.append(host)
        self._pending.clear()
        K.status_word(self.device).zero_()
        raise KernelError(f"a kernel of a step reported a fault (code {code}: {K.STATUS_TEXT.get(code, 'unknown')}); "
                          f"the step and those launched after it were rolled back")

    def _abandon(self) -> None:
        """After an error that left steps in flight whose slots were given back: forget them (nothing to roll back
        for a released sequence) and clear the status word, so that the engine can go on."""
        torch.cuda.synchronize(self.device)
        for res, host, _ in reversed(self._pending):
            if res.state in ("reserved", "advanced"):
                self.cache.rollback(res)
            self._status_host.append(host)
        self._pending.clear()
        K.status_word(self.device).zero_()

    def check(self) -> None:
        """Wait for every step launched so far and confirm it, or roll back and raise ``KernelError``. ``step`` does
        this by itself unless called with ``check=False``; ``step_device`` never does, its caller settles a step when
        it reads the step's tokens."""
        with torch.cuda.device(self.device):
            self._settle(wait=True)
            K.check_status(self.device)

    def settle(self, wait: bool = False) -> None:
        """Confirm the steps whose status has arrived; raises like ``check`` when one of them failed."""
        with torch.cuda.device(self.device):
            self._settle(wait)

    def step_note(self):
        """Where the sampler notes the tokens it chooses for the sequences of the last step: the per-slot header
        (position, draws, last token) on the device. ``step_device`` called without a token source reads them there."""
        if self._last_step is None or self.cache.header is None:
            return None
        slots, seq_slot, seq_len = self._last_step
        return StepNote(self.cache, self.cache.header, slots, seq_slot, seq_len)

    def step(self, entries, check: bool = True, greedy: bool = False) -> torch.Tensor:
        """Run the given tokens; return logits [number of wanted places, vocab] as float32 on the device.

        With ``greedy`` the result is the index of the largest logit at each wanted place instead (int32 [wanted
        places], the lowest index among equal logits): the head then keeps only the best candidate while it streams
        its rows and no logits are written. When every sequence wants exactly one place, these tokens are also noted
        in the sequences' headers (see ``step_note``).

        ``entries``: ``StepEntry`` objects or (slot, tokens, want) tuples. ``want`` holds indices into
        that entry's ``tokens``. Rows come back in the order of the entries and of their ``want``.
        Everything is checked before anything runs; a refused step leaves the cache as it was.

        The step is a transaction. With ``check`` (the default) it waits for the device's status word and
        confirms the new lengths only when no kernel reported a fault; otherwise the lengths stay, the pages it took
        go back, fixed-size state is restored and ``KernelError`` is raised: the next step runs as if this one had
        never been asked for. ``check=False`` returns without waiting; such steps are settled by the next checked
        step, by ``check()`` or ``settle()``, and until then ``length`` counts them.
        """
        ents = [(e.slot, list(e.tokens), list(e.want)) if isinstance(e, StepEntry)
                else (e[0], list(e[1]), list(e[2])) for e in entries]
        lengths, packed = self._validate(ents)
        counts = [(slot, len(toks)) for slot, toks, _ in ents]
        with torch.cuda.device(self.device):
            res = self._begin(counts)
            try:
                tables = res.tables
                one_each = all(len(w) == 1 for _, _, w in ents)
                graph = self._decode_graph(ents, lengths, greedy) if self.use_graphs and not self.profile_phases else None
                full = None
                if graph is not None:
                    try:
                        full = graph.run([t[0] for _, t, _ in ents], lengths, [s for s, _, _ in ents], tables)
                    except (RuntimeError, KernelError) as e:
                        if graph.graph is not None:
                            raise                        # a replay failed: that is a real fault
                        self._capture_refused(e)
                if full is not None:
                    arrays = (graph.batch.seq_slot, graph.batch.seq_len)
                    if one_each:
                        logits = full.clone()        # the graph's own tensor is overwritten by the next replay
                    else:
                        rows = [b for b, (_, _, w) in enumerate(ents) for _ in w]
                        logits = full[torch.tensor(rows, dtype=torch.long, device=self.device)] if rows else full[:0]
                else:
                    batch = pack_step([(sl, packed.get(i, tk), w) for i, (sl, tk, w) in enumerate(ents)], lengths,
                                      tables, self.device)
                    self.h2d_bytes += batch.h2d_bytes
                    arrays = (batch.seq_slot, batch.seq_len)
                    note = self._note_for(arrays, [s for s, _, _ in ents]) if greedy and one_each else None
                    logits = self._forward(batch, greedy, note)
            except BaseException:
                self.cache.rollback(res)
                raise
            self._launched(res, arrays)
            if greedy and one_each and (full is None or graph.noted):
                self.cache.note_sampled([s for s, _, _ in ents])
            if check:
                self._settle(wait=True)
        return logits

    def _capture_refused(self, e) -> None:
        # the capture itself was refused: run this and all later steps kernel by kernel
        print(f"[spissa_b200] CUDA graph capture failed ({type(e).__name__}: {str(e)[:120]}); "
              f"decode steps run kernel by kernel from here on", file=sys.stderr, flush=True)
        self.use_graphs = False
        self._graphs.clear()

    def _forward(self, batch, greedy, note):
        if not self.profile_phases:
            return self.model.forward(batch, self.cache, greedy, note)
        from .. import phases
        with phases.profile() as timer:
            out = self.model.forward(batch, self.cache, greedy, note)
        totals = timer.totals()
        self.last_phases = phases.summary(totals, len(self.model.spec.schedule))
        kind = "decode" if batch.all_single else "prefill"
        acc = self.phase_totals.setdefault(kind, {"steps": 0, "tokens": 0, "ms": {}})
        acc["steps"] += 1
        acc["tokens"] += batch.n_tokens
        for k, v in totals.items():
            acc["ms"][k] = acc["ms"].get(k, 0.0) + v
        return out

    def _note_for(self, arrays, slots):
        if self.cache.header is None:
            return None
        return StepNote(self.cache, self.cache.header, slots, arrays[0], arrays[1])

    def step_device(self, slots, token_source: torch.Tensor | None = None, rows=None, greedy: bool = False) -> torch.Tensor:
        """A decode step whose tokens are already on the device, so the host never waits for them: sequence i takes
        ``token_source[rows[i]]`` (int32, for instance the sampler's output of the step before) or, without a token
        source, the last token that the sampler noted in the sequence's header (see ``step_note``).

        Returns logits [len(slots), vocab] (float32), or with ``greedy`` the indices of their largest entries (int32
        [len(slots)], also noted in the headers); the tensor may be the step's own buffer and holds only
        until the next step. Token ids are not checked on the host (they come from this library's sampler); one
        outside the vocabulary makes the embedding report a fault. The step is not settled here: call ``settle``
        or ``check`` (the generation loop does when it reads a step's tokens).
        """
        slots = [int(s) for s in slots]
        if token_source is None:
            if self.cache.header is None:
                raise StepError("this cache has no header on the device to take tokens from")
            token_source = self.cache.header.view(-1)
            rows = [s * HEADER_WORDS + HEADER_LAST_TOKEN for s in slots]
        rows = [int(r) for r in rows]
        if not slots or len(rows) != len(slots):
            raise StepError("a step needs at least one sequence and one token row for each")
        if token_source.dtype != torch.int32 or token_source.dim() != 1 or not token_source.is_cuda:
            raise StepError("the token source is a one-dimensional int32 tensor on the device")
        if any(not (0 <= r < token_source.numel()) for r in rows):
            raise StepError("a token row lies outside the token source")
        lengths = [self.cache.length(s) for s in slots]
        for s, before in zip(slots, lengths):
            self._check_position(s, before, 1)
        counts = [(s, 1) for s in slots]
        ents = [(s, [0], [0]) for s in slots]
        with torch.cuda.device(self.device):
            res = self._begin(counts)
            try:
                tables = res.tables
                graph = self._decode_graph(ents, lengths, greedy) if self.use_graphs and not self.profile_phases else None
                logits = None
                if graph is not None:
                    try:
                        logits = graph.run(None, lengths, slots, tables, token_source, rows)
                        arrays = (graph.batch.seq_slot, graph.batch.seq_len)
                    except (RuntimeError, KernelError) as e:
                        if graph.graph is not None:
                            raise                        # a replay failed: that is a real fault
                        self._capture_refused(e)
                if logits is None:
                    # kernel by kernel: the packed arrays, with the tokens filled in on the device
                    batch = pack_step(ents, lengths, tables, self.device)
                    self.h2d_bytes += batch.h2d_bytes
                    idx = torch.tensor(rows, dtype=torch.int32).to(self.device)
                    K.gather_i32(token_source, idx, batch.tokens)
                    arrays = (batch.seq_slot, batch.seq_len)
                    logits = self._forward(batch, greedy, self._note_for(arrays, slots) if greedy else None)
            except BaseException:
                self.cache.rollback(res)
                raise
            self._launched(res, arrays)
            if greedy and self.cache.header is not None:
                self.cache.note_sampled(slots)
        return logits

    def _decode_graph(self, ents, lengths, greedy: bool = False):
        """The graph for this decode step, or None when the step runs kernel by kernel."""
        if any(len(t) != 1 for _, t, _ in ents):
            return None
        from .graph import DecodeGraph, length_bucket, wide_bucket
        max_len = max(lengths) + 1
        # where one kernel runs all layers and reads its split of the keys from the device, only the width of the
        # page tables depends on the length: a few wide buckets instead of one every 512 tokens
        fused = getattr(self.model, "_fused", None) or None
        if fused is not None and not fused.takes_sizes(len(ents), wide_bucket(max_len, self.page_size), self.cache):
            fused = None
        bucket = wide_bucket(max_len, self.page_size) if fused is not None else length_bucket(max_len, self.page_size)
        key = (len(ents), bucket, fused is not None, bool(greedy))
        g = self._graphs.get(key)
        if g is None:
            if not self._graphs.wants_capture(key):
                return None                      # the first step of a kind also warms every kernel up
            # an evicted graph's buffers go back to the allocator only when no replay of it is in flight any more
            g = self._graphs.put(key, DecodeGraph(self, key[0], key[1], fused, greedy),
                                 before_evict=lambda old: torch.cuda.synchronize(self.device))
        return g
