"""The cache: a slot per live sequence, keys and values per cache, state per slot.

A model's schedule names caches (``ScheduleEntry.cache``); the mixer that writes a
cache says what it needs (``KVCacheRequest`` or ``StateRequest``). Caches with the
same needs form a *group* with storage of its own:

* a KV group owns pools ``k``/``v`` [caches, pages, kv heads, page_size, head_dim] and
  a page allocator. A sequence holds ceil(len / page_size) pages of the group, taken
  when it grows and returned when its slot is released. A windowed group returns
  pages that have fallen wholly out of the window after each step.
* a state group owns ``state`` [caches, slots, *shape]; a slot's rows are zeroed when
  the slot is acquired.

* beside them every slot has a small header on the device, ``header`` [slots, 4] int32:
  position (tokens cached), draws (tokens sampled for the sequence so far), the last
  sampled token (−1: none) and a spare word. It is zeroed with the slot's state, written
  by the sampler and read by a decode step that takes its tokens from the device.

The reference keeps one append-only array per layer for its single sequence
(crates/spissa-runtime/src/rotary.rs:195-318: append checks capacity before it
changes anything, truncate undoes; a failed step truncates every layer's cache back,
crates/spissa-runtime/src/models/llama/session/mod.rs:745-771). Here all lengths live
on the host. A step is a transaction: ``reserve`` takes every page it needs or changes
nothing; ``advance`` moves the lengths once the step is launched; ``confirm`` makes that
final when the device reported no fault, ``rollback`` undoes it (lengths back, pages taken
by the reservation handed back, fixed-size state and header rows restored from the copy
that ``checkpoint`` made before the step ran).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import KVCacheRequest, StateRequest
from .slots import CacheFull, CacheMisuse, IndexPool
from .views import KVLayerView, StateLayerView


@dataclass
class SequenceState:
    slot: int
    length: int = 0
    pages: dict = field(default_factory=dict)         # kv group name -> list of pages (None = returned)
    draws: int = 0                                    # tokens sampled for this sequence (host copy of the header's word)


HEADER_WORDS = 4
HEADER_POSITION, HEADER_DRAWS, HEADER_LAST_TOKEN = 0, 1, 2


@dataclass
class Reservation:
    """One step's claim on the cache, from ``reserve`` to ``confirm`` or ``rollback``."""
    counts: list                                      # [(slot, new tokens)]
    seqs: list                                        # the sequences' records (a slot number may be reused later)
    tables: dict                                      # kv group name -> per entry the sequence's page list (returned pages as 0)
    taken: dict                                       # kv group name -> per entry how many pages this reservation added
    draws: list = field(default_factory=list)         # per entry the sequence's draw counter when the step began
    after: dict = field(default_factory=dict)         # entry -> the sequence's length once this step is in
    state: str = "reserved"                           # reserved -> advanced -> confirmed | rolled back
    checkpointed: bool = False

    def __getitem__(self, group):                     # a reservation reads like its tables
        return self.tables[group]

    def __iter__(self):
        return iter(self.tables)

    def items(self):
        return self.tables.items()


class KVGroup:
    def __init__(self, name, request: KVCacheRequest, cache_ids, n_pages, page_size, dtype, device,
                 allocate=True):
        self.name, self.request, self.cache_ids = name, request, list(cache_ids)
        self.page_size, self.n_pages = page_size, n_pages
        self.pages = IndexPool(n_pages, f"page of cache group {name}")
        shape = (len(self.cache_ids), n_pages, request.num_kv_heads, page_size, request.head_dim)
        # zeros: a masked key's weight of zero must never meet a NaN left in fresh memory
        self.k = torch.zeros(shape, dtype=dtype, device=device) if allocate else None
        self.v = torch.zeros(shape, dtype=dtype, device=device) if allocate else None
        self.index = {c: i for i, c in enumerate(self.cache_ids)}

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def bytes(self) -> int:
        return 0 if self.k is None else 2 * self.k.numel() * self.k.element_size()


class StateGroup:
    def __init__(self, name, request: StateRequest, cache_ids, n_slots, device, allocate=True):
        self.name, self.request, self.cache_ids = name, request, list(cache_ids)
        shape = (len(self.cache_ids), n_slots) + tuple(request.shape)
        self.state = torch.zeros(shape, dtype=request.dtype, device=device) if allocate else None
        # the rows as they were before the step in flight: what ``rollback`` puts back
        self.shadow = torch.zeros(shape, dtype=request.dtype, device=device) if allocate else None
        self.index = {c: i for i, c in enumerate(self.cache_ids)}


class CacheManager:
    """Slots, page accounting and storage for one model.

    ``requests``: cache id -> request of the mixer that writes it (None: no cache).
    ``max_tokens``: tokens all live sequences may hold together, each sequence rounded
    up to whole pages. ``max_seqs``: slots.
    """

    def __init__(self, requests: dict, max_tokens: int, max_seqs: int, page_size: int, dtype, device,
                 allocate: bool = True):
        if page_size <= 0 or max_tokens <= 0 or max_seqs <= 0:
            raise ValueError("page_size, max_tokens and max_seqs must be positive")
        self.page_size = page_size
        self.n_pages = (max_tokens + page_size - 1) // page_size
        self.max_seqs = max_seqs
        self.slots = IndexPool(max_seqs, "slot")
        self.seqs: dict = {}
        self.kv_groups: dict = {}
        self.state_groups: dict = {}
        self.cache_group: dict = {}
        by_need: dict = {}
        for cid, req in requests.items():
            if req is None:
                continue
            by_need.setdefault(req, []).append(cid)
        for req, cids in by_need.items():
            if isinstance(req, KVCacheRequest):
                name = f"kv{len(self.kv_groups)}" + (f"_w{req.window}" if req.window else "")
                self.kv_groups[name] = KVGroup(name, req, cids, self.n_pages, page_size, dtype, device, allocate)
            elif isinstance(req, StateRequest):
                name = f"state{len(self.state_groups)}"
                self.state_groups[name] = StateGroup(name, req, cids, max_seqs, device, allocate)
            else:
                raise TypeError(f"unknown cache request {req!r}")
            for c in cids:
                self.cache_group[c] = name
        # the per-slot header, on the device beside the state; its shadow serves ``rollback``
        self.header = None
        if allocate:
            self._fresh_header = torch.tensor([0, 0, -1, 0], dtype=torch.int32, device=device)
            self.header = self._fresh_header.repeat(max_seqs, 1).contiguous()

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.seqs[slot] = SequenceState(slot, 0, {g: [] for g in self.kv_groups})
        for g in self.state_groups.values():
            if g.state is not None:
                g.state[:, slot].zero_()
        if self.header is not None:
            self.header[slot] = self._fresh_header
        return slot

    def release(self, slot: int) -> None:
        if slot not in self.seqs:
            raise CacheMisuse(f"slot {slot} is released but not held")
        seq = self.seqs.pop(slot)
        for gname, pages in seq.pages.items():
            pool = self.kv_groups[gname].pages
            for p in pages:
                if p is not None:
                    pool.release(p)
        self.slots.release(slot)

    def length(self, slot: int) -> int:
        return self._seq(slot).length

    def draws(self, slot: int) -> int:
        return self._seq(slot).draws

    def _seq(self, slot: int) -> SequenceState:
        try:
            return self.seqs[slot]
        except KeyError:
            raise CacheMisuse(f"slot {slot} is not held") from None

    def free_tokens(self) -> int:
        """Tokens that could still be stored if given to one new sequence."""
        if not self.kv_groups:
            return 1 << 60
        return min(g.pages.free_count for g in self.kv_groups.values()) * self.page_size

    # ------------------------------------------------------------------ a step
    def reserve(self, slot_counts: list) -> Reservation:
        """Take the pages that ``[(slot, new_tokens)]`` need. All or nothing.

        The reservation's ``tables``: kv group name -> per entry the sequence's page list (returned pages as 0).
        """
        seen = set()
        for slot, n in slot_counts:
            self._seq(slot)
            if slot in seen:
                raise CacheMisuse(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n <= 0:
                raise ValueError("every sequence of a step brings at least one token")
        for g in self.kv_groups.values():
            need = sum(g.pages_for(self.seqs[s].length + n) - len(self.seqs[s].pages[g.name])
                       for s, n in slot_counts)
            if need > g.pages.free_count:
                raise CacheFull(f"cache group {g.name}: the step needs {need} more pages of {self.page_size} "
                                f"tokens, {g.pages.free_count} of {g.n_pages} are free")
        tables, taken = {}, {}
        for g in self.kv_groups.values():
            rows, added = [], []
            for s, n in slot_counts:
                seq = self.seqs[s]
                have = seq.pages[g.name]
                want = g.pages_for(seq.length + n)
                added.append(max(0, want - len(have)))
                have.extend(g.pages.acquire_many(want - len(have)))
                rows.append([p if p is not None else 0 for p in have])
            tables[g.name] = rows
            taken[g.name] = added
        seqs = [self.seqs[s] for s, _ in slot_counts]
        return Reservation([(int(s), int(n)) for s, n in slot_counts], seqs, tables, taken, [q.draws for q in seqs])

    def _live(self, res: Reservation):
        """The reservation's entries whose sequence still holds its slot (a slot may have been released since)."""
        for i, ((slot, n), seq) in enumerate(zip(res.counts, res.seqs)):
            if self.seqs.get(slot) is seq:
                yield i, seq, n

    def advance(self, res: Reservation) -> None:
        """The step is launched: lengths grow. Still undoable."""
        if res.state != "reserved":
            raise CacheMisuse(f"a reservation that is {res.state} cannot advance")
        res.after = {}
        for i, seq, n in self._live(res):
            seq.length += n
            res.after[i] = seq.length
        res.state = "advanced"

    def confirm(self, res: Reservation) -> None:
        """The step ran without a fault: windowed groups return pages no key can be read from any more."""
        if res.state != "advanced":
            raise CacheMisuse(f"a reservation that is {res.state} cannot be confirmed")
        res.state = "confirmed"
        for i, seq, _n in self._live(res):
            after = res.after.get(i, seq.length)          # later steps may be in flight: this step's own end counts
            for g in self.kv_groups.values():
                w = g.request.window
                if not w:
                    continue
                # the next query stands at ``after`` and sees keys >= after - w + 1
                first_needed = max(0, after - w + 1) // self.page_size
                pages = seq.pages[g.name]
                for i in range(min(first_needed, len(pages))):
                    if pages[i] is not None:
                        g.pages.release(pages[i])
                        pages[i] = None

    def rollback(self, res: Reservation) -> None:
        """Undo a reservation that was not confirmed: lengths back, its pages handed back, state and header rows
        as ``checkpoint`` saved them. Reservations are rolled back in the reverse of the order they were made in."""
        if res.state not in ("reserved", "advanced"):
            raise CacheMisuse(f"a reservation that is {res.state} cannot be rolled back")
        advanced = res.state == "advanced"
        res.state = "rolled back"
        restore = []
        for i, seq, n in self._live(res):
            if advanced:
                seq.length -= n
            for g in self.kv_groups.values():
                pages = seq.pages[g.name]
                for _ in range(res.taken[g.name][i]):
                    p = pages.pop()
                    if p is not None:
                        g.pages.release(p)
            seq.draws = res.draws[i]
            restore.append(seq)
        if restore and self.header is not None:
            # the header from the host's books; the token a rolled-back step led to is forgotten
            rows = torch.tensor([[q.length, q.draws, -1, 0] for q in restore], dtype=torch.int32)
            idx = torch.tensor([q.slot for q in restore], dtype=torch.long)
            self.header.index_copy_(0, idx.to(self.header.device), rows.to(self.header.device))
            if res.checkpointed:
                self._copy_state_rows([q.slot for q in restore], back=True)

    def commit(self, res) -> None:
        """``advance`` and ``confirm`` in one: for a step whose success is known when it returns."""
        self.advance(res)
        self.confirm(res)

    # ------------------------------------------------------------------ fixed-size state as part of the transaction
    def has_state(self) -> bool:
        return bool(self.state_groups)

    def checkpoint(self, res: Reservation) -> None:
        """Before the step runs: keep the fixed-size state rows of its sequences, so that ``rollback`` can put them
        back: state cannot be truncated the way a length can. (Keys and values need none: what a rolled-back step
        wrote lies beyond the lengths. The header is rewritten from the host's books.) Only one step with a
        checkpoint can be in flight: the next one would overwrite the copy."""
        if not any(g.state is not None for g in self.state_groups.values()):
            return
        self._copy_state_rows([seq.slot for _, seq, _ in self._live(res)], back=False)
        res.checkpointed = True

    def _copy_state_rows(self, slots: list, back: bool) -> None:
        idx = None
        for g in self.state_groups.values():
            if g.state is None:
                continue
            if idx is None:
                idx = torch.tensor(slots, dtype=torch.long).to(g.state.device)
            src, dst = (g.shadow, g.state) if back else (g.state, g.shadow)
            dst.index_copy_(1, idx, src.index_select(1, idx))

    def note_sampled(self, slots: list) -> None:
        """The host's copy of the header's draw counter: one more token was sampled for each of ``slots``."""
        for s in slots:
            seq = self.seqs.get(s)
            if seq is not None:
                seq.draws += 1

    # ------------------------------------------------------------------ views
    def view(self, cache_id: int, step, writes: bool):
        gname = self.cache_group.get(cache_id)
        if gname is None:
            return None
        if gname in self.kv_groups:
            g = self.kv_groups[gname]
            i = g.index[cache_id]
            return KVLayerView(g.k[i], g.v[i], step.page_tables[gname], self.page_size, step.token_seq,
                               step.positions, step.seq_row, g.request.window, writes)
        g = self.state_groups[gname]
        return StateLayerView(g.state[g.index[cache_id]], writes)

    def check(self) -> None:
        """No slot or page lost, held twice or freed twice."""
        self.slots.check()
        if sorted(self.seqs) != self.slots.held():
            raise CacheMisuse("the slots held and the sequences known differ")
        for g in self.kv_groups.values():
            g.pages.check()
            owned = [p for s in self.seqs.values() for p in s.pages[g.name] if p is not None]
            if len(owned) != len(set(owned)):
                raise CacheMisuse(f"a page of group {g.name} belongs to two sequences")
            if sorted(owned) != g.pages.held():
                raise CacheMisuse(f"pages held and pages owned differ in group {g.name}")

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.kv_groups.values())
