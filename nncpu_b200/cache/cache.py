"""The cache of a session: a slot per sequence, keys and values per layer in
pages, and fixed-size state per sequence.

* A **slot** is one sequence's place: its length, its page tables and its row
  in every state area.  Slots are handed out when a batch starts and given
  back when its sequences end; the next batch uses them again.
* Keys and values live in **pages** of ``PAGE`` tokens.  Schedule entries
  whose mixers ask for the same (KV heads, head size, window) form a **group**
  with storage, page pool and page tables of its own, so a group that needs
  every key and a group that needs only a window of them do not share a
  shape or a lifetime: a windowed group gives pages back as soon as no later
  query can see them.  An entry that reads another entry's cache owns nothing.
* **State** is a tensor ``[n_slots + 1, *shape]`` per entry that asks for one; a
  sequence that starts (length 0) starts with zeros.  The last row belongs to
  no sequence: the padding rows of a captured decode step carry slot -1, which
  indexes it, so a part may read and write "its" state for them unconditionally.

The reference keeps one sequence per cache (crates/nncpu/src/model/kv.rs:133-180):
per-layer buffers, ring buffers for sliding layers
(crates/nncpu/src/model/kv.rs:259-290), layers that read another layer's cache
and own nothing (crates/nncpu/src/model/kv.rs:272-275), and a recurrent-state
area cleared at position 0 (crates/nncpu/src/model/forward.rs:887-891).  Slots
and pages are this library's way of holding a batch of such sequences.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import ContextFull, InvalidArgument, translating_oom
from .slots import IndexPool

PAGE = 64  # tokens per page; also the unit in which a request's tokens are counted


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


@dataclass(frozen=True)
class KVRequest:
    """Keys and values of ``n_kv_heads`` heads of ``head_dim`` lanes for every
    position (``window`` 0) or for the last ``window`` positions."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """A tensor of ``shape`` per sequence, kept from step to step."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class KVGroup:
    """Storage and page bookkeeping of the entries that share one KVRequest."""

    def __init__(self, request: KVRequest, entries: List[int], n_pages: int, dtype, device):
        self.request = request
        self.entries = list(entries)
        self.n_pages = n_pages
        shape = (len(entries), n_pages, request.n_kv_heads, PAGE, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pool = IndexPool(n_pages, "cache page")
        self.tables: Dict[int, List[int]] = {}  # slot -> page ids by page index, -1 = given back

    def first_needed_page(self, length: int) -> int:
        """Pages below this index hold no key that a query at position
        ``length`` or later can see."""
        w = self.request.window
        if w <= 0 or length + 1 <= w:
            return 0
        return (length + 1 - w) // PAGE

    def pages_missing(self, slot: int, new_len: int) -> int:
        return max(0, pages_for(new_len) - len(self.tables.get(slot, ())))

    def grow(self, slot: int, new_len: int) -> None:
        table = self.tables.setdefault(slot, [])
        while len(table) < pages_for(new_len):
            table.append(self.pool.take())

    def trim(self, slot: int, length: int) -> None:
        table = self.tables.get(slot, [])
        for i in range(min(self.first_needed_page(length), len(table))):
            if table[i] >= 0:
                self.pool.give_back(table[i])
                table[i] = -1

    def release(self, slot: int) -> None:
        for p in self.tables.pop(slot, []):
            if p >= 0:
                self.pool.give_back(p)

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class Cache:
    """``requests[i]`` is what schedule entry ``i`` asks for: a pair
    (KVRequest or None, StateRequest or None).  ``cache_of[i]`` names the entry
    whose keys and values entry ``i`` reads instead of its own, or None.

    ``max_tokens`` is the most tokens the live sequences hold at any time, each
    sequence's count rounded up to a multiple of ``PAGE``."""

    def __init__(self, requests: Sequence[Tuple[Optional[KVRequest], Optional[StateRequest]]],
                 cache_of: Sequence[Optional[int]], max_tokens: int, dtype: torch.dtype, device,
                 n_slots: Optional[int] = None, max_seq_len: Optional[int] = None):
        if max_tokens < 1:
            raise InvalidArgument(f"a cache for {max_tokens} tokens")
        self.dtype, self.device = dtype, torch.device(device)
        self.n_pages = pages_for(max_tokens)
        self.max_tokens = self.n_pages * PAGE
        self.max_seq_len = min(max_seq_len or self.max_tokens, self.max_tokens)
        # every live sequence holds at least one page, so there are never more of them than pages
        self.n_slots = n_slots if n_slots is not None else self.n_pages
        self.slots = IndexPool(self.n_slots, "sequence slot")
        self.lengths = [0] * self.n_slots
        # counts the sequences a slot has held: whoever remembers a slot's page table must forget it when
        # the number has changed
        self.generation = [0] * self.n_slots
        self.groups: List[KVGroup] = []
        self._entry_group: List[Optional[Tuple[int, int]]] = [None] * len(requests)
        self._owns: List[bool] = [False] * len(requests)
        by_request: Dict[KVRequest, List[int]] = {}
        for i, (kv, _) in enumerate(requests):
            if cache_of[i] is not None:
                j = cache_of[i]
                if not (0 <= j < i) or cache_of[j] is not None or requests[j][0] is None:
                    raise InvalidArgument(f"schedule entry {i} reads the cache of entry {j}, "
                                          "which is not an earlier entry with keys and values of its own")
            elif kv is not None:
                by_request.setdefault(kv, []).append(i)
        esize = torch.empty((), dtype=dtype).element_size()
        need = sum(2 * len(e) * self.n_pages * kv.n_kv_heads * PAGE * kv.head_dim * esize for kv, e in by_request.items())
        for kv, entries in by_request.items():
            g = len(self.groups)
            with translating_oom(f"a cache of {self.max_tokens} tokens ({need / 2 ** 30:.2f} GiB of keys and values "
                                 f"for {sum(len(e) for e in by_request.values())} layer runs)"):
                self.groups.append(KVGroup(kv, entries, self.n_pages, dtype, self.device))
            for k, e in enumerate(entries):
                self._entry_group[e] = (g, k)
                self._owns[e] = True
        for i, j in enumerate(cache_of):
            if j is not None:
                self._entry_group[i] = self._entry_group[j]
        with translating_oom(f"per-sequence state for {self.n_slots} sequence slots"):
            self.states: List[Optional[torch.Tensor]] = [
                None if st is None else torch.zeros((self.n_slots + 1, *st.shape), dtype=st.dtype, device=self.device)
                for _, st in requests]

    @property
    def has_state(self) -> bool:
        """Whether some part keeps per-sequence state of fixed size beside the keys and values."""
        return any(s is not None for s in self.states)

    # -- slots ---------------------------------------------------------------

    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        self.generation[slot] += 1
        return slot

    def free_slot(self, slot: int) -> None:
        """Gives back the slot and every page it holds."""
        self.slots.give_back(slot)
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        self._need_held(slot)
        return self.lengths[slot]

    def truncate(self, slot: int, length: int) -> None:
        """Forgets the tokens from ``length`` on.  Pages stay with the slot.  A
        windowed group cannot go back past what it already gave up, and state
        cannot be rewound at all (crates/nncpu/src/model/kv.rs:380-412)."""
        self._need_held(slot)
        if not 0 <= length <= self.lengths[slot]:
            raise InvalidArgument(f"cannot truncate slot {slot} of length {self.lengths[slot]} to {length}")
        if length < self.lengths[slot]:
            if any(s is not None for s in self.states) and length > 0:
                raise InvalidArgument("a sequence with per-sequence state cannot be rewound, only restarted")
            for g in self.groups:
                if g.first_needed_page(self.lengths[slot]) > g.first_needed_page(length):
                    raise InvalidArgument(f"slot {slot}: the window has already moved past position {length}")
        self.lengths[slot] = length

    def _need_held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise InvalidArgument(f"sequence slot {slot!r} is not in use")

    # -- a step ----------------------------------------------------------------

    def prepare(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """Makes room for ``n_new[b]`` more tokens in ``slots[b]``.  Fails with
        ContextFull before anything is changed; zeroes the state of sequences
        that start."""
        if len(set(slots)) != len(slots):
            raise InvalidArgument("a sequence slot appears twice in one step")
        for s, n in zip(slots, n_new):
            self._need_held(s)
            if n < 1:
                raise InvalidArgument(f"slot {s}: a step of {n} tokens")
            if self.lengths[s] + n > self.max_seq_len:
                raise ContextFull(f"{n} more tokens do not fit slot {s}: it holds {self.lengths[s]} of "
                                  f"at most {self.max_seq_len} tokens")
        for g in self.groups:
            missing = sum(g.pages_missing(s, self.lengths[s] + n) for s, n in zip(slots, n_new))
            if missing > g.pool.n_free:
                raise ContextFull(f"the step needs {missing} more cache pages of {PAGE} tokens, "
                                  f"{g.pool.n_free} of {g.n_pages} are free")
        for g in self.groups:
            for s, n in zip(slots, n_new):
                g.grow(s, self.lengths[s] + n)
        for st in self.states:
            if st is not None:
                for s in slots:
                    if self.lengths[s] == 0:
                        st[s].zero_()       # a fill kernel in stream order: no host tensor, no wait

    def rollback(self, slots: Sequence[int]) -> None:
        """Undoes a ``prepare`` whose step did not happen: the pages taken beyond what each sequence's length
        needs go back to their pools."""
        for g in self.groups:
            for s in slots:
                table = g.tables.get(s)
                while table is not None and len(table) > pages_for(self.lengths[s]):
                    p = table.pop()
                    if p >= 0:
                        g.pool.give_back(p)
                if table is not None and not table:
                    del g.tables[s]

    def commit(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """The step's launches are enqueued: lengths advance, and windowed
        groups give back the pages no later query can see."""
        for s, n in zip(slots, n_new):
            self.lengths[s] += n
            for g in self.groups:
                if g.request.window > 0:
                    g.trim(s, self.lengths[s])

    def block_table(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> List[List[int]]:
        """Page ids by page index for each slot, padded with -1 to ``width``."""
        g = self.groups[group]
        rows = [g.tables.get(s, []) for s in slots]
        width = width if width is not None else max([len(r) for r in rows] + [1])
        return [r + [-1] * (width - len(r)) for r in rows]

    # -- views for the parts -----------------------------------------------------

    def group_of(self, entry: int) -> Optional[int]:
        eg = self._entry_group[entry]
        return None if eg is None else eg[0]

    def owns_kv(self, entry: int) -> bool:
        return self._owns[entry]

    def kv(self, entry: int):
        """(keys, values) of schedule entry ``entry``: [n_pages, n_kv_heads, PAGE, head_dim]."""
        g, k = self._entry_group[entry]
        return self.groups[g].k[k], self.groups[g].v[k]

    def state(self, entry: int) -> Optional[torch.Tensor]:
        return self.states[entry]

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + sum(
            s.numel() * s.element_size() for s in self.states if s is not None)

    def check(self) -> None:
        """Bookkeeping invariants, for tests: no slot or page lost or held twice."""
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            held = [p for t in g.tables.values() for p in t if p >= 0]
            assert len(held) == len(set(held)), "a cache page is in two page tables"
            assert len(held) == g.pool.n_held, "a cache page is held by no sequence"
            assert all(self.slots.is_held(s) for s in g.tables), "a free slot still has pages"
