"""The cache: a slot per sequence, paged keys and values per layer group, fixed-size state.

* A *slot* is one live sequence: its length and, for every group, the pages it holds.
* Layers whose mixers ask for the same thing form a *group* with storage of its own:
  - a key/value group keeps, per layer, pages [page][kv_head][page_size][head_dim]
    for keys and the same for values; every sequence has a row in the group's page
    table mapping position // page_size to a page. A group with a window keeps only
    the pages that still hold positions inside the window and returns the others;
  - a state group keeps, per layer, one fixed-size tensor per slot, zeroed when the
    slot is taken. Llama has none; the storage exists for mixers that do.
* Slots and pages go back to the free lists when a sequence ends and are handed out
  again, lowest number first. Stale contents are never cleared: reads are bounded by
  each sequence's own length.

(The reference gives each sequence a Session with flat per-layer buffers,
crates/model-runtime/src/session.rs:3-42; attention layers own K/V, linear layers own
fixed-size state, crates/model-runtime/src/lib.rs:119-133. Batches, slots and pages
are this library's design.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import CacheMemoryError, ContextError, InvalidError
from ..parts.base import KeyValueRequest, StateRequest
from .slots import FreeList

PAGE_SIZE = 64


@dataclass
class KeyValueView:
    """What an attention layer gets: its pages and the group's page table."""

    k: torch.Tensor  # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    page_table: torch.Tensor  # int32 [max_slots, pages_per_sequence], -1 = no page
    page_size: int
    kv_heads: int
    head_dim: int
    window: Optional[int]
    group: int = 0  # index of the storage group (a step's destination rows are per group)


@dataclass
class StateView:
    state: torch.Tensor  # [max_slots, *shape]


class KeyValueGroup:
    def __init__(self, request: KeyValueRequest, entries: List[int], pages: int, max_slots: int,
                 pages_per_sequence: int, page_size: int, dtype, device):
        self.request, self.entries, self.page_size = request, entries, page_size
        self.pool = FreeList(pages, "page")
        self.table_host = np.full((max_slots, pages_per_sequence), -1, dtype=np.int32)
        self.table_device = torch.full((max_slots, pages_per_sequence), -1, dtype=torch.int32,
                                       device=device)
        self.dirty = False
        shape = (pages, request.kv_heads, page_size, request.head_dim)
        # zeroed once: a kernel may load rows of a page that no token was ever stored in (they are
        # masked, but 0 x NaN would still be NaN)
        self.k = {e: torch.zeros(shape, dtype=dtype, device=device) for e in entries}
        self.v = {e: torch.zeros(shape, dtype=dtype, device=device) for e in entries}

    def first_kept_page(self, length: int) -> int:
        """Lowest logical page a sequence of `length` tokens still needs."""
        if self.request.window is None:
            return 0
        return max(0, length - self.request.window) // self.page_size

    def first_needed_page(self, new_length: int, reads_from: Optional[int]) -> int:
        """Lowest logical page a step needs that takes a sequence to `new_length` tokens.

        `reads_from` is the position of the first query of the step that reads this
        sequence's keys from the cache (every key its window still shows must then be
        there), or None when the step's attention reads the step's own keys and the
        cache only has to keep what later steps will see."""
        seen_by = new_length if reads_from is None else min(new_length, reads_from + 1)
        return self.first_kept_page(seen_by)

    def pages_needed(self, slot: int, new_length: int, reads_from: Optional[int] = None) -> int:
        """How many new pages taking the sequence to `new_length` tokens costs."""
        if new_length <= 0:
            return 0
        row = self.table_host[slot]
        last = (new_length - 1) // self.page_size
        first = self.first_needed_page(new_length, reads_from)
        if last >= len(row):
            return last + 1 - first  # more than the table can name: more than any pool holds
        return int(np.count_nonzero(row[first:last + 1] < 0))

    def pages_released(self, slot: int, new_length: int, reads_from: Optional[int] = None) -> int:
        first = self.first_needed_page(new_length, reads_from)
        return int(np.count_nonzero(self.table_host[slot][:first] >= 0))

    def release_stale(self, slot: int, new_length: int, reads_from: Optional[int] = None) -> None:
        """Return the pages that lie wholly before what a step to `new_length` still needs."""
        row = self.table_host[slot]
        first = self.first_needed_page(new_length, reads_from)
        stale = [int(p) for p in row[:first] if p >= 0]
        if stale:
            self.pool.give_back(stale)
            row[:first] = -1
            self.dirty = True

    def take_missing(self, slot: int, new_length: int, reads_from: Optional[int] = None) -> None:
        if new_length <= 0:
            return
        row = self.table_host[slot]
        first = self.first_needed_page(new_length, reads_from)
        last = (new_length - 1) // self.page_size
        missing = [i for i in range(first, last + 1) if row[i] < 0]
        if missing:
            for i, page in zip(missing, self.pool.take(len(missing))):
                row[i] = page
            self.dirty = True

    def release(self, slot: int) -> None:
        row = self.table_host[slot]
        held = [int(p) for p in row if p >= 0]
        if held:
            self.pool.give_back(held)
            row[:] = -1
            self.dirty = True

    def sync(self) -> None:
        if self.dirty:
            self.table_device.copy_(torch.from_numpy(self.table_host), non_blocking=False)
            self.dirty = False

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self.k.values()) + list(self.v.values()))


class StateGroup:
    def __init__(self, request: StateRequest, entries: List[int], max_slots: int, device):
        self.request, self.entries = request, entries
        self.state = {e: torch.zeros((max_slots, *request.shape), dtype=request.dtype, device=device)
                      for e in entries}

    def clear(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.state.values())


class Cache:
    """Slots, groups and their storage for one model.

    `requests[i]` is what cache entry i's mixer asked for (KeyValueRequest,
    StateRequest or None). `max_tokens` is the most tokens live sequences hold at
    any time, each sequence's count rounded up to whole pages; it sizes every
    key/value group's page pool. `max_sequence` bounds one sequence's length.
    """

    def __init__(self, requests: Sequence, dtype: torch.dtype, device, max_tokens: int,
                 max_slots: int, max_sequence: int, page_size: int = PAGE_SIZE):
        if max_tokens <= 0 or max_slots <= 0 or max_sequence <= 0 or page_size <= 0:
            raise InvalidError("cache sizes must be positive")
        self.page_size = page_size
        self.max_sequence = max_sequence
        self.max_slots = max_slots
        self.pages = -(-max_tokens // page_size)
        # the table names every page a sequence of max_sequence tokens can have; how many pages a
        # sequence may hold at once is the pool's business (a windowed group holds few of them)
        pages_per_sequence = -(-max_sequence // page_size)
        self.slots = FreeList(max_slots, "slot")
        self.lengths = np.zeros(max_slots, dtype=np.int64)  # tokens cached per slot
        self.open_mask = np.zeros(max_slots, dtype=bool)      # slot is held by a sequence
        self.kv_groups: List[KeyValueGroup] = []
        self.state_groups: List[StateGroup] = []
        self._where: Dict[int, Tuple[str, int]] = {}
        by_request: Dict[object, List[int]] = {}
        for entry, request in enumerate(requests):
            if request is not None:
                by_request.setdefault(request, []).append(entry)
        for request, entries in by_request.items():
            if isinstance(request, KeyValueRequest):
                group = KeyValueGroup(request, entries, self.pages, max_slots, pages_per_sequence,
                                      page_size, dtype, device)
                for e in entries:
                    self._where[e] = ("kv", len(self.kv_groups))
                self.kv_groups.append(group)
            elif isinstance(request, StateRequest):
                group = StateGroup(request, entries, max_slots, device)
                for e in entries:
                    self._where[e] = ("state", len(self.state_groups))
                self.state_groups.append(group)
            else:
                raise InvalidError(f"unknown cache request {request!r}")

    # -- slots -------------------------------------------------------------------
    def open_slot(self) -> int:
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        self.open_mask[slot] = True
        for group in self.state_groups:
            group.clear(slot)
        return slot

    def close_slot(self, slot: int) -> None:
        self.slots.give_back([slot])
        for group in self.kv_groups:
            group.release(slot)
        self.lengths[slot] = 0
        self.open_mask[slot] = False

    def reset_slot(self, slot: int) -> None:
        """Forget a sequence's tokens but keep the slot (reference: Session::reset)."""
        self._require(slot)
        for group in self.kv_groups:
            group.release(slot)
        for group in self.state_groups:
            group.clear(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        self._require(slot)
        return int(self.lengths[slot])

    def _require(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots) or not self.slots.is_held(slot):
            raise InvalidError(f"slot {slot} is not open")

    # -- growth --------------------------------------------------------------------
    @staticmethod
    def _growth(growth):
        """(slot, new_length[, reads_from]) -> (slot, new_length, reads_from); see grow()."""
        return [(g[0], g[1], g[2] if len(g) > 2 else None) for g in growth]

    def check_growth(self, growth: Sequence[Tuple]) -> None:
        """Raise, changing nothing, unless every (slot, new_length[, reads_from]) of a step fits."""
        growth = self._growth(growth)
        for slot, new_length, _ in growth:
            self._require(slot)
            if new_length > self.max_sequence:
                raise ContextError(self.max_sequence, new_length)
        for group in self.kv_groups:
            need = sum(group.pages_needed(s, n, r) for s, n, r in growth)
            freed = sum(group.pages_released(s, n, r) for s, n, r in growth)
            if need > group.pool.available + freed:
                raise CacheMemoryError(
                    f"step needs {need} pages of {self.page_size} tokens, "
                    f"{group.pool.available + freed} free of {group.pool.count}")

    def grow(self, growth: Sequence[Tuple]) -> None:
        """Give every sequence of a step the pages it needs up to its new length.

        An entry is (slot, new_length) or (slot, new_length, reads_from): `reads_from` is
        the position of the step's first query for that sequence when the step's attention
        reads the cache (a windowed group then keeps every page that query still sees);
        without it the step attends to its own keys and a windowed group keeps only what
        later steps will see."""
        growth = self._growth(growth)
        self.check_growth(growth)
        for group in self.kv_groups:
            for slot, new_length, reads_from in growth:  # release first so the freed pages can be reused
                group.release_stale(slot, new_length, reads_from)
            for slot, new_length, reads_from in growth:
                group.take_missing(slot, new_length, reads_from)

    def grow_by_one(self, slots: np.ndarray):
        """The decode step's bookkeeping for many sequences at once: every listed (open, distinct,
        non-empty) slot grows by one token. Checks capacity and pages first and changes nothing
        if the step does not fit. Returns (lengths before, per key/value group the row each new
        token is stored at), or None for an empty step. A windowed group gives back the pages
        that the new token no longer sees. The caller commits with commit_lengths()."""
        if len(slots) == 0:
            return None
        before = self.lengths[slots]
        if int(before.max()) + 1 > self.max_sequence:
            raise ContextError(self.max_sequence, int(before.max()) + 1)
        ps = self.page_size
        index = before // ps
        missing, stale = [], []
        for group in self.kv_groups:
            lacking = np.nonzero(group.table_host[slots, index] < 0)[0]
            leaving = np.zeros(0, dtype=np.int64)
            if group.request.window is not None:
                # Pages below the first one the new token still sees. Pages leave a window lowest
                # first, so a sequence holds stale pages exactly when it holds the one right below.
                first = np.maximum(0, before + 1 - group.request.window) // ps
                leaving = np.nonzero((first > 0) & (group.table_host[slots, np.maximum(first - 1, 0)] >= 0))[0]
            freed = sum(int(np.count_nonzero(group.table_host[slots[i], :first[i]] >= 0)) for i in leaving)
            stale.append(leaving)
            if len(lacking) > group.pool.available + freed:
                raise CacheMemoryError(f"step needs {len(lacking)} pages of {ps} tokens, "
                                       f"{group.pool.available + freed} free of {group.pool.count}")
            missing.append(lacking)
        rows = []
        for group, lacking, leaving in zip(self.kv_groups, missing, stale):
            for i in leaving:
                group.release_stale(int(slots[i]), int(before[i]) + 1)
            if len(lacking):
                pages = group.pool.take(len(lacking))
                group.table_host[slots[lacking], index[lacking]] = pages
                group.dirty = True
            rows.append((group.table_host[slots, index].astype(np.int64) * ps + before % ps).astype(np.int32))
        return before, rows

    def commit_lengths(self, slots: np.ndarray, lengths: np.ndarray) -> None:
        self.lengths[slots] = lengths

    def commit(self, growth: Sequence[Tuple]) -> None:
        for entry in growth:
            self.lengths[entry[0]] = entry[1]

    def shorten(self, slots: Sequence[int], tokens: int = 1) -> None:
        """Take the last `tokens` tokens of some sequences back: only the lengths change. The
        pages stay with their sequences and the rows are written again when those positions are
        fed again (a windowed group keeps the same pages for the same position). Fixed-size
        state cannot be taken back, so a cache with state groups refuses."""
        if self.state_groups:
            raise InvalidError("sequences with fixed-size state cannot be shortened")
        slots = [int(s) for s in slots]
        for slot in slots:
            self._require(slot)
            if tokens < 0 or self.lengths[slot] < tokens:
                raise InvalidError(f"slot {slot} holds {int(self.lengths[slot])} tokens, cannot take back {tokens}")
        for slot in slots:
            self.lengths[slot] -= tokens

    def sync(self) -> None:
        for group in self.kv_groups:
            group.sync()

    def destination_rows(self, slots: Sequence[int], before: Sequence[int], counts: Sequence[int]):
        """For every key/value group, where each token of a step is stored: an int32 array over
        the step's packed tokens, page * page_size + row in page, -1 where the group does not
        keep that position. Call after grow()."""
        out = []
        for group in self.kv_groups:
            ps = group.page_size
            parts = []
            for slot, start, n in zip(slots, before, counts):
                pos = np.arange(start, start + n, dtype=np.int64)
                pages = group.table_host[slot][pos // ps].astype(np.int64)
                parts.append(np.where(pages >= 0, pages * ps + pos % ps, -1))
            out.append(np.concatenate(parts).astype(np.int32) if parts else np.zeros(0, np.int32))
        return out

    # -- views ---------------------------------------------------------------------
    def view(self, entry: int):
        kind, index = self._where.get(entry, (None, None))
        if kind == "kv":
            g = self.kv_groups[index]
            return KeyValueView(g.k[entry], g.v[entry], g.table_device, g.page_size,
                                g.request.kv_heads, g.request.head_dim, g.request.window, index)
        if kind == "state":
            return StateView(self.state_groups[index].state[entry])
        return None

    def snapshot(self, slot: int, entry: int):
        """Keys and values of one sequence and cache entry as [tokens, kv_heads, head_dim]
        (diagnostic copy, like crates/model-runtime/src/session.rs:45-83). Positions a
        windowed group no longer keeps are NaN."""
        kind, index = self._where[entry]
        if kind != "kv":
            return self.state_groups[index].state[entry][slot].clone()
        g = self.kv_groups[index]
        n = self.length(slot)
        shape = (n, g.request.kv_heads, g.request.head_dim)
        k = torch.full(shape, float("nan"), dtype=torch.float32)
        v = torch.full(shape, float("nan"), dtype=torch.float32)
        for p in range(n):
            page = int(g.table_host[slot][p // g.page_size])
            if page >= 0:
                k[p] = g.k[entry][page, :, p % g.page_size].float().cpu()
                v[p] = g.v[entry][page, :, p % g.page_size].float().cpu()
        return k, v

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.kv_groups) + sum(g.bytes() for g in self.state_groups)

    def held_pages(self) -> List[int]:
        return [g.pool.held for g in self.kv_groups]
