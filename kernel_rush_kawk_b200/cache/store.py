"""The cache: a slot for each live sequence, storage for each run of a layer.

Storage is paged: a page holds 64 consecutive positions of one run's keys (or
values) for all kv heads, ``[kv_heads, 64, head_dim]``, and a sequence's slot
owns a row of a page table that maps position // 64 to a page. Kernels read the
table on the device, so a sequence's positions need not be contiguous and the
cache is sized by tokens in flight, not by slots x longest sequence. (The
reference keeps ``[layers, batch, kv_heads, capacity, head_dim]`` with the batch
row as the slot and a capacity fixed per plan: engine/model.py:223,231-234 of
willzeng274/kernel-rush-kawk.)

Runs whose needs differ get storage groups of their own: runs that keep every
key share one group, runs that keep a window of W keys another, whose slots cycle
through a ring of pages, position p living in ring entry (p // 64) % ring. Each
kind of fixed-size per-sequence state is a group too: ``[runs, slots, *shape]``,
zeroed when the slot is handed out.

Pages are not cleared when a slot is given back: every read is bounded by the
sequence's length, as in the reference, whose reset is ``pos.zero_()`` (:290).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .allocator import CacheError, FreeList, PageLedger

PAGE = 64  # positions per page; the attention kernels' key block


@dataclass
class KVView:
    """What a mixer's kernels get: this run's pages and its group's page table."""

    k: torch.Tensor  # [pages, kv_heads, PAGE, head_dim]
    v: torch.Tensor
    table: torch.Tensor  # int32 [slots, width] on the device
    width: int  # logical pages per slot; position p is in table[slot, (p // PAGE) % width]
    window: int | None
    kv_heads: int
    head_dim: int


@dataclass
class StateView:
    state: torch.Tensor  # [slots, *shape]


class _KVGroup:
    def __init__(self, need: KVNeed, runs: list[int], n_pages: int, n_slots: int, width: int, ring: int | None,
                 device, dtype):
        self.need = need
        self.runs = runs
        self.width = ring if ring is not None else width
        self.ledger = PageLedger(n_pages, n_slots, self.width, PAGE, ring)
        shape = (len(runs), n_pages, need.kv_heads, PAGE, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table_host = np.zeros((n_slots, self.width), dtype=np.int32)
        self.table = torch.zeros((n_slots, self.width), dtype=torch.int32, device=device)
        self.dirty: set[int] = set()

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class _StateGroup:
    def __init__(self, need: StateNeed, runs: list[int], n_slots: int, device, dtype):
        self.need = need
        self.runs = runs
        dt = torch.float32 if need.dtype == "float32" else dtype
        self.state = torch.zeros((len(runs), n_slots) + tuple(need.shape), dtype=dt, device=device)


class SequenceCache:
    """needs: one entry per schedule run: KVNeed, StateNeed, None, or ("from", j) for
    a run that reads run j's storage.

    max_tokens: positions all live sequences may hold together, each sequence's
    count rounded up to whole pages. max_slots: live sequences. max_context: the
    longest sequence. step_tokens: the most tokens one sequence brings in one step;
    it sizes the rings of window groups."""

    def __init__(self, needs: list, max_tokens: int, max_slots: int, max_context: int, device, dtype,
                 step_tokens: int = 2048):
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_slots = int(max_slots)
        self.max_context = int(max_context)
        self.step_tokens = int(step_tokens)
        self.n_pages = max(1, -(-int(max_tokens) // PAGE))
        self.width = max(1, -(-self.max_context // PAGE))
        self.slots = FreeList(self.max_slots, "cache slot")
        self.length = [0] * self.max_slots
        self.h2d_bytes = 0  # page-table rows (and their indices) copied to the device so far
        self._kv_groups: list[_KVGroup] = []
        self._state_groups: list[_StateGroup] = []
        self._where: list = [None] * len(needs)  # run -> (group, line) or None

        by_need: dict = {}
        for run, need in enumerate(needs):
            if isinstance(need, (KVNeed, StateNeed)):
                by_need.setdefault(need, []).append(run)
        for need, runs in by_need.items():
            if isinstance(need, KVNeed):
                ring = None
                pages = self.n_pages
                if need.window is not None:
                    ring = min(self.width, -(-(need.window + self.step_tokens - 1) // PAGE) + 1)
                    pages = min(self.n_pages, self.max_slots * ring)
                group = _KVGroup(need, runs, pages, self.max_slots, self.width, ring, self.device, dtype)
                self._kv_groups.append(group)
            else:
                group = _StateGroup(need, runs, self.max_slots, self.device, dtype)
                self._state_groups.append(group)
            for line, run in enumerate(runs):
                self._where[run] = (group, line)
        for run, need in enumerate(needs):
            if isinstance(need, tuple) and need and need[0] == "from":
                src = self._where[need[1]]
                if src is None or not isinstance(src[0], _KVGroup):
                    raise CacheError(f"run {run} reads the cache of run {need[1]}, which keeps no keys and values")
                self._where[run] = src

    # -- slots --------------------------------------------------------------
    def alloc(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        for g in self._state_groups:
            g.state[:, slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        self.slots.give(slot)  # raises on a slot that is not held
        for g in self._kv_groups:
            g.ledger.release(slot)
        self.length[slot] = 0

    def reserve(self, slot: int, length: int) -> None:
        """Make room for ``slot`` to hold ``length`` positions."""
        if not self.slots.is_held(slot):
            raise CacheError(f"cache slot {slot} is not held")
        if length > self.max_context:
            raise CacheError(f"a sequence of {length} tokens exceeds the longest the cache was built for ({self.max_context})")
        for g in self._kv_groups:
            if not g.ledger.can_grow(slot, length):
                g.ledger.grow(slot, length)  # raises with the numbers
        for g in self._kv_groups:
            for logical, page in g.ledger.grow(slot, length):
                g.table_host[slot, logical] = page
                g.dirty.add(slot)

    def advance(self, slot: int, n: int) -> None:
        self.length[slot] += n

    def sync(self) -> None:
        """Bring the device's page tables up to date (rows that changed)."""
        for g in self._kv_groups:
            if not g.dirty:
                continue
            rows = sorted(g.dirty)
            idx = torch.as_tensor(rows, dtype=torch.int64, device=self.device)
            g.table.index_copy_(0, idx, torch.from_numpy(g.table_host[rows]).to(self.device))
            self.h2d_bytes += len(rows) * (8 + 4 * g.width)
            g.dirty.clear()

    def save_state(self, slots) -> list:
        """Copies of the fixed-size state that these slots hold, one tensor per state group."""
        idx = torch.as_tensor(list(slots), dtype=torch.int64, device=self.device)
        return [g.state.index_select(1, idx) for g in self._state_groups]

    def restore_state(self, slots, saved: list) -> None:
        idx = torch.as_tensor(list(slots), dtype=torch.int64, device=self.device)
        for g, s in zip(self._state_groups, saved):
            g.state.index_copy_(1, idx, s)

    def per_sequence_step_limit(self) -> int | None:
        """The most tokens one sequence may bring in one pass, or None if any number will do. A group that
        keeps a window of keys cycles through a ring of pages sized for ``step_tokens`` new positions;
        a longer pass would overwrite keys that its own first rows still have to read."""
        if any(g.need.window is not None for g in self._kv_groups):
            return self.step_tokens
        return None

    # -- views --------------------------------------------------------------
    def view(self, run: int):
        where = self._where[run]
        if where is None:
            return None
        group, line = where
        if isinstance(group, _KVGroup):
            return KVView(group.k[line], group.v[line], group.table, group.width, group.need.window,
                          group.need.kv_heads, group.need.head_dim)
        return StateView(group.state[line])

    # -- accounting ---------------------------------------------------------
    @property
    def live(self) -> int:
        return self.slots.held

    def free_pages(self) -> int:
        return min((len(g.ledger.pool) for g in self._kv_groups), default=0)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self._kv_groups) + sum(
            g.state.numel() * g.state.element_size() for g in self._state_groups)

    def check(self) -> None:
        """Raise if a slot or page is lost or held twice."""
        self.slots.check()
        for g in self._kv_groups:
            g.ledger.check()
            for slot in range(self.max_slots):
                if not self.slots.is_held(slot) and g.ledger.pages[slot]:
                    raise CacheError(f"slot {slot} is free but still holds pages")
