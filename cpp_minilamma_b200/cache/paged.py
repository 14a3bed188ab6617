"""The sequence cache: slots, pages, groups of layers, and fixed-size state.

* A **slot** belongs to one live sequence.  It records the sequence's length and, per
  group, the pages that hold its keys and values.  Slots are handed out by `acquire`,
  given back by `release`, and used again by later batches.
* A **page** holds PAGE consecutive positions of one sequence for every cache entry of
  one group: tensors `k, v [entries, pages, kv_heads, PAGE, head_dim]`.  Pages come from a
  free list per group, so a budget of N tokens (each sequence rounded up to whole pages)
  is all the memory the cache ever needs, however the tokens are spread over sequences.
* A **group** gathers the schedule entries whose mixers declare the same need
  (kv heads, head size, window).  Each group has storage and a block table of its own.
  A group with a window w gives pages back as soon as no later query can read them.
* **State** is per-slot storage of fixed size for mixers that keep a running state
  instead of (or beside) keys and values: `state[name] [slots, *shape]`, float32, zeroed
  when the slot is handed out.
* One **padding slot** beyond the slots that are handed out, with a page and a state row of its own,
  stands in for the spare rows of a decode step whose batch size was rounded up.

The reference keeps one contiguous cache per sequence, `[layers, max_seq_len, kv_heads,
head_dim]` float32 (src/kvcache.cc:16-54, src/cuda_kvcache.cc:116-179), and a `Context`
with `pos` and the token history (include/context.h:15-35); positions there play the
part that pages in slots play here.

All bookkeeping is host-side Python on integers; device memory is touched only through
the block-table upload (`flush`) and the zeroing of state rows, so the allocator can be
exercised on a CPU device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheNeed, KVNeed, StateNeed

PAGE = 64


class CacheError(RuntimeError):
    """Misuse of the cache: a slot that is not live, freed twice, and the like."""


class CacheFull(CacheError):
    """Not enough free slots or pages; nothing was changed."""


class PagePool:
    """Free list of page numbers with double-free and leak checks."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise CacheError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))  # pop() hands out 0 first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} pages wanted, {len(self._free)} of {self.n_pages} free")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            self._held[p] = True
        return pages

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise CacheError(f"page {p} does not exist")
            if not self._held[p]:
                raise CacheError(f"page {p} given back twice")
        for p in pages:
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        held = sum(self._held)
        if held + len(self._free) != self.n_pages:
            raise CacheError(f"pages lost: {held} held + {len(self._free)} free != {self.n_pages}")
        for p in self._free:
            if self._held[p]:
                raise CacheError(f"page {p} is both free and held")


@dataclass
class CacheView:
    """What one schedule entry's mixer sees."""

    k: Optional[torch.Tensor]            # [pages, kv_heads, PAGE, head_dim] or None
    v: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]  # int32 [slots, max_blocks] of the entry's group
    window: int
    state: Dict[str, torch.Tensor]       # name -> [slots, *shape] float32
    owns_kv: bool                        # False when the entry reads another entry's cache


class CacheGroup:
    def __init__(self, need: KVNeed, entries: List[int], n_pages: int, n_slots: int, max_blocks: int,
                 dtype: torch.dtype, device):
        self.need = need
        self.entries = list(entries)
        self.pool = PagePool(n_pages)
        self.max_blocks = max_blocks
        # one page and one block-table row beyond those that are handed out: the padding slot's (SequenceCache.pad_slot)
        shape = (len(entries), n_pages + 1, need.n_kv_heads, PAGE, need.head_dim)
        self.k = torch.empty(shape, dtype=dtype, device=device)
        self.v = torch.empty(shape, dtype=dtype, device=device)
        self.table_host = np.full((n_slots + 1, max_blocks), -1, dtype=np.int32)
        self.table_host[n_slots, 0] = n_pages
        self.table_dev = torch.from_numpy(self.table_host.copy()).to(device)
        self._dirty: set = set()
        # pages of each slot by block index (None once a window let go of it)
        self.pages: List[List[Optional[int]]] = [[] for _ in range(n_slots)]

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, (new_len + PAGE - 1) // PAGE - len(self.pages[slot]))

    def grow(self, slot: int, old_len: int, new_len: int) -> None:
        blocks = (new_len + PAGE - 1) // PAGE
        if blocks > self.max_blocks:
            raise CacheFull(f"sequence of {new_len} tokens needs {blocks} pages, the block table holds "
                            f"{self.max_blocks}")
        have = len(self.pages[slot])
        if blocks > have:
            fresh = self.pool.take(blocks - have)
            for i, p in enumerate(fresh):
                self.table_host[slot, have + i] = p
            self.pages[slot].extend(fresh)
            self._dirty.add(slot)
        if self.need.window > 0:
            # the earliest query of this step sits at old_len and reads keys > old_len - window
            first_needed = max(0, old_len - self.need.window + 1) // PAGE
            gone = []
            for b in range(min(first_needed, len(self.pages[slot]))):
                if self.pages[slot][b] is not None:
                    gone.append(self.pages[slot][b])
                    self.pages[slot][b] = None
                    self.table_host[slot, b] = -1
            if gone:
                self.pool.give_back(gone)
                self._dirty.add(slot)

    def drop(self, slot: int) -> None:
        held = [p for p in self.pages[slot] if p is not None]
        self.pool.give_back(held)
        n = len(self.pages[slot])
        self.pages[slot] = []
        if n:
            # nobody reads the row of a slot that is not live, so the device's copy may stay as it is
            # until the slot is handed out again and grows
            self.table_host[slot, :n] = -1
            self._dirty.discard(slot)

    def take_updates(self) -> Optional[np.ndarray]:
        """The rows that changed since the last call as int32 [n, 1 + max_blocks] (column 0: the slot), or
        None.  The caller brings them to the device (`scatter_rows` into `table_dev`)."""
        if not self._dirty:
            return None
        slots = sorted(self._dirty)
        self._dirty.clear()
        rows = np.empty((len(slots), 1 + self.max_blocks), dtype=np.int32)
        rows[:, 0] = slots
        rows[:, 1:] = self.table_host[slots]
        return rows

    def flush(self) -> None:
        """Upload the changed rows now, one blocking copy each (for callers outside an engine's step)."""
        for slot in sorted(self._dirty):
            self.table_dev[slot].copy_(torch.from_numpy(self.table_host[slot]), non_blocking=False)
        self._dirty.clear()


class SequenceCache:
    """Slots + groups + state for one model on one device."""

    def __init__(self, needs: Sequence[Tuple[int, Optional[int], CacheNeed]], max_tokens: int, n_slots: int,
                 max_positions: int, dtype: torch.dtype, device):
        """needs: (schedule entry index, cache_of or None, the mixer's CacheNeed) per entry.
        max_tokens: the most tokens live sequences hold together, each rounded up to PAGE."""
        if max_tokens < 1:
            raise CacheError("max_tokens must be positive")
        self.n_pages = (max_tokens + PAGE - 1) // PAGE
        self.n_slots = max(1, min(n_slots, self.n_pages))
        self.max_blocks = max(1, min(self.n_pages, (max_positions + PAGE - 1) // PAGE))
        self.max_positions = max_positions
        self.device = device
        self.dtype = dtype
        self.groups: List[CacheGroup] = []
        self._entry_group: Dict[int, Tuple[int, int]] = {}  # entry -> (group, index in group)
        self._entry_source: Dict[int, int] = {}
        self.state: Dict[int, Dict[str, torch.Tensor]] = {}
        by_need: Dict[KVNeed, List[int]] = {}
        for entry, cache_of, need in needs:
            if cache_of is not None:
                if cache_of >= entry:
                    raise CacheError(f"schedule entry {entry} reads the cache of entry {cache_of}, which runs later")
                self._entry_source[entry] = cache_of
                continue
            if need.kv is not None:
                by_need.setdefault(need.kv, []).append(entry)
            if need.state is not None:
                self.state[entry] = {
                    name: torch.zeros((self.n_slots + 1, *shape), dtype=torch.float32, device=device)
                    for name, shape in need.state.tensors}
        for need, entries in by_need.items():
            g = len(self.groups)
            self.groups.append(CacheGroup(need, entries, self.n_pages, self.n_slots, self.max_blocks, dtype, device))
            for i, entry in enumerate(entries):
                self._entry_group[entry] = (g, i)
        for entry, source in self._entry_source.items():
            if source in self._entry_source:
                raise CacheError(f"entry {entry} reads entry {source}, which itself owns no cache")
        # The padding slot: never handed out.  A captured decode step of a rounded-up batch size fills its
        # spare rows with it (one token at position 0 of a page of its own, which those rows write and read);
        # what they compute is thrown away.
        self.pad_slot = self.n_slots
        self._free_slots: List[int] = list(range(self.n_slots - 1, -1, -1))
        self._live = [False] * self.n_slots
        self.seq_len = [0] * self.n_slots

    # ---- slots -------------------------------------------------------------- #
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> int:
        return min((g.pool.n_free for g in self.groups), default=self.n_pages)

    def acquire(self, count: int = 1) -> List[int]:
        if count > len(self._free_slots):
            raise CacheFull(f"{count} slots wanted, {len(self._free_slots)} of {self.n_slots} free")
        slots = [self._free_slots.pop() for _ in range(count)]
        for s in slots:
            self._live[s] = True
            self.seq_len[s] = 0
        if self.state and slots:
            index = torch.tensor(slots, dtype=torch.long, device=self.device)
            for tensors in self.state.values():
                for t in tensors.values():
                    t.index_fill_(0, index, 0.0)
        return slots

    def release(self, slot: int) -> None:
        self._require_live(slot)
        for g in self.groups:
            g.drop(slot)
        self._live[slot] = False
        self.seq_len[slot] = 0
        self._free_slots.append(slot)

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def _require_live(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots:
            raise CacheError(f"slot {slot} does not exist (0..{self.n_slots - 1})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is not live (released twice or never acquired)")

    # ---- growth -------------------------------------------------------------- #
    def reserve(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Make room for `extra` more tokens in each (slot, extra); all or nothing."""
        seen = set()
        for slot, extra in growth:
            self._require_live(slot)
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if extra < 1:
                raise CacheError(f"slot {slot}: a step must bring at least one token")
            if self.seq_len[slot] + extra > self.max_positions:
                raise CacheFull(f"slot {slot}: {self.seq_len[slot]} + {extra} tokens exceed the "
                                f"{self.max_positions} positions of the model")
            if (self.seq_len[slot] + extra + PAGE - 1) // PAGE > self.max_blocks:
                raise CacheFull(f"slot {slot}: {self.seq_len[slot] + extra} tokens exceed the block table "
                                f"({self.max_blocks} pages)")
        for g in self.groups:
            wanted = sum(g.pages_needed(slot, self.seq_len[slot] + extra) for slot, extra in growth)
            # pages a window frees in this same step are not counted on
            if wanted > g.pool.n_free:
                raise CacheFull(f"{wanted} pages wanted, {g.pool.n_free} of {g.pool.n_pages} free; "
                                f"the cache was sized for {self.n_pages * PAGE} tokens")
        for slot, extra in growth:
            old = self.seq_len[slot]
            for g in self.groups:
                g.grow(slot, old, old + extra)
            self.seq_len[slot] = old + extra

    def flush(self) -> None:
        """Upload the block-table rows that changed since the last call (blocking copies; the engine's
        steps use `take_table_updates` instead and send the rows along with their index arrays)."""
        for g in self.groups:
            g.flush()

    def take_table_updates(self) -> List[Tuple[CacheGroup, np.ndarray]]:
        """(group, int32 [n, 1 + max_blocks]) for every group whose block table changed since the last
        call; the caller owns bringing them to the device before the next kernel reads the tables."""
        out = []
        for g in self.groups:
            rows = g.take_updates()
            if rows is not None:
                out.append((g, rows))
        return out

    def table_update_capacity(self, n_seqs: int) -> int:
        """Integers that the updates of a step with `n_seqs` sequences can take at most."""
        return len(self.groups) * n_seqs * (1 + self.max_blocks)

    # ---- views ---------------------------------------------------------------- #
    def view(self, entry: int) -> CacheView:
        source = self._entry_source.get(entry, entry)
        owns = source == entry
        state = self.state.get(source, {})
        if source in self._entry_group:
            g, i = self._entry_group[source]
            group = self.groups[g]
            return CacheView(group.k[i], group.v[i], group.table_dev, group.need.window, state, owns)
        return CacheView(None, None, None, 0, state, owns)

    def check(self) -> None:
        """Invariants: no slot lost or held twice, no page lost, tables match the page lists."""
        if len(set(self._free_slots)) != len(self._free_slots):
            raise CacheError("a slot is on the free list twice")
        if sum(self._live) + len(self._free_slots) != self.n_slots:
            raise CacheError("slots lost")
        for s in self._free_slots:
            if self._live[s]:
                raise CacheError(f"slot {s} is both free and live")
        for g in self.groups:
            g.pool.check()
            held = [p for s in range(self.n_slots) for p in g.pages[s] if p is not None]
            if len(set(held)) != len(held):
                raise CacheError("a page belongs to two sequences")
            if len(held) + g.pool.n_free != g.pool.n_pages:
                raise CacheError("pages held by slots and free pages do not add up")
            for s in range(self.n_slots):
                if not self._live[s] and g.pages[s]:
                    raise CacheError(f"free slot {s} still holds pages")
                for b, p in enumerate(g.pages[s]):
                    if g.table_host[s, b] != (-1 if p is None else p):
                        raise CacheError(f"block table of slot {s} disagrees with its page list")

    def kv_bytes_per_token(self) -> int:
        width = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.need.n_kv_heads * g.need.head_dim * width for g in self.groups)

    def read_kv(self, entry: int, slot: int, length: Optional[int] = None):
        """Keys and values of a sequence as [length, kv_heads, head_dim] (for tests)."""
        self._require_live(slot)
        view = self.view(entry)
        g, _ = self._entry_group[self._entry_source.get(entry, entry)]
        group = self.groups[g]
        length = self.seq_len[slot] if length is None else length
        ks, vs = [], []
        for pos in range(length):
            page = group.pages[slot][pos // PAGE]
            if page is None:
                raise CacheError(f"position {pos} of slot {slot} fell out of the window")
            ks.append(view.k[page, :, pos % PAGE, :])
            vs.append(view.v[page, :, pos % PAGE, :])
        return torch.stack(ks), torch.stack(vs)
