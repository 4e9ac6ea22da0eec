"""Host-side bookkeeping of the paged cache: pools, groups, block tables, slots.

Keys and values live in fixed-size pages.  Layers with the same needs (all keys, or a
window of them, for a given head geometry) form a *group* with a pool and a block table of
its own; every layer of a group uses the same page ids.  A request holds a *slot* (its row
in every block table and in every per-request state tensor) and, per group, a list of
pages.  Pages go back to the pool when the request ends, or, in a windowed group, as soon
as the window has passed them; they are handed out again to whoever asks next.

The reference keeps the same bookkeeping in ``BlockPool`` (null block 0, all-or-nothing
``get_new_blocks``, freed blocks reused first: ``rapid_llm/engine/block_pool.py:156-303``),
``KVCacheCoordinator`` (per-group block lists, ``remove_skipped_blocks`` for windows:
``rapid_llm/engine/kv_cache_spec.py:480-549,595-634``) and a free-slot stack
(``rapid_llm/engine/batch_planner.py:348``), but expands blocks to token rows for the
device (``rapid_llm/executor/slot_batch.py:130-178``); here tables hold page ids end to end.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np

from ..parts.base import CacheNeed

NULL_PAGE = 0


class CacheError(RuntimeError):
    """A bookkeeping invariant was violated (double free, unknown request, ...)."""


class PagePool:
    """Page ids ``1 .. num_pages``; id 0 is the null page and is never handed out."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(1, num_pages + 1))
        self._held = [False] * (num_pages + 1)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, count: int) -> list[int] | None:
        """``count`` pages, or ``None`` (and nothing taken) when the pool is short."""
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            return None
        pages = [self._free.popleft() for _ in range(count)]
        for page in pages:
            if self._held[page]:
                raise CacheError(f"page {page} was in the free list while held")
            self._held[page] = True
        return pages

    def free(self, pages: Sequence[int]) -> None:
        """Give pages back; they are the next to be handed out."""
        real = [page for page in pages if page != NULL_PAGE]
        for page in real:                       # check everything before anything changes
            if not 1 <= page <= self.num_pages:
                raise CacheError(f"page {page} does not belong to this pool")
            if not self._held[page]:
                raise CacheError(f"page {page} freed twice")
        if len(set(real)) != len(real):
            raise CacheError("a page is named twice in one free")
        for page in real:
            self._held[page] = False
        for page in reversed(real):
            self._free.appendleft(page)

    def check(self) -> None:
        """Raise unless every page is exactly once either free or held."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise CacheError("a page is in the free list twice")
        for page in free:
            if self._held[page]:
                raise CacheError(f"page {page} is both free and held")
        if len(free) + sum(self._held[1:]) != self.num_pages:
            raise CacheError("a page was lost")


@dataclass(frozen=True)
class GroupSpec:
    """One cache group: its need and the positions of the run order that use it."""

    need: CacheNeed
    entries: tuple[int, ...]

    @property
    def window(self) -> int:
        return self.need.window if self.need.kind == "window" else 0


def plan_groups(needs: Sequence[CacheNeed | None]) -> tuple[list[GroupSpec], list[int | None]]:
    """Group the run order's cache needs; returns the groups and each entry's group index."""
    keys: list[tuple] = []
    members: list[list[int]] = []
    first_need: list[CacheNeed] = []
    entry_group: list[int | None] = []
    for position, need in enumerate(needs):
        if need is None:
            entry_group.append(None)
            continue
        if need.kind not in ("full", "window"):
            raise ValueError(f"unknown cache kind {need.kind!r}")
        if need.kind == "window" and need.window < 1:
            raise ValueError("a windowed cache needs window >= 1")
        if need.elements_per_token() < 1:
            raise ValueError("a cache need must give kv heads and a head size, or the shape of a token's row")
        key = need.group_key()
        if key not in keys:
            keys.append(key)
            members.append([])
            first_need.append(need)
        index = keys.index(key)
        members[index].append(position)
        entry_group.append(index)
    groups = [GroupSpec(first_need[i], tuple(members[i])) for i in range(len(keys))]
    return groups, entry_group


@dataclass
class _Held:
    slot: int
    num_tokens: int = 0                      # tokens whose K/V are (being) cached
    pages: list[list[int]] = field(default_factory=list)   # per group, NULL_PAGE where released


class CacheManager:
    """Slots, pools and block tables for ``max_num_seqs`` live requests.

    ``num_pages`` may be one number (every group gets that many) or one per group.
    ``extra_table_rows`` appends block-table rows that no request ever gets; they stay all
    null and serve as the slot of padding rows.
    """

    def __init__(
        self,
        groups: Sequence[GroupSpec],
        *,
        page_size: int,
        num_pages: int | Sequence[int],
        max_num_seqs: int,
        max_seq_len: int,
        extra_table_rows: int = 0,
    ) -> None:
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.max_num_seqs = int(max_num_seqs)
        self.max_seq_len = int(max_seq_len)
        self.max_pages_per_seq = -(-self.max_seq_len // self.page_size)
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise ValueError("num_pages must be one number or one per group")
        self.pools = [PagePool(count) for count in counts]
        self.block_tables = [
            np.zeros((self.max_num_seqs + extra_table_rows, self.max_pages_per_seq), dtype=np.int32)
            for _ in self.groups
        ]
        self._free_slots = list(range(self.max_num_seqs - 1, -1, -1))
        self._held: dict[Hashable, _Held] = {}
        self.dirty_slots: list[set[int]] = [set() for _ in self.groups]

    # -- queries ------------------------------------------------------------------ #
    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def has(self, request_id: Hashable) -> bool:
        return request_id in self._held

    def slot_of(self, request_id: Hashable) -> int:
        return self._get(request_id).slot

    def num_tokens(self, request_id: Hashable) -> int:
        return self._get(request_id).num_tokens

    def pages_of(self, request_id: Hashable) -> list[list[int]]:
        """Per group, the request's pages in position order (0 where released)."""
        return [list(pages) for pages in self._get(request_id).pages]

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def _get(self, request_id: Hashable) -> _Held:
        try:
            return self._held[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} holds no slot") from None

    # -- life of a request ---------------------------------------------------------- #
    def admit(self, request_id: Hashable) -> int | None:
        """Give the request a slot; ``None`` when all are taken."""
        if request_id in self._held:
            raise CacheError(f"request {request_id!r} is already admitted")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._held[request_id] = _Held(slot=slot, pages=[[] for _ in self.groups])
        for table, dirty in zip(self.block_tables, self.dirty_slots):
            if table[slot].any():
                table[slot] = NULL_PAGE
                dirty.add(slot)
        return slot

    def pages_needed(self, request_id: Hashable, upto_tokens: int) -> list[int]:
        """New pages per group that growing to ``upto_tokens`` would take."""
        held = self._get(request_id)
        last_page = (upto_tokens - 1) // self.page_size
        return [max(0, last_page + 1 - len(pages)) for pages in held.pages]

    def reserve(self, request_id: Hashable, upto_tokens: int) -> bool:
        """Make room for positions ``< upto_tokens`` in every group, all or nothing."""
        held = self._get(request_id)
        if upto_tokens > self.max_seq_len:
            raise CacheError(
                f"request {request_id!r} would reach {upto_tokens} tokens, beyond max_seq_len {self.max_seq_len}"
            )
        if upto_tokens < held.num_tokens:
            raise CacheError("a request cannot shrink")
        needed = self.pages_needed(request_id, upto_tokens)
        if any(count > pool.num_free for count, pool in zip(needed, self.pools)):
            return False
        for index, count in enumerate(needed):
            if not count:
                continue
            fresh = self.pools[index].allocate(count)
            assert fresh is not None
            start = len(held.pages[index])
            held.pages[index].extend(fresh)
            self.block_tables[index][held.slot, start : start + count] = fresh
            self.dirty_slots[index].add(held.slot)
        held.num_tokens = upto_tokens
        return True

    def release_passed(self, request_id: Hashable) -> int:
        """Free the pages of windowed groups that no later query can reach.

        The next query sits at position ``num_tokens`` and reaches back to
        ``num_tokens - window + 1``; pages wholly below that are dead.  Returns how many
        pages were given back.
        """
        held = self._get(request_id)
        released = 0
        for index, group in enumerate(self.groups):
            window = group.window
            if not window:
                continue
            oldest = max(held.num_tokens - window + 1, 0)
            keep_from = min(oldest // self.page_size, len(held.pages[index]))
            dead = [page for page in held.pages[index][:keep_from] if page != NULL_PAGE]
            if not dead:
                continue
            for position in range(keep_from):
                held.pages[index][position] = NULL_PAGE
            self.block_tables[index][held.slot, :keep_from] = NULL_PAGE
            self.dirty_slots[index].add(held.slot)
            self.pools[index].free(dead)
            released += len(dead)
        return released

    def release(self, request_id: Hashable) -> None:
        """The request ended: all its pages and its slot go back."""
        held = self._held.pop(request_id, None)
        if held is None:
            raise CacheError(f"request {request_id!r} released twice or never admitted")
        for index, pages in enumerate(held.pages):
            self.pools[index].free([page for page in reversed(pages) if page != NULL_PAGE])
            if pages:
                self.block_tables[index][held.slot, : len(pages)] = NULL_PAGE
                self.dirty_slots[index].add(held.slot)
        self._free_slots.append(held.slot)

    # -- per-step views ------------------------------------------------------------ #
    def kv_destinations(self, group: int, slot: int, start: int, count: int) -> np.ndarray:
        """``page * page_size + offset`` for positions ``start .. start + count - 1``."""
        positions = np.arange(start, start + count, dtype=np.int64)
        pages = self.block_tables[group][slot, positions // self.page_size].astype(np.int64)
        return (pages * self.page_size + positions % self.page_size).astype(np.int32)

    def take_dirty(self, group: int) -> list[int]:
        slots = sorted(self.dirty_slots[group])
        self.dirty_slots[group].clear()
        return slots

    def check(self) -> None:
        """Raise unless no page is lost, held twice or both held and free."""
        for index, pool in enumerate(self.pools):
            pool.check()
            owned: list[int] = []
            for held in self._held.values():
                owned.extend(page for page in held.pages[index] if page != NULL_PAGE)
            if len(set(owned)) != len(owned):
                raise CacheError(f"group {index}: a page is held by two requests")
            if len(owned) != pool.num_held:
                raise CacheError(
                    f"group {index}: requests hold {len(owned)} pages, the pool says {pool.num_held}"
                )
        slots = [held.slot for held in self._held.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a slot is held twice or both held and free")
        if len(slots) + len(self._free_slots) != self.max_num_seqs:
            raise CacheError("a slot was lost")
