"""Device side of the cache: page tensors, block tables, per-request state tensors.

Per group one tensor ``[entries, pages + 1, *page]`` where ``page`` is what the group's mixers
asked for (``CacheNeed.page_shape``: a key and a value per kv head, ``[2, kv_heads, page_size, head_dim]``,
unless the mixer names a row per token of its own); page 0
is the null page that padding and released table entries point at, one int32 block table
``[slots, max_pages]`` mirrored from the host bookkeeping (the step function uploads the rows that changed with its metadata), and
per run-order entry that asks for it one state tensor ``[slots, *shape]``, zeroed when a
slot is handed to a new request.  The reference stores one row per token,
``[max_tokens, 2 * kv_heads, head_dim]`` per layer (``rapid_llm/executor/kv_cache_manager.py:230-249``).
"""

from __future__ import annotations

from typing import Sequence

import torch

from ..parts.base import StateNeed
from .manager import CacheManager


class CacheStorage:
    def __init__(
        self,
        manager: CacheManager,
        entry_group: Sequence[int | None],
        state_needs: Sequence[StateNeed | None],
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        self.manager = manager
        self.dtype = dtype
        self.device = device
        self.entry_group = list(entry_group)
        self.pages: list[torch.Tensor] = []
        for group, pool in zip(manager.groups, manager.pools):
            need = group.need
            shape = (len(group.entries), pool.num_pages + 1, *need.page_shape(manager.page_size))
            self.pages.append(torch.zeros(shape, dtype=dtype, device=device))
        self.num_rows = manager.block_tables[0].shape[0] if manager.block_tables else manager.max_num_seqs
        self.block_tables = [
            torch.zeros(table.shape, dtype=torch.int32, device=device) for table in manager.block_tables
        ]
        self.states: list[torch.Tensor | None] = [
            None if need is None
            else torch.zeros((self.num_rows, *need.shape), dtype=need.dtype, device=device)
            for need in state_needs
        ]
        # a state tensor of zero bytes keeps the path alive for architectures without state
        self.empty_state = torch.zeros((self.num_rows, 0), dtype=torch.uint8, device=device)

    def entry_pages(self, position: int, source: int | None = None) -> tuple[int | None, torch.Tensor | None]:
        """Group index and page tensor of one run-order entry (or of the entry it reads)."""
        owner = position if source is None else source
        group = self.entry_group[owner]
        if group is None:
            return None, None
        local = self.manager.groups[group].entries.index(owner)
        return group, self.pages[group][local]

    def reset_state(self, slot: int) -> None:
        for state in self.states:
            if state is not None:
                state[slot].zero_()

    def nbytes(self) -> int:
        total = sum(p.numel() * p.element_size() for p in self.pages)
        total += sum(s.numel() * s.element_size() for s in self.states if s is not None)
        return total
