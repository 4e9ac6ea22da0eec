"""One step's batch as the parts see it: packed tokens plus per-request metadata.

The reference describes a pass with ``ModelInput`` / ``AttentionMetadata`` and runs
one *kind* of pass at a time over padded rectangles (``rapid_llm/executor/worker.py:69-126``,
``rapid_llm/executor/attention_metadata.py:19-72``).  Here a step is one packed ragged
batch: portions of prompts beside single decoded tokens, no padding tokens.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch


@dataclass
class GroupView:
    """What a cache group contributes to a step.

    Attributes:
        block_table: int32 ``[slots, max_pages]`` on the device; entry ``[s, p // page]``
            is the page that holds position ``p`` of the request in slot ``s``.
        kv_dest: int32 ``[T]``; ``page * page_size + offset`` where each token of the step
            writes its key and value.
        page_size: Tokens per page.
        window: Positions a query reaches back (its own included); 0 = all of them.
    """

    block_table: torch.Tensor
    kv_dest: torch.Tensor
    page_size: int
    window: int


@dataclass
class LayerCache:
    """What one entry of the run order may touch.

    Attributes:
        group: Index into :attr:`StepBatch.groups`, or ``None`` when the mixer keeps no pages.
        pages: This entry's page tensor ``[pages, 2, kv_heads, page_size, head_dim]``.
        writes: ``False`` when the entry reads another entry's cache and must not write.
        state: Per-request state of fixed size, ``[slots, *shape]``, or ``None``.
    """

    group: int | None = None
    pages: torch.Tensor | None = None
    writes: bool = True
    state: torch.Tensor | None = None


class Workspace:
    """Named activation buffers; after warm-up a step allocates nothing.

    A buffer is created with ``max_tokens`` rows (or ``min_rows`` if given) the first time
    its name is asked for and grows only if a later step asks for more rows.  A buffer that
    is replaced is kept alive, since a captured graph may still hold its address.
    """

    def __init__(self, max_tokens: int, device: torch.device) -> None:
        self.max_tokens = max_tokens
        self.device = device
        self._buffers: dict[tuple[str, int, torch.dtype], torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []
        # the views handed out, by (name, cols, dtype, rows): a step asks for hundreds of them, and making
        # one costs as much as a launch's other bookkeeping
        self._views: dict[tuple[str, int, torch.dtype, int], torch.Tensor] = {}

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype, min_rows: int | None = None) -> torch.Tensor:
        view = self._views.get((name, cols, dtype, rows))
        if view is not None:
            return view
        key = (name, cols, dtype)
        buffer = self._buffers.get(key)
        if buffer is None or buffer.shape[0] < rows:
            want = max(rows, self.max_tokens if min_rows is None else min_rows)
            if buffer is not None:
                self._retired.append(buffer)
                for stale in [k for k in self._views if k[:3] == key]:
                    del self._views[stale]
            buffer = torch.empty((want, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buffer
        view = buffer[:rows]
        if len(self._views) < 4096:
            self._views[(name, cols, dtype, rows)] = view
        return view

    def nbytes(self) -> int:
        live = sum(b.numel() * b.element_size() for b in self._buffers.values())
        return live + sum(b.numel() * b.element_size() for b in self._retired)


@dataclass
class StepBatch:
    """Device and host views of one step.

    Device tensors (int32): ``token_ids [T]``, ``positions [T]``, ``token_slot [T]``,
    ``cu_seqlens [n + 1]``, ``entry_slot [n]``, ``entry_start [n]`` (tokens the request had
    cached before this step), ``logit_rows [R]`` (rows of the packed batch whose logits are
    wanted).  The ``h_*`` arrays are their host copies, for launch decisions without a sync.
    """

    num_tokens: int
    num_entries: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_slot: torch.Tensor
    cu_seqlens: torch.Tensor
    entry_slot: torch.Tensor
    entry_start: torch.Tensor
    logit_rows: torch.Tensor
    h_cu_seqlens: np.ndarray
    h_entry_slot: np.ndarray
    h_entry_start: np.ndarray
    max_query_len: int
    max_context_len: int
    groups: list[GroupView]
    workspace: Workspace
    fault: torch.Tensor
    dtype: torch.dtype
    decode_only: bool = False
    extras: dict[str, Any] = field(default_factory=dict)
    feedback: torch.Tensor | None = None     # ids the previous step sampled, for token ids -(row + 1)
    # Parts may queue their products for one persistent kernel (``ops.gemm`` with ``defer``): set by the model's
    # forward pass, which runs the queue before anything but a kernel of ``ops.kernels`` reads a result.  A part
    # called by itself gets finished results.
    defer_products: bool = False

    @property
    def num_logit_rows(self) -> int:
        return int(self.logit_rows.numel())
