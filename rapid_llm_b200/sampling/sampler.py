"""Turns a step's logits rows into one token per row with the CUDA sampling kernel.

One launch handles a batch whose rows disagree about temperature, top-p and repetition
penalty, as the reference's batched sampler does with per-row tensors
(``rapid_llm/engine/sampler.py:448-520,689-696``).  A wholly greedy batch without penalties
passes no parameter arrays at all; otherwise every per-row parameter of the step (temperatures,
top-p, penalties, seeds, draw counters, the tokens a penalty looks at) is laid into ONE pinned buffer
and goes up in one asynchronous copy.  The sampled ids are written behind the kernels' fault
word, so the step's single device-to-host read brings both.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..ops import kernels
from .params import SamplingParams


class Sampler:
    def __init__(self, result: torch.Tensor) -> None:
        """``result``: int32 device buffer, word 0 = fault word, words 1.. = sampled ids."""
        self.result = result
        self.device = result.device
        self.max_rows = result.numel() - 1
        self._host = torch.zeros(result.numel(), dtype=torch.int32, pin_memory=True)
        # reads that are enqueued but not waited for yet: a few pinned buffers in rotation
        self._ring = [torch.zeros(result.numel(), dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._events = [torch.cuda.Event() for _ in range(4)]
        self._turn = 0
        # the step's sampling parameters: pinned buffers in rotation (one is written again only after the
        # copy that last read it has run) and their place on the device; both grow when a step needs more
        self._up_host: list[torch.Tensor | None] = [None] * 4
        self._up_events: list[torch.cuda.Event | None] = [None] * 4
        self._up_turn = 0
        self._up_device = torch.zeros(0, dtype=torch.int32, device=self.device)
        self._up_retired: list[torch.Tensor] = []

    def launch(
        self,
        logits: torch.Tensor,
        params: Sequence[SamplingParams],
        seeds: Sequence[int],
        counters: Sequence[int],
        generated: Sequence[Sequence[int]],
    ) -> None:
        """Sample into ``result[1 : 1 + rows]`` without reading anything back."""
        rows = logits.shape[0]
        if rows != len(params) or rows > self.max_rows:
            raise ValueError(f"{rows} logits rows for {len(params)} parameter sets (at most {self.max_rows})")
        if rows == 0:
            return
        out = self.result[1 : 1 + rows]
        use_penalty = any(p.repetition_penalty != 1.0 and len(g) for p, g in zip(params, generated))
        if all(p.is_greedy for p in params) and not use_penalty:
            kernels.sample(logits, out)
            return
        # one buffer of 32-bit words: temperature, top-p, penalty, counters (rows each), seeds (two words a row,
        # on an 8-byte boundary), then the offsets and the tokens the penalties look at
        offsets, flat = [0], []
        if use_penalty:
            for p, tokens in zip(params, generated):
                if p.repetition_penalty != 1.0:
                    flat.extend(tokens)
                offsets.append(len(flat))
        at_seeds = (4 * rows + 1) // 2 * 2
        at_offsets = at_seeds + 2 * rows
        at_seen = at_offsets + rows + 1
        words = at_seen + max(len(flat), 1)
        host = self._staging(words)
        as_float = host.view(np.float32)
        as_float[0:rows] = [p.temperature for p in params]
        as_float[rows : 2 * rows] = [p.top_p for p in params]
        as_float[2 * rows : 3 * rows] = [p.repetition_penalty for p in params]
        host[3 * rows : 4 * rows] = list(counters)
        host[at_seeds:at_offsets].view(np.int64)[:] = [seed if seed < 1 << 63 else seed - (1 << 64) for seed in seeds]
        if use_penalty:
            host[at_offsets:at_seen] = offsets
            host[at_seen : at_seen + len(flat)] = flat
        device = self._upload(words)
        floats = device[: 3 * rows].view(torch.float32)
        kernels.sample(
            logits, out, temperature=floats[:rows], top_p=floats[rows : 2 * rows],
            penalty=floats[2 * rows : 3 * rows] if use_penalty else None,
            seeds=device[at_seeds:at_offsets].view(torch.int64), counters=device[3 * rows : 4 * rows],
            seen_tokens=device[at_seen : at_seen + max(len(flat), 1)] if use_penalty else None,
            seen_offsets=device[at_offsets:at_seen] if use_penalty else None,
        )

    def _staging(self, words: int) -> np.ndarray:
        """The next pinned buffer of the rotation as int32 words, at least ``words`` long and no longer in use."""
        turn = self._up_turn
        if self._up_events[turn] is not None:
            self._up_events[turn].synchronize()
        if self._up_host[turn] is None or self._up_host[turn].numel() < words:
            self._up_host[turn] = torch.zeros(max(1024, 1 << (words - 1).bit_length()), dtype=torch.int32, pin_memory=True)
        return self._up_host[turn].numpy()

    def _upload(self, words: int) -> torch.Tensor:
        """One asynchronous copy of the staged words; returns their place on the device."""
        turn = self._up_turn
        self._up_turn = (turn + 1) % len(self._up_host)
        if self._up_device.numel() < words:
            self._up_retired.append(self._up_device)       # a kernel in flight may still read it
            self._up_device = torch.zeros(max(1024, 1 << (words - 1).bit_length()), dtype=torch.int32, device=self.device)
        self._up_device[:words].copy_(self._up_host[turn][:words], non_blocking=True)
        if self._up_events[turn] is None:
            self._up_events[turn] = torch.cuda.Event()
        self._up_events[turn].record()
        return self._up_device

    def read(self, rows: int) -> list[int]:
        """The step's one device-to-host read: fault word and ``rows`` sampled ids."""
        self._host[: rows + 1].copy_(self.result[: rows + 1], non_blocking=False)
        values = self._host[: rows + 1].tolist()
        if values[0]:
            self.result[:1].zero_()
            raise RuntimeError(f"a kernel reported a fault: {kernels.describe_fault(values[0])}")
        return values[1:]

    def read_later(self, rows: int) -> tuple[int, int]:
        """Enqueue the read of the fault word and ``rows`` ids; :meth:`collect` waits for it."""
        turn = self._turn
        self._turn = (turn + 1) % len(self._ring)
        self._ring[turn][: rows + 1].copy_(self.result[: rows + 1], non_blocking=True)
        self._events[turn].record()
        return turn, rows

    def collect(self, ticket: tuple[int, int]) -> list[int]:
        turn, rows = ticket
        self._events[turn].synchronize()
        values = self._ring[turn][: rows + 1].tolist()
        if values[0]:
            self.result[:1].zero_()
            raise RuntimeError(f"a kernel reported a fault: {kernels.describe_fault(values[0])}")
        return values[1:]

    def sample(self, logits, params, seeds, counters, generated) -> list[int]:
        self.launch(logits, params, seeds, counters, generated)
        return self.read(logits.shape[0])
