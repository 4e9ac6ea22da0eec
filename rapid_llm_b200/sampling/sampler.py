"""Turns a step's logits rows into one token per row with the CUDA sampling kernel.

One launch handles a batch whose rows disagree about temperature, top-p and repetition
penalty, as the reference's batched sampler does with per-row tensors
(``rapid_llm/engine/sampler.py:448-520,689-696``).  A wholly greedy batch without penalties
passes no parameter arrays at all.  The sampled ids are written behind the kernels' fault
word, so the step's single device-to-host read brings both.
"""

from __future__ import annotations

from typing import Sequence

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
        device = self.device
        floats = torch.tensor(
            [[p.temperature for p in params], [p.top_p for p in params], [p.repetition_penalty for p in params]],
            dtype=torch.float32,
        ).to(device, non_blocking=True)
        seed_t = torch.tensor(list(seeds), dtype=torch.int64).to(device, non_blocking=True)
        counter_t = torch.tensor(list(counters), dtype=torch.int32).to(device, non_blocking=True)
        seen_t = offsets_t = None
        if use_penalty:
            offsets, flat = [0], []
            for p, tokens in zip(params, generated):
                if p.repetition_penalty != 1.0:
                    flat.extend(tokens)
                offsets.append(len(flat))
            seen_t = torch.tensor(flat or [0], dtype=torch.int32).to(device, non_blocking=True)
            offsets_t = torch.tensor(offsets, dtype=torch.int32).to(device, non_blocking=True)
        kernels.sample(
            logits, out, temperature=floats[0], top_p=floats[1], penalty=floats[2] if use_penalty else None,
            seeds=seed_t, counters=counter_t, seen_tokens=seen_t, seen_offsets=offsets_t,
        )

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
