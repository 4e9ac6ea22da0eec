"""Turns a step's logits rows into one token per row with the CUDA sampling kernel.

One launch handles a batch whose rows disagree about temperature, top-p and repetition
penalty, as the reference's batched sampler does with per-row tensors
(``rapid_llm/engine/sampler.py:448-520,689-696``).  A wholly greedy batch without penalties
passes no parameter arrays at all.  The sampled ids are written behind the kernels' fault
word, so the step's single device-to-host read brings both.

Log-probability records (``SamplingParams.logprobs`` / ``prompt_logprobs``) come from a second
kernel over the same logits rows, under the distribution the row was drawn from, as the
reference computes them after the draw (``rapid_llm/engine/sampler.py:698-718``); their read
rides behind the read of the ids.
"""

from __future__ import annotations

from typing import Sequence

import torch

from ..ops import kernels
from .params import PositionLogprobs, SamplingParams


class ScoreRead:
    """Log-probabilities on their way to the host: pinned copies and the event behind them."""

    def __init__(self, chosen, top_values, top_ids, event) -> None:
        self.chosen, self.top_values, self.top_ids, self.event = chosen, top_values, top_ids, event

    def records(self, token_ids: Sequence[int], widths: Sequence[int | None]) -> list[PositionLogprobs | None]:
        """One record per row (``None`` where ``widths`` has ``None``); waits for the copies."""
        self.event.synchronize()
        chosen = self.chosen.tolist()
        values = self.top_values.tolist() if self.top_values is not None else None
        ids = self.top_ids.tolist() if self.top_ids is not None else None
        out: list[PositionLogprobs | None] = []
        for row, (token, width) in enumerate(zip(token_ids, widths)):
            if width is None:
                out.append(None)
                continue
            kept = [] if ids is None else [j for j in range(min(width, len(ids[row]))) if ids[row][j] >= 0]
            out.append(PositionLogprobs(
                int(token), chosen[row],
                tuple(ids[row][j] for j in kept), tuple(values[row][j] for j in kept),
            ))
        return out


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
        self._row_arguments: dict = {}

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
        self._row_arguments = {}
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
        # the distribution of each row, for the records that may be asked for next
        self._row_arguments = {"temperature": floats[0], "penalty": floats[2] if use_penalty else None,
                               "seen_tokens": seen_t, "seen_offsets": offsets_t}

    def score_sampled(self, logits: torch.Tensor, width: int) -> ScoreRead:
        """Records for the rows :meth:`launch` has just sampled from ``logits``: the sampled
        token's log-probability and the ``width`` most likely, under the row's own temperature
        and penalty.  Enqueues the kernel and the copies; nothing is waited for."""
        return self._score(logits, self.result[1 : 1 + logits.shape[0]], width, self._row_arguments)

    def score_given(self, logits: torch.Tensor, token_ids: Sequence[int], width: int) -> ScoreRead:
        """Records for known tokens (a prompt's own) under the raw logits of their rows."""
        ids = torch.tensor(list(token_ids), dtype=torch.int32).to(self.device, non_blocking=True)
        return self._score(logits, ids, width, {})

    def _score(self, logits, ids, width, arguments) -> ScoreRead:
        rows = logits.shape[0]
        chosen = torch.empty(rows, dtype=torch.float32, device=self.device)
        top_values = top_ids = None
        if width > 0:
            top_values = torch.empty((rows, width), dtype=torch.float32, device=self.device)
            top_ids = torch.empty((rows, width), dtype=torch.int32, device=self.device)
        kernels.logprobs(logits, ids, chosen, top_values=top_values, top_ids=top_ids, **arguments)

        def to_host(tensor):
            if tensor is None:
                return None
            host = torch.empty(tensor.shape, dtype=tensor.dtype, pin_memory=True)
            host.copy_(tensor, non_blocking=True)
            return host

        copies = [to_host(chosen), to_host(top_values), to_host(top_ids)]
        event = torch.cuda.Event()
        event.record()
        return ScoreRead(*copies, event)

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
