"""The device executor under the scheduler: planned entries in, sampled tokens out.

It turns the plan into one call of the step function, samples the rows that reached the end
of their request's tokens, and reads the sampled ids (with the kernels' fault word) back in
the step's single device-to-host copy, as the reference does once per step
(``rapid_llm/engine/scheduler.py:1000-1005``).  Requests that ask for log-probability records
get them from the same logits: the sampled rows under their own distribution, the prompt's
positions (whose logits are asked of the step function as extra rows) under the raw one.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

from ..sampling.params import PositionLogprobs
from ..sampling.sampler import Sampler, ScoreRead
from .runner import ModelRunner, StepEntry


@dataclass
class StepTicket:
    """What a launched step will bring: the sampled ids and, where asked for, records."""

    ids: tuple[int, int] | None = None                   # the sampler's read of the ids
    sampled: ScoreRead | None = None
    sampled_widths: list[int | None] = field(default_factory=list)      # per sampled row
    prompt: ScoreRead | None = None
    prompt_rows: list[tuple[object, int, int, int]] = field(default_factory=list)   # request, position, token, width
    token_ids: list[int] | None = None                   # the ids, once collected


class DeviceExecutor:
    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self.cache = runner.cache
        self.sampler = Sampler(runner.result)

    def admit(self, request_id: Hashable) -> bool:
        return self.runner.admit(request_id)

    def release(self, request_id: Hashable) -> None:
        self.runner.release(request_id)

    def launch(self, entries: Sequence):
        """Enqueue the batch, its sampling and the read of the sampled ids; returns a ticket
        (``None`` for a step that brings nothing back).

        A token id ``-(row + 1)`` among the entries' tokens is taken on the device from row
        ``row`` of the ids the previously launched batch sampled."""
        step_entries = []
        prompt_rows: list[tuple[object, int, int, int]] = []
        for e in entries:
            request = e.request
            score: list[int] = []
            width = request.params.prompt_logprobs
            if width is not None:
                # position p predicts the prompt's token p + 1; the last position predicts the first
                # generated token and is the sampler's business
                prompt = request.prompt_token_ids
                for place in range(len(e.tokens)):
                    target = e.start + place + 1
                    if target < len(prompt):
                        score.append(place)
                        prompt_rows.append((request, target, prompt[target], width))
            step_entries.append(StepEntry(request.request_id, e.tokens, [len(e.tokens) - 1] if e.samples else [], score))
        sampling = [e.request for e in entries if e.samples]
        decode_only = all(len(e.tokens) == 1 and e.samples for e in entries) and not prompt_rows
        if decode_only and self.runner.config.use_cuda_graph and len(entries) <= self.runner.config.max_num_seqs:
            logits = self.runner.step_decode(step_entries)
        else:
            logits = self.runner.step(step_entries)
        if not sampling and not prompt_rows:
            return None
        ticket = StepTicket(prompt_rows=prompt_rows)
        if sampling:
            sampled_logits = logits[: len(sampling)]
            self.sampler.launch(
                sampled_logits,
                [r.params for r in sampling],
                [r.seed for r in sampling],
                [len(r.output_token_ids) for r in sampling],
                [r.output_token_ids for r in sampling],
            )
            ticket.sampled_widths = [r.params.logprobs for r in sampling]
            widths = [w for w in ticket.sampled_widths if w is not None]
            if widths:
                ticket.sampled = self.sampler.score_sampled(sampled_logits, max(widths))
            ticket.ids = self.sampler.read_later(len(sampling))
        if prompt_rows:
            ticket.prompt = self.sampler.score_given(
                logits[len(sampling):], [token for _, _, token, _ in prompt_rows], max(w for *_, w in prompt_rows)
            )
        return ticket

    def collect(self, ticket) -> list[int]:
        """The ids a launched step sampled, one per sampled row (waits for them)."""
        if ticket is None:
            return []
        if ticket.token_ids is None:
            ticket.token_ids = self.sampler.collect(ticket.ids) if ticket.ids is not None else []
        return ticket.token_ids

    def records(self, ticket) -> tuple[list[PositionLogprobs | None], list[tuple[object, int, PositionLogprobs]]]:
        """The step's log-probability records: one per sampled row (``None`` where none was
        asked for), and ``(request, prompt position, record)`` for every scored prompt position."""
        if ticket is None:
            return [], []
        sampled: list[PositionLogprobs | None] = [None] * len(ticket.sampled_widths)
        if ticket.sampled is not None:
            sampled = ticket.sampled.records(self.collect(ticket), ticket.sampled_widths)
        prompt = []
        if ticket.prompt is not None:
            made = ticket.prompt.records([token for _, _, token, _ in ticket.prompt_rows], [w for *_, w in ticket.prompt_rows])
            prompt = [(request, position, record) for (request, position, _, _), record in zip(ticket.prompt_rows, made)]
        return sampled, prompt

    def execute(self, entries: Sequence) -> list[int]:
        return self.collect(self.launch(entries))
