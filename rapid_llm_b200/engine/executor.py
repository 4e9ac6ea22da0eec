"""The device executor under the scheduler: planned entries in, sampled tokens out.

It turns the plan into one call of the step function, samples the rows that reached the end
of their request's tokens, and reads the sampled ids (with the kernels' fault word) back in
the step's single device-to-host copy, as the reference does once per step
(``rapid_llm/engine/scheduler.py:1000-1005``).
"""

from __future__ import annotations

from typing import Hashable, Sequence

from ..sampling.sampler import Sampler
from .runner import ModelRunner, StepEntry


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
        """Enqueue the batch, its sampling and the read of the sampled ids; returns a ticket.

        A token id ``-(row + 1)`` among the entries' tokens is taken on the device from row
        ``row`` of the ids the previously launched batch sampled."""
        step_entries = [
            StepEntry(e.request.request_id, e.tokens, [len(e.tokens) - 1] if e.samples else [])
            for e in entries
        ]
        sampling = [e.request for e in entries if e.samples]
        decode_only = all(len(e.tokens) == 1 and e.samples for e in entries)
        if decode_only and self.runner.config.use_cuda_graph and len(entries) <= self.runner.config.max_num_seqs:
            logits = self.runner.step_decode(step_entries)
        else:
            logits = self.runner.step(step_entries)
        if not sampling:
            return None
        self.sampler.launch(
            logits,
            [r.params for r in sampling],
            [r.seed for r in sampling],
            [len(r.output_token_ids) for r in sampling],
            [r.output_token_ids for r in sampling],
        )
        return self.sampler.read_later(len(sampling))

    def collect(self, ticket) -> list[int]:
        return [] if ticket is None else self.sampler.collect(ticket)

    def execute(self, entries: Sequence) -> list[int]:
        return self.collect(self.launch(entries))
