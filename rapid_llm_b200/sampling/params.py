"""Per-request decoding parameters, with the reference's names, meanings and checks.

``rapid_llm/engine/sampler.py:44-97``: ``temperature`` 0 means greedy; ``top_p`` in (0, 1];
``max_gen_len`` ``None`` fills the context; ``repetition_penalty`` > 0 with 1.0 off;
values are validated at construction.  ``seed`` is an addition: draws come from a
counter-based generator keyed by (seed, index of the generated token), so a request's
tokens do not depend on what else is in the batch.  ``stop_on_repeat`` ends a request whose
generated text loops (finish reason ``"repeat"``); the test is on decoded text, so it acts only
when the model folder has a tokenizer, and requests of token ids alone are never ended by it.
``logprobs`` and ``prompt_logprobs`` (reporting, not sampling) are accepted only as ``None``;
any other value is refused at construction rather than ignored.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.6
    top_p: float = 0.9
    max_gen_len: int | None = None
    repetition_penalty: float = 1.1
    stop_on_repeat: bool = True
    logprobs: int | None = None
    prompt_logprobs: int | None = None
    seed: int | None = None

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.max_gen_len is not None and self.max_gen_len < 1:
            raise ValueError(f"max_gen_len must be >= 1 or None, got {self.max_gen_len}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if self.logprobs is not None or self.prompt_logprobs is not None:
            raise ValueError("logprobs and prompt_logprobs are not reported by this engine; leave them None")
        if self.seed is not None and not 0 <= self.seed < 2**63:
            raise ValueError(f"seed must be in [0, 2**63), got {self.seed}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0

    @classmethod
    def greedy(cls, max_gen_len: int | None = None) -> "SamplingParams":
        return cls(temperature=0.0, top_p=1.0, repetition_penalty=1.0, max_gen_len=max_gen_len)
