"""Result records of a generation call, shaped like the reference's
(``rapid_llm/engine/outputs.py:22-59``): one ``RequestOutput`` per prompt holding its
completions; token ids ride along because random-weight models have no tokenizer.
``logprobs`` (one record per generated token) and ``prompt_logprobs`` (one per prompt position,
``None`` at position 0) are filled when the request's ``SamplingParams`` ask for them and are
``None`` otherwise."""

from __future__ import annotations

from dataclasses import dataclass, field

from ..sampling.params import PositionLogprobs


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    finish_reason: str | None
    logprobs: list[PositionLogprobs] | None = None


@dataclass
class RequestOutput:
    prompt: str | None
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput] = field(default_factory=list)
    metrics: dict = field(default_factory=dict)
    prompt_logprobs: list[PositionLogprobs | None] | None = None

    @property
    def text(self) -> str:
        return self.outputs[0].text if self.outputs else ""

    @property
    def token_ids(self) -> list[int]:
        return self.outputs[0].token_ids if self.outputs else []
