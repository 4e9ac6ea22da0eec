"""Result records of a generation call, shaped like the reference's
(``rapid_llm/engine/outputs.py:22-59``): one ``RequestOutput`` per prompt holding its
completions; token ids ride along because random-weight models have no tokenizer.  The
reference's ``logprobs`` and ``prompt_logprobs`` attributes exist and are always ``None``
(log-probabilities are not reported)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    finish_reason: str | None
    logprobs: None = None


@dataclass
class RequestOutput:
    prompt: str | None
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput] = field(default_factory=list)
    metrics: dict = field(default_factory=dict)
    prompt_logprobs: None = None

    @property
    def text(self) -> str:
        return self.outputs[0].text if self.outputs else ""

    @property
    def token_ids(self) -> list[int]:
        return self.outputs[0].token_ids if self.outputs else []
