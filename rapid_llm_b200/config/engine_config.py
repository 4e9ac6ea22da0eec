"""Run-time sizes of an engine, apart from the model's own configuration.

The reference keeps ``max_seq_len`` and the cache dtype on its model
configuration (``rapid_llm/models/config.py:82-103``) and the batching limits on
``SchedulerConfig`` (``rapid_llm/engine/batch_planner.py:151-240``); the defaults
below are the reference's.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "fp32": torch.float32,
}


def parse_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"engine dtype must be bfloat16 or float32, got {name!r}") from None


@dataclass(frozen=True)
class EngineConfig:
    """Sizes the engine is built for.

    Attributes:
        dtype: ``torch.bfloat16`` (serving precision) or ``torch.float32`` (every
            product and sum in true 32-bit).
        max_seq_len: Longest sequence (prompt plus generated) a request may reach.
        page_size: Tokens per cache page.
        num_pages: Pages per cache group, the reserved null page not counted;
            ``None`` sizes the pool from free device memory.
        max_num_seqs: Requests live at a time (= rows of the block tables).
        max_num_batched_tokens: Tokens one step may carry.
        max_chunk_size: Largest portion of one prompt in a step; 0 is the reference's older way
            of switching chunked prefill off and is folded into ``enable_chunked_prefill``.
        enable_chunked_prefill: Cut prompts into portions; off = whole prompts only, and a step
            must then be able to carry the longest prompt (``max_num_batched_tokens >=
            max_seq_len``), or such a prompt would wait for ever.
        enable_preemption: Let a request that cannot grow evict the youngest one.
        memory_fraction: Share of the device's memory the cache may claim when
            ``num_pages`` is ``None``.
        use_cuda_graph: Replay decode-only steps from captured graphs.
        run_ahead: Enqueue a step before the host has read the previous step's tokens (they
            are fed back on the device); off = read every step's tokens before planning the next.
        use_dependent_launch: Launch the step's kernels as programmatic dependents of one
            another, so that each starts (and fetches its weights) while its predecessor drains.
    """

    dtype: torch.dtype = torch.bfloat16
    max_seq_len: int = 2048
    page_size: int = 16
    num_pages: int | None = None
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 8192
    max_chunk_size: int = 512
    enable_chunked_prefill: bool = True
    enable_preemption: bool = True
    memory_fraction: float = 0.9
    use_cuda_graph: bool = True
    use_dependent_launch: bool = True
    run_ahead: bool = True

    def __post_init__(self) -> None:
        parse_dtype(self.dtype)
        if self.max_seq_len < 2:
            raise ValueError(f"max_seq_len must be >= 2 (a prompt token and a generated one), got {self.max_seq_len}")
        for name in ("page_size", "max_num_seqs", "max_num_batched_tokens"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1, got {getattr(self, name)}")
        if self.max_chunk_size < 0:
            raise ValueError(f"max_chunk_size must be >= 0, got {self.max_chunk_size}")
        if self.max_chunk_size == 0:
            object.__setattr__(self, "enable_chunked_prefill", False)
        if not self.enable_chunked_prefill and self.max_num_batched_tokens < self.max_seq_len:
            raise ValueError(
                f"max_num_batched_tokens ({self.max_num_batched_tokens}) is smaller than max_seq_len "
                f"({self.max_seq_len}) with chunked prefill off: a whole prompt must fit one step. Raise "
                "max_num_batched_tokens, lower max_seq_len, or leave chunked prefill on."
            )
        if self.num_pages is not None and self.num_pages < 1:
            raise ValueError(f"num_pages must be >= 1, got {self.num_pages}")
        if not 0.0 < self.memory_fraction <= 1.0:
            raise ValueError(f"memory_fraction must be in (0, 1], got {self.memory_fraction}")

    @property
    def max_pages_per_seq(self) -> int:
        return -(-self.max_seq_len // self.page_size)
