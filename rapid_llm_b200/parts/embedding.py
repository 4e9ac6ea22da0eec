"""Token embedding and output head.

``x_t = E[id_t]`` without scaling (``rapid_llm/modules/vocab_parallel.py:101-103``); the
head is ``logits = h @ W^T`` without bias over the wanted rows only
(``rapid_llm/models/base.py:625-631``).  With tied embeddings the head has no tensor of its
own and uses the embedding's; a shipped ``lm_head.weight`` wins over the tie
(``rapid_llm/models/weights.py:165-172,197-214``).
"""

from __future__ import annotations

import torch

from ..ops import gemm, kernels
from .base import EMBEDDINGS, HEADS, MATRIX, Part, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, *, vocab_size: int, hidden_size: int, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.weight = self.new_storage((self.vocab, self.hidden), MATRIX)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden))}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight":
            raise KeyError(name)
        self.weight.copy_(tensor)

    def parameter_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, batch) -> torch.Tensor:
        out = batch.workspace.get("embedded", batch.num_tokens, self.hidden, self.dtype)
        return kernels.embedding(out, self.weight, batch.token_ids, batch.fault, batch.feedback)


@HEADS.register("lm_head")
class LMHead(Part):
    def __init__(self, *, vocab_size: int, hidden_size: int, tied: bool, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: torch.Tensor | None = None
        self._embedding: TokenEmbedding | None = None

    def tie_to(self, embedding: TokenEmbedding) -> None:
        self._embedding = embedding

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden), optional=self.tied)}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight":
            raise KeyError(name)
        if self.weight is None:
            self.weight = self.new_storage((self.vocab, self.hidden), MATRIX)
        self.weight.copy_(tensor)

    def finalize(self, loaded: set[str]) -> None:
        if "weight" not in loaded:
            if not self.tied or self._embedding is None:
                raise ValueError("the output head has no weight and is not tied to the embedding")
            self.weight = self._embedding.weight  # one tensor, not a copy

    def parameter_bytes(self) -> int:
        if self.weight is None or (self._embedding is not None and self.weight is self._embedding.weight):
            return 0
        return self.weight.numel() * self.weight.element_size()

    def forward(self, hidden_rows: torch.Tensor, batch) -> torch.Tensor:
        out = batch.workspace.get("logits", hidden_rows.shape[0], self.vocab, hidden_rows.dtype, min_rows=64)
        return gemm.linear(hidden_rows, self.weight, out, batch.fault)
