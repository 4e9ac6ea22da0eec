"""Regenerates tests/golden/sampling.npz: what harleyszhang/rapid_llm's OWN sampler code makes
of a few rows of random logits, on the CPU in float32.

Run from the repository root with the reference tree importable:

    python tests/golden/make_sampling_golden.py /path/to/rapid_llm_checkout

Stored per row: the logits, the row's temperature, top-p, repetition penalty and generated
tokens; and from the reference (``rapid_llm/engine/sampler.py``): the penalised logits
(``apply_repetition_penalty``, :134-179), the greedy id (``greedy_ids``, :266-283), the tokens
its nucleus keeps (``sample_top_p`` with the whole vocabulary as the pool, :189-244; the draw
itself is random there, so ``torch.multinomial`` is replaced by a recorder for the call) and
the log-probability records of a given token with the five most likely
(``_distribution_records``, :345-369).  The rows have no equal logits, so no result depends on
how ties are ordered.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROWS, VOCAB, TOP = 24, 384, 5


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from rapid_llm.engine import sampler as ref

    generator = torch.Generator().manual_seed(77)
    logits = torch.randn((ROWS, VOCAB), generator=generator) * 2.0
    temperature = torch.tensor([0.7, 1.0, 1.3] * 8)
    top_p = torch.tensor([0.3, 0.5, 0.9, 0.95] * 6)
    penalty = torch.tensor([1.0, 1.1, 2.0, 1.0, 1.3, 1.0] * 4)
    lengths = [row % 5 * 6 for row in range(ROWS)]
    span = max(lengths)
    generated = torch.zeros((ROWS, span), dtype=torch.long)
    mask = torch.zeros((ROWS, span), dtype=torch.bool)
    for row, count in enumerate(lengths):
        generated[row, :count] = torch.randint(0, VOCAB, (count,), generator=generator)
        mask[row, :count] = True
    token = torch.randint(0, VOCAB, (ROWS, 1), generator=generator)

    penalised = ref.apply_repetition_penalty(logits, ref.GeneratedSpan(generated, mask), penalty[:, None])
    greedy = ref.greedy_ids(penalised, None).reshape(-1)
    scaled = penalised / temperature[:, None]
    probs = torch.softmax(scaled, dim=-1)

    handed = {}

    def recorder(weights, num_samples=1, **_):
        handed["weights"] = weights.clone()
        return weights.argmax(dim=-1, keepdim=True)

    real, torch.multinomial = torch.multinomial, recorder
    try:
        ref.sample_top_p(probs.clone(), top_p[:, None], k=None)
    finally:
        torch.multinomial = real
    # the pool is the whole row in descending order: map the kept candidates back to token ids
    order = torch.topk(probs, VOCAB, dim=-1).indices
    kept = torch.zeros((ROWS, VOCAB), dtype=torch.bool)
    kept.scatter_(1, order, handed["weights"] > 0)

    chosen, top_values, top_ids = ref._distribution_records(scaled, token, None, TOP)
    out = Path(__file__).resolve().parent / "sampling.npz"
    np.savez_compressed(
        out, logits=logits.numpy(), temperature=temperature.numpy(), top_p=top_p.numpy(), penalty=penalty.numpy(),
        generated=generated.numpy().astype(np.int32), generated_count=np.asarray(lengths, dtype=np.int32),
        token=token.reshape(-1).numpy().astype(np.int32), penalised=penalised.numpy(), greedy=greedy.numpy().astype(np.int32),
        kept=kept.numpy(), chosen_logprob=chosen.reshape(-1).numpy(), top_logprobs=top_values.numpy(),
        top_ids=top_ids.numpy().astype(np.int32),
    )
    print("wrote", out, "kept per row:", kept.sum(dim=1).tolist())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_sampling_golden.py /path/to/rapid_llm_checkout")
    main(sys.argv[1])
