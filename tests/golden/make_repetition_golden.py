"""Regenerates tests/golden/repetition.json: what harleyszhang/rapid_llm's OWN repeat breaker
(``detect_repetition``, ``rapid_llm/engine/stop_criteria.py:63-79``) says of a set of texts.

Run from the repository root with the reference tree importable:

    python tests/golden/make_repetition_golden.py /path/to/rapid_llm_checkout

The texts are made here from a seed: prose of random words, the same with a block repeated a few
times at the end or in the middle, loops whose only change is a number that counts up, texts just
below and just at the shortest length the breaker looks at, and texts that are mostly digits.
Stored: each text with the reference's verdict.
"""

from __future__ import annotations

import json
import random
import sys
from pathlib import Path

WORDS = "the of a sea stone seven river glass quiet under between lantern copper field rain".split()


def prose(rng: random.Random, characters: int) -> str:
    out = ""
    while len(out) < characters:
        out += rng.choice(WORDS) + rng.choice([" ", " ", ", ", ". "])
    return out[:characters]


def texts(seed: int = 5) -> list[str]:
    rng = random.Random(seed)
    out: list[str] = []
    for _ in range(6):
        out.append(prose(rng, rng.randint(300, 1500)))
    for repeats in (2, 3, 4, 5, 8):
        for block_len in (40, 128, 131, 200):
            block = prose(rng, block_len)
            out.append(prose(rng, rng.randint(0, 400)) + block * repeats)
            out.append(prose(rng, 200) + block * repeats + prose(rng, rng.choice([3, 60, 128, 300])))
    for repeats in (3, 4, 6):
        line = prose(rng, 90)
        out.append("".join(f"{line} for {n + 7} years and {n * 13} days. " for n in range(repeats)))
        out.append(prose(rng, 100) + "".join(f"step {n}: {line}\n" for n in range(repeats + 1)))
    block = prose(rng, 128)
    for characters in (511, 512, 513, 640):
        out.append((block * 6)[:characters])
    out.append("7" * 2000)
    out.append("".join(str(rng.randint(0, 10**6)) + " " for _ in range(300)))
    out.append(prose(rng, 700) + "12345678901234567890" * 40)
    out.append("")
    return out


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from rapid_llm.engine.stop_criteria import detect_repetition

    cases = [{"text": text, "repeats": bool(detect_repetition(text))} for text in texts()]
    target = Path(__file__).with_name("repetition.json")
    target.write_text(json.dumps(cases, indent=0) + "\n")
    print(f"wrote {target}: {len(cases)} texts, {sum(c['repeats'] for c in cases)} of them loops")


if __name__ == "__main__":
    main(sys.argv[1])
