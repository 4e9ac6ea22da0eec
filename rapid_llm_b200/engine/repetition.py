"""The repeat breaker: has a request's generated text fallen into a loop?

The reference ends a request with the finish reason ``"repeat"`` when the text it has generated
keeps returning to the same block: it takes the last 128 characters, with every run of digits
replaced by one placeholder (so that a loop that only counts upwards is still a loop), and asks
whether that block already stands at least three times in the text before it
(``rapid_llm/engine/stop_criteria.py:56-79``); the scheduler asks this every eighth step for
requests whose ``SamplingParams.stop_on_repeat`` is set
(``rapid_llm/engine/scheduler.py:1414,1452-1453``).

The test is on text, so it needs a tokenizer: the scheduler here applies it only when it was
given a function that turns token ids into text (``LLM`` passes its tokenizer's when the model
folder has one).  Requests of token ids alone are never ended by it.
"""

from __future__ import annotations

import re

WINDOW = 128          # characters of the trailing block
MIN_REPEATS = 3       # earlier occurrences of that block that make a loop
CHECK_EVERY = 8       # scheduler steps between two looks at a request's text

_DIGITS = re.compile(r"\d+")
_PLACEHOLDER = "<n>"


def text_repeats(text: str, window: int = WINDOW, min_repeats: int = MIN_REPEATS) -> bool:
    """True when the last ``window`` characters of ``text`` (digit runs made equal) occur at
    least ``min_repeats`` times, without overlap, in what precedes them.

    Text shorter than ``window * (min_repeats + 1)`` characters cannot hold that many and is
    never a loop.
    """
    if window < 1 or len(text) < window * (min_repeats + 1):
        return False
    flat = _DIGITS.sub(_PLACEHOLDER, text)
    if len(flat) <= window:            # long runs of digits shrank it: nothing stands before the block
        return False
    block = flat[len(flat) - window:]
    before = flat[: len(flat) - window]
    found, at = 0, before.find(block)
    while at >= 0:
        found += 1
        if found >= min_repeats:
            return True
        at = before.find(block, at + len(block))
    return False
