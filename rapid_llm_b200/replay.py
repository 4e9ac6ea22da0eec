"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
:class:`rapid_llm_b200.engine.runner.ModelRunner`, the step function generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  A request is admitted when its id is first seen
and gives back what it holds when a step lists it under ``end``.  For a step in which
something is wanted, ``OUT/<step>.f32`` receives the logits at the wanted places, in the
order of the entries and of ``want``, as little-endian float32 ``[wanted, vocab]``.  Every
step also writes ``OUT/<step>.pages.json``: for each request of the step, the page ids it held
after the step, one list per cache group in position order (0 = a page given back because the
window has passed it), so that a reader can see pages used again.  After
every step ``done <step>`` is printed and flushed.  ``--max-tokens`` sizes the cache pool:
the most tokens live requests hold at any time, each request's count rounded up to a whole
number of pages.

The reference has nothing like it; its nearest tools record greedy texts or diff one
prefill per layer (``scripts/verify/golden_tokens.py``, ``rapid_llm/tools/accuracy/divergence.py``).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.splitlines()[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (sizes the cache pool)")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-live", type=int, default=8, help="requests live at a time")
    parser.add_argument("--device", default="cuda:0")
    return parser


class Replayer:
    """Feeds trace records to a runner; the loop behind ``trace_run``."""

    def __init__(self, runner, out_dir: Path | None = None) -> None:
        self.runner = runner
        self.out_dir = out_dir
        self._staging = None
        self.last_pages: dict[str, list[list[int]]] = {}

    def run_step(self, record: dict) -> np.ndarray | None:
        """Run one record; returns (and, with ``out_dir``, writes) the wanted logits."""
        from .engine.runner import StepEntry
        from .ops import kernels

        runner, step = self.runner, record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = item["id"]
            if not runner.cache.has(request_id):
                if not runner.admit(request_id):
                    raise RuntimeError(f"step {step}: no free slot for request {request_id!r}")
            entries.append(StepEntry(request_id, list(item["tokens"]), list(item.get("want", []))))
        host = None
        if entries:
            logits = runner.step(entries)
            rows = logits.shape[0]
            if rows:
                vocab = logits.shape[1]
                if self._staging is None or self._staging.shape[0] < rows:
                    self._staging = torch.empty((max(rows, 64), vocab), dtype=torch.float32, device=runner.device)
                as_float = kernels.to_float(logits.contiguous(), self._staging[:rows])
                host = np.ascontiguousarray(as_float.cpu().numpy().astype("<f4", copy=False))
                if self.out_dir is not None:
                    host.tofile(self.out_dir / f"{step}.f32")
            runner.check_fault()
        self.last_pages = {str(entry.request_id): [list(map(int, group)) for group in runner.cache.pages_of(entry.request_id)]
                           for entry in entries}
        if self.out_dir is not None:
            (self.out_dir / f"{step}.pages.json").write_text(json.dumps(self.last_pages))
        for request_id in record.get("end", []):
            if runner.cache.has(request_id):
                runner.release(request_id)
        return host


def engine_config_for(model_config, dtype: str, max_tokens: int, page_size: int = 16, max_live: int = 8):
    """Engine sizes for a replay whose live requests hold at most ``max_tokens`` tokens."""
    from .config import EngineConfig, parse_dtype

    max_tokens = max(int(max_tokens), page_size)
    num_pages = -(-max_tokens // page_size)
    capacity = num_pages * page_size
    return EngineConfig(
        dtype=parse_dtype(dtype),
        max_seq_len=min(model_config.to_spec().max_positions, capacity),
        page_size=page_size,
        num_pages=num_pages,
        max_num_seqs=max_live,
        max_num_batched_tokens=max(capacity, 64),
        max_chunk_size=max(capacity, 64),
        use_cuda_graph=False,
    )


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    from .config import load_config
    from .engine.runner import ModelRunner

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model_config = load_config(args.model)
    engine = engine_config_for(model_config, args.dtype, args.max_tokens, args.page_size, args.max_live)
    print(f"[trace_run] loading {args.model} as {args.dtype}; kernels are compiled on first use",
          file=sys.stderr, flush=True)
    runner = ModelRunner.from_folder(args.model, engine, device=args.device)
    replayer = Replayer(runner, out_dir)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        replayer.run_step(record)
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
