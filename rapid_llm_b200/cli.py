"""Command line in the manner of the reference's ``rapid-llm`` (``rapid_llm/cli.py:57-165,614-701``).

``batch`` runs prompts through the continuous-batching engine and keeps the reference's
option names and defaults: ``--model-dir`` (or ``$RAPID_LLM_MODEL_DIR``), ``--max-seq-len 2048``,
``--max-gpu-num-blocks``, ``--device cuda``, ``--temperature 0.6``, ``--top-p 0.9``,
``--max-gen-len``, ``--repetition-penalty 1.1``, ``--max-num-seqs 32``,
``--cuda-graph/--no-cuda-graph`` (on for ``batch``), ``--prompts-file``, ``--show-stats``.
Added here: ``--prompt-ids-file`` (one prompt per line as token ids, for models without a
tokenizer), ``--seed``, ``--dtype``, ``--page-size``, ``--max-num-batched-tokens``,
``--max-chunk-size``, ``--stop-token-ids`` (ids that end a request, added to those of the folder's
``generation_config.json`` as the reference unions its sources, ``rapid_llm/engine/stop_criteria.py:29-54``;
a folder of random weights has no such file).  ``random-init`` writes a seeded random model folder and ``replay``
is ``bin/trace_run``.  The reference's ``chat``, ``vl-chat``, ``serve`` and
``acc.divergence`` commands (a REPL, vision, a server, a transformers diff) are not built.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

DEMO_PROMPTS = [
    "What is the capital of France?",
    "Write a haiku about the sea.",
    "List three prime numbers.",
    "Explain what a GPU is in one sentence.",
]


def _add_engine_options(sub: argparse.ArgumentParser) -> None:
    sub.add_argument("--model-dir", help="Checkpoint directory (or $RAPID_LLM_MODEL_DIR)")
    sub.add_argument("--max-seq-len", type=int, default=2048)
    sub.add_argument("--max-gpu-num-blocks", type=int, default=None, help="cache pages; default sizes from free memory")
    sub.add_argument("--device", default="cuda")
    sub.add_argument("--temperature", type=float, default=0.6)
    sub.add_argument("--top-p", type=float, default=0.9)
    sub.add_argument("--max-gen-len", type=int, default=None)
    sub.add_argument("--repetition-penalty", type=float, default=1.1,
                     help="Penalise logits of already-generated tokens (1.0 disables it)")
    # the reference's options for what this engine does not do: taken at their neutral values only
    sub.add_argument("--quantization", default=None, help="not supported (weights stay bfloat16 or float32)")
    sub.add_argument("--kv-cache-dtype", default="auto", help='only "auto": the cache has the model\'s dtype')
    sub.add_argument("--tensor-parallel-size", type=int, default=1, help="only 1: one GPU")
    sub.add_argument("--enable-expert-parallel", action="store_true", help="not supported")
    sub.add_argument("--prefill-context-parallel-size", type=int, default=1, help="only 1")
    sub.add_argument("--prefill-context-parallel-strategy", default="zigzag", help="without meaning on one GPU")
    sub.add_argument("--decode-context-parallel-size", type=int, default=1, help="only 1")
    sub.add_argument("--dcp-comm-backend", default="ag_rs", help="without meaning on one GPU")
    sub.add_argument("--seed", type=int, default=None, help="seed of the sampling draws")
    sub.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    sub.add_argument("--page-size", type=int, default=16)
    sub.add_argument("--max-num-batched-tokens", type=int, default=8192)
    sub.add_argument("--max-chunk-size", type=int, default=512)
    sub.add_argument("--stop-token-ids", default="", help="token ids that end a request, separated by commas or "
                     "spaces; added to the eos ids of the folder's generation_config.json")


def _model_dir(args) -> str:
    folder = args.model_dir or os.environ.get("RAPID_LLM_MODEL_DIR")
    if not folder:
        raise SystemExit("pass --model-dir or set RAPID_LLM_MODEL_DIR")
    return folder


def _sampling(args):
    from .sampling.params import SamplingParams

    return SamplingParams(
        temperature=args.temperature, top_p=args.top_p, max_gen_len=args.max_gen_len,
        repetition_penalty=args.repetition_penalty, seed=args.seed,
    )


def run_batch(args) -> int:
    if args.prompt_ids_file:
        lines = [line.strip() for line in Path(args.prompt_ids_file).read_text().splitlines()]
        prompts = [[int(t) for t in line.replace(",", " ").split()] for line in lines if line]
    elif args.prompts_file:
        prompts = [line.strip() for line in Path(args.prompts_file).read_text().splitlines() if line.strip()]
    else:
        prompts = list(DEMO_PROMPTS)
    if not prompts:
        raise SystemExit("the prompt file contains no prompts")
    try:
        llm = _build_llm(args)
    except (ValueError, FileNotFoundError) as error:       # a refused option, a folder without a model
        raise SystemExit(f"rapid-llm-b200: {error}") from None
    started = time.perf_counter()
    try:
        outputs = llm.generate(prompts, _sampling(args))
    except ValueError as error:                            # a refused prompt or sampling option
        raise SystemExit(f"rapid-llm-b200: {error}") from None
    elapsed = time.perf_counter() - started
    return _report(args, outputs, started, elapsed)


def _stop_token_ids(text: str) -> list[int]:
    try:
        return [int(token) for token in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"rapid-llm-b200: --stop-token-ids takes integers, got {text!r}") from None


def _build_llm(args):
    from .engine.llm import LLM

    return LLM(
        _model_dir(args), max_seq_len=args.max_seq_len, max_gpu_num_blocks=args.max_gpu_num_blocks,
        device=args.device, use_cuda_graph=args.cuda_graph, dtype=args.dtype, page_size=args.page_size,
        max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
        max_chunk_size=args.max_chunk_size, run_ahead=args.run_ahead,
        quantization=args.quantization, kv_cache_dtype=args.kv_cache_dtype,
        tensor_parallel_size=args.tensor_parallel_size, enable_expert_parallel=args.enable_expert_parallel,
        prefill_context_parallel_size=args.prefill_context_parallel_size,
        decode_context_parallel_size=args.decode_context_parallel_size,
        stop_token_ids=_stop_token_ids(args.stop_token_ids),
    )


def _report(args, outputs, started: float, elapsed: float) -> int:
    for index, output in enumerate(outputs):
        completion = output.outputs[0]
        print(f"--- [{index}] {completion.finish_reason} ---")
        print(completion.text.strip() if completion.text else " ".join(map(str, completion.token_ids)))
        print()
    if args.show_stats:
        generated = sum(len(o.outputs[0].token_ids) for o in outputs)
        ttfts = [(o.metrics["first_token"] - started) * 1000 for o in outputs if o.metrics.get("first_token")]
        print(f"{len(outputs)} requests, {generated} tokens in {elapsed:.2f}s")
        print(f"throughput {generated / elapsed:7.1f} tok/s")
        if ttfts:
            print(f"TTFT mean {sum(ttfts) / len(ttfts):7.1f} ms | max {max(ttfts):7.1f} ms")
    return 0


def run_random_init(args) -> int:
    import torch

    from .config import resolve_architecture
    from .weights import write_random_model

    raw = json.loads(Path(args.config).read_text())
    config = resolve_architecture(raw).from_dict(raw)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    folder = write_random_model(args.out, config, args.seed, dtype=dtype, std=args.std, norm_std=args.norm_std)
    print(f"wrote {folder}/config.json and {folder}/model.safetensors (seed {args.seed}, {args.dtype})")
    return 0


def run_bench(argv: list[str]) -> int:
    """``bench.py`` of the source checkout, as a child process with the same interpreter."""
    script = Path(__file__).resolve().parent.parent / "bench.py"
    if not script.is_file():
        raise SystemExit(f"rapid-llm-b200: {script} is missing; the benchmark ships with the source checkout")
    return subprocess.call([sys.executable, str(script), *argv])


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="rapid-llm-b200", description=__doc__.splitlines()[0])
    subs = parser.add_subparsers(dest="command", required=True)

    batch = subs.add_parser("batch", help="Run a prompt file through the continuous-batching engine")
    _add_engine_options(batch)
    batch.add_argument("--prompts-file", help="Text file with one prompt per line; omit to use a built-in demo set")
    batch.add_argument("--prompt-ids-file", help="Text file with one prompt per line as token ids")
    batch.add_argument("--max-num-seqs", type=int, default=32)
    batch.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=True,
                       help="Capture decode CUDA graphs (default: %(default)s)")
    batch.add_argument("--run-ahead", action=argparse.BooleanOptionalAction, default=True,
                       help="Enqueue a step before the previous step's tokens are read (default: %(default)s)")
    batch.add_argument("--show-stats", action="store_true", help="Print throughput and per-request timings")
    batch.set_defaults(handler=run_batch)

    init = subs.add_parser("random-init", help="Write a model folder with seeded random weights")
    init.add_argument("--config", required=True, help="a config.json of the architecture")
    init.add_argument("--out", required=True)
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    init.add_argument("--std", type=float, default=0.02)
    init.add_argument("--norm-std", type=float, default=0.1)
    init.set_defaults(handler=run_random_init)

    replay = subs.add_parser("replay", help="Feed token ids step by step and write logits (bin/trace_run)", add_help=False)
    replay.set_defaults(handler=None)
    bench = subs.add_parser("bench", help="Decode and prefill throughput of the 8B shape (bench.py)", add_help=False)
    bench.set_defaults(handler=None)
    return parser


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from .replay import main as replay_main

        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        return run_bench(argv[1:])
    args = build_parser().parse_args(argv)
    return args.handler(args)


if __name__ == "__main__":
    sys.exit(main())
