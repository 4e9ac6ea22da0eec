"""The reference arm of ``bench.py``: the unmodified harleyszhang/rapid_llm engine on the same workload.

It is run as a child process by ``bench.py --impl reference``.  Nothing of ``rapid_llm_b200``
is imported here: the model folder is written with torch and the ``safetensors`` package, and
the engine that is timed is the reference's own continuous-batching scheduler
(``rapid_llm.engine.Scheduler.from_pretrained`` / ``add_request`` / ``step``, the path its
``rapid-llm batch`` command and its ``benchmark/backends.py:EngineBackend`` drive), imported
from the offline install under ``baseline/_ref``.

Workload, as in ``bench.py``: Qwen3-8B layer sizes with random bfloat16 weights, ``--batch``
requests of 1,024 random token ids each, greedy, context limit 8192; ``--steps`` decode steps
are timed with CUDA events after ``--warmup`` untimed ones.  A 2,048-token prompt is timed as
the prefill.  The reference's stop ids are emptied so that a random greedy token cannot end a
request early (its own benchmarks switch stop handling off the same way,
``rapid_llm/benchmark/workloads.py:27-35``).

Prints one JSON object on the last line of standard output.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 151936, "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "attention_bias": False,
    "hidden_act": "silu", "use_sliding_window": False, "sliding_window": None,
}
# the other layer sizes of the benchmark (the same dictionary as in bench.py, written out again: this file
# imports nothing of the repository)
SHAPES = {
    "8b": {},
    "14b": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
            "intermediate_size": 17408},
    "32b": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "num_key_value_heads": 8,
            "intermediate_size": 25600},
}
CONTEXT, PROMPT_LEN, PREFILL_TOKENS = 8192, 1024, 2048


def say(message: str) -> None:
    print(f"[reference arm] {message}", file=sys.stderr, flush=True)


def write_model_folder(folder: Path, config: dict, seed: int) -> None:
    """config.json, one safetensors shard per layer (drawn on the GPU) and a word-level tokenizer."""
    import torch
    from safetensors.torch import save_file

    marker = folder / "complete.json"
    if marker.is_file() and json.loads(marker.read_text()) == {"config": config, "seed": seed}:
        return
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    device = torch.device("cuda:0")
    generator = torch.Generator(device=device).manual_seed(seed)
    h, i, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    d, hq, hkv = config["head_dim"], config["num_attention_heads"], config["num_key_value_heads"]

    def matrix(rows: int, cols: int):
        return (torch.randn((rows, cols), device=device, generator=generator) * 0.02).to(torch.bfloat16).cpu()

    def ones(n: int):
        return torch.ones(n, dtype=torch.bfloat16)

    save_file({"model.embed_tokens.weight": matrix(v, h)}, str(folder / "model-00000-embed.safetensors"))
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        save_file(
            {
                p + "input_layernorm.weight": ones(h),
                p + "post_attention_layernorm.weight": ones(h),
                p + "self_attn.q_proj.weight": matrix(hq * d, h),
                p + "self_attn.k_proj.weight": matrix(hkv * d, h),
                p + "self_attn.v_proj.weight": matrix(hkv * d, h),
                p + "self_attn.o_proj.weight": matrix(h, hq * d),
                p + "self_attn.q_norm.weight": ones(d),
                p + "self_attn.k_norm.weight": ones(d),
                p + "mlp.gate_proj.weight": matrix(i, h),
                p + "mlp.up_proj.weight": matrix(i, h),
                p + "mlp.down_proj.weight": matrix(h, i),
            },
            str(folder / f"model-{layer + 1:05d}-layer.safetensors"),
        )
    save_file({"model.norm.weight": ones(h), "lm_head.weight": matrix(v, h)}, str(folder / "model-99999-head.safetensors"))

    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from transformers import PreTrainedTokenizerFast

    tokenizer = Tokenizer(WordLevel({"<unk>": 0, "<s>": 1, "</s>": 2, "hello": 3, "world": 4}, unk_token="<unk>"))
    tokenizer.pre_tokenizer = Whitespace()
    PreTrainedTokenizerFast(
        tokenizer_object=tokenizer, unk_token="<unk>", bos_token="<s>", eos_token="</s>", pad_token="<unk>",
    ).save_pretrained(str(folder))
    marker.write_text(json.dumps({"config": config, "seed": seed}))


def random_prompts(count: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import torch

    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count, length), generator=generator).tolist()


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None)
    parser.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    parser.add_argument("--workload", choices=["decode", "serve"], default="decode")
    parser.add_argument("--requests", type=int, default=64)
    parser.add_argument("--workdir", default="/tmp/rapid_llm_b200_reference_arm")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b")
    parser.add_argument("--context", type=int, default=CONTEXT)
    args = parser.parse_args()
    globals()["PROMPT_LEN"] = args.prompt_len
    globals()["CONTEXT"] = args.context

    import torch

    config = dict(QWEN3_8B, **SHAPES[args.shape])
    layers_full = config["num_hidden_layers"]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    folder = Path(args.workdir) / f"qwen3_{args.shape}_random_L{config['num_hidden_layers']}"
    say(f"writing the random model folder {folder}")
    write_model_folder(folder, config, seed=0)

    sys.path.insert(0, str(HERE / "_ref"))
    from rapid_llm import SamplingParams
    from rapid_llm.engine import Scheduler

    say("building the reference engine")
    scheduler = Scheduler.from_pretrained(
        str(folder), max_seq_len=CONTEXT, max_num_seqs=max(args.batch, 8, min(args.requests, 64) if args.workload == "serve" else 0),
        max_num_batched_tokens=PREFILL_TOKENS if args.workload == "serve" else 8192,
        max_chunk_size=PREFILL_TOKENS, use_cuda_graph=True,
    )
    scheduler.stop_token_ids = set()
    vocab = config["vocab_size"]

    def greedy(max_gen_len: int):
        return SamplingParams(temperature=0.0, top_p=1.0, repetition_penalty=1.0, stop_on_repeat=False,
                              max_gen_len=max_gen_len)

    def drain() -> None:
        while scheduler.has_unfinished_requests():
            scheduler.step()

    if args.workload == "serve":
        # the continuous-batching workload of bench.py's serve_run, the same requests in the same order
        generator = torch.Generator().manual_seed(3)
        count = args.requests
        prompt_lengths = torch.randint(128, 4097, (count,), generator=generator).tolist()
        output_lengths = torch.randint(64, 513, (count,), generator=generator).tolist()
        prompts = [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in prompt_lengths]
        for prompt, n in zip(prompts, output_lengths):          # once untimed: loads, graphs, compilation
            scheduler.add_request("", greedy(n), prompt_token_ids=prompt)
        drain()
        torch.cuda.synchronize()
        started = time.perf_counter()
        requests = [scheduler.add_request("", greedy(n), prompt_token_ids=p) for p, n in zip(prompts, output_lengths)]
        drain()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        print(json.dumps({
            "seconds": seconds, "generated_tokens": sum(len(r.output_token_ids) for r in requests),
            "prompt_tokens": sum(prompt_lengths), "wanted_tokens": sum(output_lengths),
            "layers": config["num_hidden_layers"], "layers_full": layers_full,
        }))
        return 0

    # prefill of one 2,048-token prompt: submit, step until its first token; best of three
    prefill_ms, prefill_device_ms = [], []
    for trial in range(max(args.warmup, 1) + 3):
        request = scheduler.add_request("", greedy(1), prompt_token_ids=random_prompts(1, PREFILL_TOKENS, vocab, 11 + trial)[0])
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        started = time.perf_counter()
        begin.record()
        while not request.output_token_ids and request.finish_reason is None:
            scheduler.step()
        end.record()
        torch.cuda.synchronize()
        if trial >= max(args.warmup, 1):
            prefill_ms.append((time.perf_counter() - started) * 1000.0)
            prefill_device_ms.append(begin.elapsed_time(end))
        drain()
    say(f"prefill {min(prefill_ms):.2f} ms")

    # decode: the whole batch past its prompts, then warm-up, then exactly K timed steps
    budget = 2 * (args.steps + args.warmup) + 16 + args.batch * PROMPT_LEN // PREFILL_TOKENS
    requests = [
        scheduler.add_request("", greedy(budget), prompt_token_ids=prompt)
        for prompt in random_prompts(args.batch, PROMPT_LEN, vocab, args.batch)
    ]
    while any(not r.output_token_ids for r in requests):
        scheduler.step()
    for _ in range(args.warmup):
        scheduler.step()
    torch.cuda.synchronize()
    before = sum(len(r.output_token_ids) for r in requests)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(args.steps):
        scheduler.step()
    end.record()
    torch.cuda.synchronize()
    device_ms = begin.elapsed_time(end)
    tokens = sum(len(r.output_token_ids) for r in requests) - before

    started = time.perf_counter()
    before = sum(len(r.output_token_ids) for r in requests)
    for _ in range(args.steps):
        scheduler.step()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - started) * 1000.0
    wall_tokens = sum(len(r.output_token_ids) for r in requests) - before
    for request in requests:
        scheduler.abort(request.request_id)

    print(json.dumps({
        "device_ms": device_ms, "tokens": tokens, "wall_ms": wall_ms, "wall_tokens": wall_tokens,
        "prefill_ms": min(prefill_ms), "prefill_device_ms": min(prefill_device_ms), "layers": config["num_hidden_layers"], "layers_full": layers_full,
        "finished_early": sum(1 for r in requests if r.finish_reason not in (None, "abort")),
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
