"""Regenerates tests/golden/greedy.npz: token ids that harleyszhang/rapid_llm's OWN continuous-
batching engine generates greedily for the tiny random models A and B, on the CPU in float32.

Run from the repository root with the reference tree importable:

    python tests/golden/make_greedy_golden.py /path/to/rapid_llm_checkout

Each model folder (the repository's seeded random-weights mode, plus a five-word tokenizer,
which the reference's engine insists on as its own CPU test does, tests/cpu/test_inference.py:42-52)
is loaded with ``rapid_llm.engine.Scheduler.from_pretrained(device="cpu")`` with the dtype
property overridden to float32 (rapid_llm/models/config.py:134-146 would downgrade to
bfloat16).  All prompts of a model are queued at once with portions of 13 tokens, so prompt
portions run beside decode steps, and ``step()`` is called until nothing is unfinished; stop
tokens are switched off so that every request produces its full count.
"""

from __future__ import annotations

import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

WORKLOADS = {"A": ([5, 17, 33], 8), "B": ([1, 7, 31, 64, 100], 12)}      # prompt lengths, tokens generated


def prompts_for(name: str, vocab: int) -> list[list[int]]:
    generator = torch.Generator().manual_seed(2000 + ord(name))
    return [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in WORKLOADS[name][0]]


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from rapid_llm.engine.sampler import SamplingParams
    from rapid_llm.engine.scheduler import Scheduler
    from rapid_llm.models import config as ref_config
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from transformers import PreTrainedTokenizerFast

    ref_config.ModelConfig.dtype = property(lambda self: torch.float32)

    from tiny_configs import CONFIGS, SEEDS

    from rapid_llm_b200.config import Qwen3Config
    from rapid_llm_b200.weights import write_random_model

    stored = {}
    for name, (_, count) in WORKLOADS.items():
        raw = CONFIGS[name]
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_random_model(Path(tmp) / name, Qwen3Config.from_dict(raw), SEEDS[name], dtype=torch.float32)
            words = Tokenizer(WordLevel({"<unk>": 0, "<s>": 1, "</s>": 2, "hello": 3, "world": 4}, unk_token="<unk>"))
            words.pre_tokenizer = Whitespace()
            PreTrainedTokenizerFast(tokenizer_object=words, unk_token="<unk>", bos_token="<s>", eos_token="</s>",
                                    pad_token="<unk>").save_pretrained(folder)
            engine = Scheduler.from_pretrained(
                str(folder), max_seq_len=raw["max_position_embeddings"], max_num_seqs=8, max_chunk_size=13,
                max_gpu_num_blocks=4096, device="cpu", use_cuda_graph=False,
            )
            engine.stop_token_ids = set()
            params = SamplingParams(temperature=0.0, top_p=1.0, repetition_penalty=1.0, max_gen_len=count, stop_on_repeat=False)
            prompts = prompts_for(name, raw["vocab_size"])
            requests = [engine.add_request("", params, prompt_token_ids=prompt) for prompt in prompts]
            steps = 0
            while engine.has_unfinished_requests():
                engine.step()
                steps += 1
                assert steps < 1000
            for index, (prompt, request) in enumerate(zip(prompts, requests)):
                assert len(request.output_token_ids) == count, request.finish_reason
                stored[f"{name}_prompt{index}"] = np.asarray(prompt, dtype=np.int32)
                stored[f"{name}_tokens{index}"] = np.asarray(request.output_token_ids, dtype=np.int32)
            print(name, steps, "steps", [request.output_token_ids for request in requests])
    np.savez_compressed(Path(__file__).resolve().parent / "greedy.npz", **stored)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_greedy_golden.py /path/to/rapid_llm_checkout")
    main(sys.argv[1])
