"""Regenerates tests/golden/*.npz: logits of harleyszhang/rapid_llm's OWN model code, run on
the CPU in float32, for the tiny random models A and B.

Run from the repository root with the reference tree importable:

    python tests/golden/make_golden.py /path/to/rapid_llm_checkout

It writes the two model folders (config.json + model.safetensors, from the repository's
seeded random-weights mode) into a temporary folder, loads each with the reference's
``ModelRunner.build(device="cpu")`` with its dtype property overridden to float32 (the
reference otherwise downgrades float32 checkpoints to bfloat16,
rapid_llm/models/config.py:134-146), feeds whole prompts through ``runner.model`` and stores
the logits of every position, together with the weights' seed, so the test can rebuild the
same folder.  Only transformers' *configuration* classes are touched by the reference on
this path (AutoConfig), none of its model code.
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

PROMPT_LENGTHS = {"A": [5, 17, 33], "B": [1, 7, 31, 64, 100]}


def prompts_for(name: str, vocab: int) -> list[list[int]]:
    generator = torch.Generator().manual_seed(1000 + ord(name))
    return [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in PROMPT_LENGTHS[name]]


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from rapid_llm.executor.model_runner import ModelRunner
    from rapid_llm.models import config as ref_config

    ref_config.ModelConfig.dtype = property(lambda self: torch.float32)

    from tiny_configs import CONFIGS, SEEDS

    from rapid_llm_b200.config import Qwen3Config
    from rapid_llm_b200.weights import write_random_model

    out_dir = Path(__file__).resolve().parent
    for name in ("A", "B"):
        raw = CONFIGS[name]
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_random_model(Path(tmp) / name, Qwen3Config.from_dict(raw), SEEDS[name], dtype=torch.float32)
            runner = ModelRunner.build(str(folder), raw["max_position_embeddings"], max_gpu_num_blocks=4096, device="cpu")
            rows = {}
            for index, prompt in enumerate(prompts_for(name, raw["vocab_size"])):
                runner.kv_mem_manager.free_all() if hasattr(runner, "kv_mem_manager") else None
                count = len(prompt)
                runner.prefill_alloc_kv_cache(count, torch.tensor([count], dtype=torch.int32), torch.tensor([0], dtype=torch.int32))
                ids = torch.tensor([prompt], dtype=torch.long)
                with torch.no_grad():
                    logits = runner.model(ids, torch.arange(count)[None], runner.atten_info)
                rows[f"prompt{index}"] = np.asarray(prompt, dtype=np.int32)
                rows[f"logits{index}"] = logits.reshape(count, -1).float().numpy()
            np.savez_compressed(out_dir / f"tiny_{name}.npz", seed=SEEDS[name], **rows)
            print(name, {k: v.shape for k, v in rows.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/rapid_llm_checkout")
    main(sys.argv[1])
