"""The command line without a GPU: its options carry the reference's names
(``rapid_llm/cli.py:57-165,614-701``), ``random-init`` writes a loadable model folder, and an
option that asks for what is not built ends with a message."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
from tiny_configs import TINY_B

ROOT = Path(__file__).resolve().parents[1]


def run_cli(*args, check=True):
    done = subprocess.run([sys.executable, "-m", "rapid_llm_b200.cli", *args], cwd=ROOT, capture_output=True, text=True)
    if check:
        assert done.returncode == 0, done.stderr
    return done


def test_batch_takes_the_references_options():
    text = run_cli("batch", "--help").stdout
    for flag in ("--model-dir", "--max-seq-len", "--max-gpu-num-blocks", "--device", "--temperature", "--top-p",
                 "--max-gen-len", "--repetition-penalty", "--quantization", "--kv-cache-dtype", "--tensor-parallel-size",
                 "--prompts-file", "--max-num-seqs", "--show-stats", "--cuda-graph", "--no-cuda-graph", "--stop-token-ids"):
        assert flag in text, flag


def test_random_init_writes_a_model_folder(tmp_path):
    from rapid_llm_b200.config import load_config
    from rapid_llm_b200.weights import SafetensorsFile

    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    run_cli("random-init", "--config", str(config), "--out", str(out), "--seed", "3", "--dtype", "bfloat16")
    assert load_config(out).num_hidden_layers == TINY_B["num_hidden_layers"]
    with SafetensorsFile(out / "model.safetensors") as handle:
        names = set(handle.keys())
    assert "model.embed_tokens.weight" in names and "lm_head.weight" in names
    again = tmp_path / "again"
    run_cli("random-init", "--config", str(config), "--out", str(again), "--seed", "3", "--dtype", "bfloat16")
    assert (out / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()      # seeded


def test_an_option_for_what_is_not_built_ends_with_a_message(tmp_path):
    done = run_cli("batch", "--model-dir", str(tmp_path), "--tensor-parallel-size", "2", check=False)
    assert done.returncode != 0 and "tensor_parallel_size=2" in done.stderr and "Traceback" not in done.stderr
    words = run_cli("batch", "--model-dir", str(tmp_path), "--stop-token-ids", "7,eos", check=False)
    assert words.returncode != 0 and "--stop-token-ids" in words.stderr and "Traceback" not in words.stderr
    missing = run_cli("batch", check=False)
    assert missing.returncode != 0 and "model-dir" in missing.stderr


def test_bench_refuses_more_than_one_gpu_with_one_line():
    done = subprocess.run([sys.executable, "bench.py", "--gpus", "2"], cwd=ROOT, capture_output=True, text=True)
    assert done.returncode == 2 and len(done.stdout.strip().splitlines()) == 1 and "single-GPU" in done.stdout


def test_the_bench_command_is_the_checkouts_bench_program():
    done = run_cli("bench", "--gpus", "2", check=False)
    assert done.returncode == 2 and "single-GPU" in done.stdout


def test_replay_sizes_the_pool_from_max_tokens():
    """``--max-tokens`` is what live requests hold at most: whole pages, the context bounded by the
    model's positions and by the pool, steps as large as the pool so that a whole prompt is one step."""
    import torch
    from tiny_configs import TINY_A, TINY_B

    from rapid_llm_b200.config import Qwen3Config
    from rapid_llm_b200.replay import build_parser, engine_config_for

    engine = engine_config_for(Qwen3Config.from_dict(TINY_B), "float32", 130, page_size=8, max_live=4)
    assert engine.num_pages == 17 and engine.page_size == 8 and engine.max_num_seqs == 4
    assert engine.max_seq_len == 136 and engine.max_num_batched_tokens == 136 and engine.dtype == torch.float32
    assert not engine.use_cuda_graph
    small = engine_config_for(Qwen3Config.from_dict(TINY_A), "bfloat16", 1024)
    assert small.max_seq_len == 128 and small.num_pages == 64 and small.dtype == torch.bfloat16     # 128 positions in the model
    tiny = engine_config_for(Qwen3Config.from_dict(TINY_A), "float32", 3)
    assert tiny.num_pages == 1 and tiny.max_seq_len == 16 and tiny.max_num_batched_tokens == 64
    args = build_parser().parse_args(["--model", "m", "--dtype", "float32", "--out", "o", "--max-tokens", "256"])
    assert (args.page_size, args.max_live, args.device) == (16, 8, "cuda:0")
    with pytest.raises(SystemExit):
        build_parser().parse_args(["--model", "m", "--dtype", "float16", "--out", "o", "--max-tokens", "1"])
