"""Decode and prefill throughput of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  ``value`` is decoded tokens per second at
batch 8 with 1,024-token prompts (context limit 8192, pages of 16 tokens), timed on the
device with CUDA events around exactly K steps after W warm-up steps; each step includes
the upload of its metadata, the captured forward graph, the sampling kernel and the read
of the sampled ids; three such windows of K steps are timed and the median one is reported.
The weights streamed per step (15 GB) exceed L2 by two orders of
magnitude, so no flush is needed between iterations.  Before anything is timed, the logits of a
decode step replayed from a captured graph are compared with those of the same step run eagerly.  ``e2e`` is the same measured by the
wall clock through the Python entry point's scheduler (host token ids in and out).  The
line also carries a 2,048-token prefill, decode at batch 1 and 64, the decode step's HBM
roofline and the clocks sampled while timing.  For more than one GPU it says so and exits 2.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 151936, "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16",
}
# the other shapes of the baseline description: the same architecture, other sizes
SHAPES = {
    "8b": ("Qwen3-8B", {}),
    "14b": ("Qwen3-14B", {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40,
                          "num_key_value_heads": 8, "intermediate_size": 17408}),
    "32b": ("Qwen3-32B", {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64,
                          "num_key_value_heads": 8, "intermediate_size": 25600}),
}
CONTEXT, PROMPT_LEN, PREFILL_TOKENS, PAGE = 8192, 1024, 2048, 16
PUBLISHED_TOK_S = 216.6   # Qwen3-8B bf16, batch 8, 1x A10: docs/benchmark_models.md:191 of the reference (other hardware)
# The reference publishes no B200 number.  What `value` is divided by is the reference's own engine on this
# workload on one B200, measured by `bench.py --impl reference --steps 20 --warmup 5` on a fresh machine.
REFERENCE_SAME_GPU_TOK_S = 1500.4
BASELINE_NOTE = ("1500.4 tok/s: the unmodified reference engine, this workload, one B200 (bench.py --impl reference); "
                 "its only published figure is 216.6 tok/s on 1x A10 (docs/benchmark_models.md:191)")


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML in this process
    (a read every 10 ms), or by calling nvidia-smi where NVML's Python module is missing.  Reads only."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            top = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            bits = [pynvml.nvmlClocksEventReasonHwSlowdown, pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                    pynvml.nvmlClocksEventReasonSwThermalSlowdown, pynvml.nvmlClocksEventReasonSwPowerCap]
        except Exception:                      # no module, no library, an older binding: ask the tool instead
            return self._run_smi()
        while not self._stop.is_set():
            try:
                clock = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
            except Exception:
                return
            self.samples.append([str(clock), str(top)] + ["Active" if reasons & bit else "Not Active" for bit in bits])
            self._stop.wait(0.01)

    def _run_smi(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5,
                ).stdout.strip()
                if out:
                    self.samples.append([field.strip() for field in out.splitlines()[0].split(",")])
            except (OSError, subprocess.SubprocessError):
                return
            self._stop.wait(0.02)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        reasons = [name for i, name in enumerate(self.NAMES) if any(len(s) > 2 + i and s[2 + i] == "Active" for s in self.samples)]
        return {
            "sm_mhz": int(statistics.median(clocks)) if clocks else None,
            "sm_max_mhz": int(self.samples[0][1]) if self.samples and self.samples[0][1].isdigit() else None,
            "reasons": reasons, "samples": len(self.samples),
        }


def weight_bytes_per_step(cfg: dict, layers: int) -> int:
    """Every weight a decode step uses once: the layers' matrices and norms plus the head (the
    embedding is a gather of a few rows)."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d, hq, hkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_layer = ((hq + 2 * hkv) * d * h + h * hq * d + 3 * i * h) * 2 + (2 * h + 2 * d) * 4
    return layers * per_layer + v * h * 2 + h * 4


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, layers: int, tokens: int) -> float:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d, hq, hkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    linear = 2.0 * tokens * ((hq + 2 * hkv) * d * h + h * hq * d + 3 * i * h)
    attention = 4.0 * hq * d * tokens * (tokens + 1) / 2
    return layers * (linear + attention) + 2.0 * v * h     # the head runs on the last row only


def random_prompts(count: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import torch

    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count, length), generator=generator).tolist()


TEMPERATURE = 0.0      # > 0: every request samples with this temperature and top-p 0.9 (set by --temperature)


def sampling_params(max_gen_len: int, index: int):
    from rapid_llm_b200 import SamplingParams

    if TEMPERATURE > 0:
        return SamplingParams(temperature=TEMPERATURE, top_p=0.9, repetition_penalty=1.0, max_gen_len=max_gen_len, seed=index)
    return SamplingParams.greedy(max_gen_len=max_gen_len)


def decode_run(llm, batch: int, steps: int, warmup: int, seed: int) -> dict:
    """Prefill ``batch`` prompts, then time ``steps`` decode steps on the device and by wall clock."""
    import torch

    from rapid_llm_b200 import SamplingParams
    from rapid_llm_b200.ops import kernels

    scheduler, runner = llm.scheduler, llm.runner
    # every request must still be decoding when the last timed step runs: the prompts are
    # prefilled two per step while the earlier requests already decode
    prefill_steps = -(-batch * PROMPT_LEN // PREFILL_TOKENS)
    vocab = runner.model.spec.vocab_size
    requests = [scheduler.add_request(p, sampling_params(4 * steps + warmup + prefill_steps + 8, index))
                for index, p in enumerate(random_prompts(batch, PROMPT_LEN, vocab, seed))]
    while any(r.num_computed_tokens < len(r.prompt_token_ids) for r in requests):
        scheduler.step()                                   # prefill, untimed
    for _ in range(warmup):
        scheduler.step()
    torch.cuda.synchronize()

    windows = []
    for _ in range(3):                                      # three windows of exactly `steps` steps; the median counts
        context = requests[0].num_tokens
        launches_before = kernels.LAUNCHES.count
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            scheduler.step()
        end.record()
        torch.cuda.synchronize()
        windows.append((begin.elapsed_time(end), context + steps / 2.0, kernels.LAUNCHES.count - launches_before))
    device_ms, context_mean, launches = sorted(windows)[1]

    started = time.perf_counter()
    for _ in range(steps):
        scheduler.step()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - started) * 1000.0
    for request in requests:
        scheduler.abort(request)
    return {
        "device_ms": device_ms, "wall_ms": wall_ms, "launches": launches, "context_mean": context_mean,
        "tokens": batch * steps, "windows_ms": [round(w[0], 3) for w in windows],
    }


def prefill_run(llm, warmup: int, seed: int) -> dict:
    """One 2,048-token prompt as a single step, best of three after warm-up: milliseconds on the device (CUDA
    events around the step function) and by the wall clock through the scheduler, from the request's
    submission to its first sampled token on the host (what the reference arm's first-token time is)."""
    import torch

    from rapid_llm_b200 import SamplingParams
    from rapid_llm_b200.engine.runner import StepEntry

    runner, scheduler = llm.runner, llm.scheduler
    vocab = runner.model.spec.vocab_size
    device, wall = [], []
    for trial in range(max(warmup, 1) + 3):
        tokens = random_prompts(1, PREFILL_TOKENS, vocab, seed + trial)[0]
        runner.admit("prefill")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        runner.step([StepEntry("prefill", tokens, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        torch.cuda.synchronize()
        started = time.perf_counter()
        request = scheduler.add_request(tokens, SamplingParams.greedy(max_gen_len=1))
        while request.finish_reason is None:
            scheduler.step()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - started
        if trial >= max(warmup, 1):
            device.append(begin.elapsed_time(end))
            wall.append(seconds * 1000.0)
    return {"device_ms": min(device), "e2e_ms": min(wall)}


def graph_check(llm, seed: int) -> dict:
    """The benchmarked path against the eager one before anything is timed: two short prompts, one decode
    step each way (eager; replayed from a captured graph) on the same tokens at the same positions.  The
    kernels and their sums are the same, so the logits agree bit for bit; the ids must."""
    import torch

    from rapid_llm_b200.engine.runner import StepEntry

    runner = llm.runner
    vocab = runner.model.spec.vocab_size
    names = ["check0", "check1"][: min(2, runner.config.max_num_seqs)]
    prompts = random_prompts(len(names), 40, vocab, seed)

    def prefill():
        for name in names:
            runner.admit(name)
        logits = runner.step([StepEntry(name, prompt, [len(prompt) - 1]) for name, prompt in zip(names, prompts)])
        return torch.argmax(logits.float(), dim=-1).tolist()

    def done():
        for name in names:
            runner.release(name)

    first = prefill()
    runner.step_decode([StepEntry(name, [token], [0]) for name, token in zip(names, first)])     # captures the graph of this size
    done()
    first = prefill()
    eager = runner.step([StepEntry(name, [token], [0]) for name, token in zip(names, first)]).float().clone()
    done()
    assert prefill() == first
    replayed = runner.step_decode([StepEntry(name, [token], [0]) for name, token in zip(names, first)]).float().clone()
    done()
    runner.check_fault()
    same = torch.argmax(eager, dim=-1).tolist() == torch.argmax(replayed, dim=-1).tolist()
    diff = float((eager - replayed).abs().max())
    if not same or diff > 0.05 * float(eager.abs().max()):
        raise SystemExit(f"bench.py: the graph's decode step disagrees with the eager one (ids equal: {same}, largest difference {diff})")
    return {"graph_vs_eager_ids": "equal", "max_abs_diff": diff, "vocab": vocab}


def write_timeline(llm, batch: int, path: str, seed: int, step: str = "decode") -> dict:
    """Start, duration and overlap of every kernel of three decode steps, or of one step over a
    2,048-token prompt (CUPTI through torch.profiler)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from rapid_llm_b200 import SamplingParams
    from rapid_llm_b200.engine.runner import StepEntry

    scheduler, runner = llm.scheduler, llm.runner
    vocab = runner.model.spec.vocab_size
    if step == "prefill":
        for trial in range(3):
            tokens = random_prompts(1, PREFILL_TOKENS, vocab, seed + trial)[0]
            runner.admit("prefill")
            torch.cuda.synchronize()
            if trial < 2:
                runner.step([StepEntry("prefill", tokens, [PREFILL_TOKENS - 1])])
            else:
                with profile(activities=[ProfilerActivity.CUDA]) as prof:
                    runner.step([StepEntry("prefill", tokens, [PREFILL_TOKENS - 1])])
                    torch.cuda.synchronize()
            torch.cuda.synchronize()
            runner.release("prefill")
        return dump_timeline(prof, path, {"step": "prefill", "tokens": PREFILL_TOKENS})
    params = SamplingParams.greedy(max_gen_len=64 + -(-batch * PROMPT_LEN // PREFILL_TOKENS))
    requests = [scheduler.add_request(p, params) for p in random_prompts(batch, PROMPT_LEN, vocab, seed)]
    while any(r.num_computed_tokens < len(r.prompt_token_ids) for r in requests):
        scheduler.step()
    for _ in range(5):
        scheduler.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            scheduler.step()
        torch.cuda.synchronize()
    for request in requests:
        scheduler.abort(request)
    return dump_timeline(prof, path, {"step": "decode", "batch": batch})


def dump_timeline(prof, path: str, what: dict) -> dict:
    import torch

    events = sorted(
        (e.time_range.start, e.time_range.end - e.time_range.start, e.name)
        for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
    )
    origin, latest = events[0][0], events[0][0]
    lines = ["start_us  duration_us  gap_to_previous_end_us  kernel"]
    for begin, duration, name in events:
        lines.append(f"{begin - origin:9.1f} {duration:8.1f} {begin - latest:8.1f}  {name[:80]}")
        latest = max(latest, begin + duration)
    Path(path).write_text("\n".join(lines) + "\n")
    return {"timeline": path, "events": len(events), **what}


def serve_run(args, config, raw: dict, shape_name: str, layers: int, layers_full: int) -> dict:
    """Continuous batching as a user meets it: ``--requests`` prompts of uniform-random length
    (128 to 4,096 tokens) with 64 to 512 tokens to generate each, all handed to ``generate`` at
    once; prompts are cut into portions of 2,048 tokens a step beside the decoding requests.
    Run once untimed, then timed by the wall clock around the call, host token ids in and out."""
    import torch

    from rapid_llm_b200 import LLM, EngineConfig, SamplingParams
    from rapid_llm_b200.engine.runner import ModelRunner
    from rapid_llm_b200.ops import kernels

    generator = torch.Generator().manual_seed(3)
    count = args.requests
    prompt_lengths = torch.randint(128, 4097, (count,), generator=generator).tolist()
    output_lengths = torch.randint(64, 513, (count,), generator=generator).tolist()
    vocab = raw["vocab_size"]
    prompts = [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in prompt_lengths]
    live = min(count, 64)
    pages = sum(sorted((-(-(p + o) // PAGE) + 1 for p, o in zip(prompt_lengths, output_lengths)), reverse=True)[:live])
    engine = EngineConfig(
        dtype=torch.bfloat16, max_seq_len=CONTEXT, page_size=PAGE, num_pages=pages + PREFILL_TOKENS // PAGE,
        max_num_seqs=live, max_num_batched_tokens=PREFILL_TOKENS, max_chunk_size=PREFILL_TOKENS, use_cuda_graph=True,
    )
    llm = LLM.from_runner(ModelRunner.from_random(config, seed=0, config=engine))
    params = [SamplingParams.greedy(max_gen_len=n) for n in output_lengths]
    llm.scheduler.stop_token_ids = set()
    llm.generate(prompts, params)      # the whole workload once untimed: loads, graphs, workspaces
    torch.cuda.synchronize()
    before, steps_before = kernels.LAUNCHES.count, llm.runner.steps_run
    with ClockSampler() as clocks:
        begin = time.perf_counter()
        outputs = llm.generate(prompts, params)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
    generated = sum(len(o.token_ids) for o in outputs)
    assert generated == sum(output_lengths), (generated, sum(output_lengths))
    return {
        "metric": f"generated tok/s, continuous batching of {count} requests ({shape_name} shape)",
        "value": round(generated / seconds, 1), "unit": "tok/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "impl": "ours", "seconds": round(seconds, 3),
        "prompt_tokens": sum(prompt_lengths), "generated_tokens": generated,
        "all_tokens_per_second": round((sum(prompt_lengths) + generated) / seconds, 1),
        "steps": llm.runner.steps_run - steps_before, "preemptions": llm.scheduler.num_preemptions,
        "gpu_launches": kernels.LAUNCHES.count - before,
        "config": {
            "model": f"{shape_name} shape, random weights", "layers": layers, "layers_full": layers_full,
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": vocab,
            "requests": count, "prompt_lengths": "uniform 128-4096", "output_lengths": "uniform 64-512",
            "tokens_per_step": PREFILL_TOKENS, "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "single GPU",
        },
        "clocks": clocks.summary(),
    }


def run_ours(args) -> dict:
    import torch

    from rapid_llm_b200 import LLM, EngineConfig, Qwen3Config
    from rapid_llm_b200.engine.runner import ModelRunner

    if args.prompt_len + 4 * args.steps + args.warmup + 128 > CONTEXT:
        raise SystemExit(f"--prompt-len {args.prompt_len} leaves no room to decode within the context of {CONTEXT}")
    peaks = measured_peaks()
    shape_name, sizes = SHAPES[args.shape]
    raw = dict(QWEN3_8B, **sizes)
    layers_full = raw["num_hidden_layers"]
    layers = args.layers or layers_full
    raw["num_hidden_layers"] = layers
    config = Qwen3Config.from_dict(raw)
    if args.workload == "serve":
        return serve_run(args, config, raw, shape_name, layers, layers_full)
    batches = sorted({args.batch, *args.points}) if "points" in args.parts else [args.batch]
    longest = PROMPT_LEN + 4 * args.steps + args.warmup + max(batches) * PROMPT_LEN // PREFILL_TOKENS + 64
    pages = max(batches) * (-(-longest // PAGE)) + PREFILL_TOKENS // PAGE + 8
    engine = EngineConfig(
        dtype=torch.bfloat16, max_seq_len=CONTEXT, page_size=PAGE, num_pages=pages, max_num_seqs=max(batches),
        max_num_batched_tokens=max(PREFILL_TOKENS, 2048), max_chunk_size=2048, use_cuda_graph=True,
    )
    runner = ModelRunner.from_random(config, seed=0, config=engine)
    llm = LLM.from_runner(runner)

    if args.timeline:
        return write_timeline(llm, args.batch, args.timeline, seed=args.batch, step=args.timeline_step)
    check = {"graph_vs_eager_ids": "skipped"} if args.skip_check else graph_check(llm, seed=5)
    prefill = prefill_run(llm, args.warmup, seed=11) if "prefill" in args.parts else None
    results = {}
    for batch in batches:
        if batch == args.batch or "points" not in args.parts:
            continue
        results[batch] = decode_run(llm, batch, args.steps, args.warmup, seed=batch)
    with ClockSampler() as clocks:
        results[args.batch] = decode_run(llm, args.batch, args.steps, args.warmup, seed=args.batch)
    main = results[args.batch]

    def step_figures(batch: int, result: dict) -> tuple[float, float, float]:
        """tokens a second, milliseconds a step, and the bytes a step must read over its time, in GB/s"""
        ms = result["device_ms"] / args.steps
        need = weight_bytes_per_step(raw, layers) + batch * result["context_mean"] * kv_bytes_per_token(raw, layers)
        return result["tokens"] / (result["device_ms"] / 1000.0), ms, need / (ms / 1000.0) / 1e9

    value, ms_per_step, achieved = step_figures(args.batch, main)
    flops = prefill_flops(raw, layers, PREFILL_TOKENS)
    meta_bytes = 4 * (args.batch * (3 + 1) + 3 * args.batch + 1 + args.batch)
    return {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name} shape, {PROMPT_LEN}-token prompts)",
        "value": round(value, 1),
        "unit": "tok/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(value / REFERENCE_SAME_GPU_TOK_S, 2) if (args.shape, args.batch, args.prompt_len, layers) == ("8b", 8, 1024, layers_full) else None,
        "dtype": "bf16",
        "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": f"{shape_name} shape, random weights", "layers": layers, "layers_full": layers_full,
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights streamed per step)",
            "baseline_ref": BASELINE_NOTE, "peaks": peaks["source"], "timed": "median of 3 windows of `steps` steps",
            "sampling": f"temperature {TEMPERATURE}, top-p 0.9" if TEMPERATURE > 0 else "greedy",
        },
        "e2e": {
            "value": round(main["tokens"] / (main["wall_ms"] / 1000.0), 1), "unit": "tok/s",
            "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": 4 * (args.batch + 1),
            "ttft_ms": round(prefill["e2e_ms"], 3) if prefill else None, "tpot_ms": round(main["wall_ms"] / args.steps, 4),
        },
        "windows_ms": main["windows_ms"],
        "check": check,
        "gpu_launches": main["launches"],
        "prefill": None if prefill is None else {
            "value": round(PREFILL_TOKENS / (prefill["device_ms"] / 1000.0), 1), "tokens": PREFILL_TOKENS,
            "ms": round(prefill["device_ms"], 3),
            "frac": round(flops / (prefill["device_ms"] / 1000.0) / (peaks["bf16_tflops"] * 1e12), 4),
            "e2e_ms": round(prefill["e2e_ms"], 3),
        },
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4),
        },
        "points": {
            f"decode_b{batch}": round(step_figures(batch, result)[0], 1)
            for batch, result in sorted(results.items()) if batch != args.batch
        },
        "points_detail": {
            f"decode_b{batch}": {"ms": round(step_figures(batch, result)[1], 4),
                                 "frac": round(step_figures(batch, result)[2] / peaks["hbm_gbs"], 4)}
            for batch, result in sorted(results.items()) if batch != args.batch
        },
        "clocks": clocks.summary(),
    }


def run_reference(args) -> dict:
    """The unmodified reference engine on the same workload, in a child process of its own.

    The child (``baseline/reference_arm.py``) imports nothing of this package.  Any failure
    (no offline install, a kernel of the reference that does not build or run on this GPU,
    the time limit) yields the ``unavailable`` line instead of a number.
    """
    arm = ROOT / "baseline" / "reference_arm.py"
    if not (ROOT / "baseline" / "_ref" / "rapid_llm").is_dir():
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}
    command = [sys.executable, str(arm), "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--batch", str(args.batch), "--prompt-len", str(args.prompt_len),
               "--workload", args.workload, "--requests", str(args.requests), "--shape", args.shape,
               "--context", str(CONTEXT)]
    if args.layers:
        command += ["--layers", str(args.layers)]
    try:
        with ClockSampler() as clocks:
            done = subprocess.run(command, capture_output=True, text=True, timeout=args.reference_timeout)
    except subprocess.TimeoutExpired:
        return {"impl": "reference", "unavailable": f"the reference did not finish within {args.reference_timeout} s"}
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    if done.returncode != 0 or not lines:
        tail = " | ".join((done.stderr or done.stdout).strip().splitlines()[-3:])[:400]
        return {"impl": "reference", "unavailable": f"the reference engine failed here (exit {done.returncode}): {tail}"}
    got = json.loads(lines[-1])
    shape_name, sizes = SHAPES[args.shape]
    if args.workload == "serve":
        return {
            "metric": f"generated tok/s, continuous batching of {args.requests} requests ({shape_name} shape)",
            "value": round(got["generated_tokens"] / got["seconds"], 1), "unit": "tok/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "seconds": round(got["seconds"], 3), "prompt_tokens": got["prompt_tokens"],
            "generated_tokens": got["generated_tokens"], "wanted_tokens": got["wanted_tokens"],
            "all_tokens_per_second": round((got["prompt_tokens"] + got["generated_tokens"]) / got["seconds"], 1),
            "config": {"model": f"{shape_name} shape, random weights", "layers": got["layers"], "layers_full": got["layers_full"],
                       "requests": args.requests, "engine": "rapid_llm.engine.Scheduler (stock path, CUDA graphs on)"},
            "clocks": clocks.summary(),
        }
    peaks = measured_peaks()
    raw = dict(QWEN3_8B, **sizes)
    layers = got["layers"]
    ms_per_step = got["device_ms"] / args.steps
    value = got["tokens"] / (got["device_ms"] / 1000.0)
    context_mean = PROMPT_LEN + args.warmup + args.steps / 2.0
    step_bytes = weight_bytes_per_step(raw, layers) + args.batch * context_mean * kv_bytes_per_token(raw, layers)
    achieved = step_bytes / (ms_per_step / 1000.0) / 1e9
    flops = prefill_flops(raw, layers, PREFILL_TOKENS)
    return {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name} shape, {PROMPT_LEN}-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / REFERENCE_SAME_GPU_TOK_S, 2) if args.shape == "8b" else None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": {
            "model": f"{shape_name} shape, random weights", "layers": layers, "layers_full": got["layers_full"],
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights streamed per step)",
            "engine": "rapid_llm.engine.Scheduler (stock path, CUDA graphs on)", "peaks": peaks["source"],
            "finished_early": got["finished_early"],
        },
        "e2e": {"value": round(got["wall_tokens"] / (got["wall_ms"] / 1000.0), 1), "unit": "tok/s",
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "prefill": {      # on the device (CUDA events from submission to the first token), and the same by the wall clock
            "value": round(PREFILL_TOKENS / (got["prefill_device_ms"] / 1000.0), 1), "tokens": PREFILL_TOKENS,
            "ms": round(got["prefill_device_ms"], 3),
            "frac": round(flops / (got["prefill_device_ms"] / 1000.0) / (peaks["bf16_tflops"] * 1e12), 4),
            "e2e_ms": round(got["prefill_ms"], 3),
        },
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "clocks": clocks.summary(),
    }


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="tokens of each request's prompt: the "
                        "context that decoding starts from (the default is the configuration's)")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes: the 8B shape is the "
                        "benchmark's; 14b and 32b are the other shapes of the same architecture")
    parser.add_argument("--context", type=int, default=CONTEXT, help="longest sequence the engine is set up for")
    parser.add_argument("--points", default="1,64", help="other batch sizes decoded beside --batch")
    parser.add_argument("--workload", choices=["decode", "serve"], default="decode", help="decode: the benchmark "
                        "(timed decode steps, a prefill, the points); serve: continuous batching of --requests "
                        "prompts of mixed lengths through generate()")
    parser.add_argument("--requests", type=int, default=64, help="requests of the serve workload")
    parser.add_argument("--temperature", type=float, default=0.0, help="sample with this temperature and top-p 0.9 "
                        "instead of greedily (the benchmark's workload is greedy)")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the full model (both numbers are reported)")
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--parts", default="prefill,points", help="extra measurements beside the main decode run "
                        "(comma-separated: prefill, points); an empty string leaves only the main run, for profiling")
    parser.add_argument("--skip-check", action="store_true", help="do not compare a replayed decode step with an eager "
                        "one before timing (for profiler captures that count launches from the program's start)")
    parser.add_argument("--timeline", default=None, help="instead of measuring, write the kernel timeline of three "
                        "decode steps at --batch (start, duration, gap; CUPTI through torch.profiler) to this file")
    parser.add_argument("--timeline-step", choices=["decode", "prefill"], default="decode",
                        help="what --timeline records: three decode steps or one step over a 2,048-token prompt")
    parser.add_argument("--reference-timeout", type=int, default=1500, help="seconds the reference arm may take")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (work on several GPUs is out of scope)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    args.parts = {part for part in args.parts.split(",") if part}
    args.points = [int(x) for x in args.points.split(",") if x]
    globals()["TEMPERATURE"] = args.temperature
    globals()["PROMPT_LEN"] = args.prompt_len
    globals()["CONTEXT"] = args.context
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
