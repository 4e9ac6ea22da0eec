"""The Python entry point: ``LLM(model_dir).generate(prompts, SamplingParams(...))``.

Argument names and meanings follow the reference's facade (``rapid_llm/engine/llm.py:78-195``):
``max_seq_len`` (default 2048) bounds prompt plus generated tokens, ``max_gpu_num_blocks``
caps the cache, ``use_cuda_graph`` replays decode steps from captured graphs,
``hf_overrides`` replaces keys of ``config.json``.  Differences: prompts may be token-id
lists (a random-weight model has no tokenizer), generation always goes through the
continuous-batching scheduler, ``max_gpu_num_blocks`` counts cache pages of ``page_size``
tokens (the reference counts token rows), ``dtype`` selects the bfloat16 or the true
float32 path, and ``run_ahead`` (on by default) lets the scheduler enqueue a step before it has
read the previous step's tokens, as the reference's launch/harvest pipeline does
(``rapid_llm/engine/scheduler.py:817-933``).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Sequence

import torch

from ..config import EngineConfig, parse_dtype
from ..sampling.params import SamplingParams
from .executor import DeviceExecutor
from .outputs import CompletionOutput, RequestOutput
from .runner import ModelRunner
from .scheduler import Scheduler


def load_stop_token_ids(model_dir: str | Path) -> set[int]:
    """``eos_token_id`` of ``generation_config.json`` (an int or a list), if the folder has one
    (``rapid_llm/engine/stop_criteria.py:29-54``)."""
    path = Path(model_dir) / "generation_config.json"
    if not path.is_file():
        return set()
    try:
        value = json.loads(path.read_text()).get("eos_token_id")
    except (json.JSONDecodeError, AttributeError):
        return set()
    if value is None:
        return set()
    return {int(v) for v in (value if isinstance(value, list) else [value])}


class LLM:
    def __init__(
        self,
        model: str | Path | None = None,
        tokenizer: str | Path | None = None,
        max_seq_len: int = 2048,
        max_gpu_num_blocks: int | None = None,
        device: str = "cuda",
        use_cuda_graph: bool | None = None,
        quantization: str | None = None,
        tensor_parallel_size: int = 1,
        data_parallel_size: int = 1,
        enable_expert_parallel: bool = False,
        prefill_context_parallel_size: int = 1,
        prefill_context_parallel_strategy: str = "zigzag",
        decode_context_parallel_size: int = 1,
        dcp_comm_backend: str = "ag_rs",
        kv_cache_dtype: str = "auto",
        cuda_graph_lazy: bool = False,
        hf_overrides: Mapping[str, Any] | None = None,
        dtype: str | torch.dtype = "bfloat16",
        page_size: int = 16,
        max_num_seqs: int = 32,
        max_num_batched_tokens: int = 8192,
        max_chunk_size: int = 512,
        enable_chunked_prefill: bool = True,
        enable_preemption: bool = True,
        run_ahead: bool = True,
        stop_token_ids: Sequence[int] | None = None,
        runner: ModelRunner | None = None,
    ) -> None:
        # The reference's options for what this engine does not do are accepted at their neutral
        # values (``rapid_llm/engine/llm.py:78-96``) and refused otherwise, never ignored.
        neutral = {
            "quantization": (quantization, None), "tensor_parallel_size": (tensor_parallel_size, 1),
            "data_parallel_size": (data_parallel_size, 1), "enable_expert_parallel": (enable_expert_parallel, False),
            "prefill_context_parallel_size": (prefill_context_parallel_size, 1),
            "decode_context_parallel_size": (decode_context_parallel_size, 1), "kv_cache_dtype": (kv_cache_dtype, "auto"),
        }
        refused = [f"{name}={value!r}" for name, (value, wanted) in neutral.items() if value != wanted]
        if refused:
            raise ValueError("this engine runs unquantised weights and caches on one GPU; not supported: " + ", ".join(refused))
        del prefill_context_parallel_strategy, dcp_comm_backend, cuda_graph_lazy   # meaningful only with the above
        if device == "cuda":
            device = "cuda:0"
        self.engine_config = EngineConfig(
            dtype=parse_dtype(dtype),
            max_seq_len=max_seq_len,
            page_size=page_size,
            num_pages=max_gpu_num_blocks,
            max_num_seqs=max_num_seqs,
            max_num_batched_tokens=max_num_batched_tokens,
            max_chunk_size=max_chunk_size,
            enable_chunked_prefill=enable_chunked_prefill,
            enable_preemption=enable_preemption,
            run_ahead=run_ahead,
            use_cuda_graph=True if use_cuda_graph is None else bool(use_cuda_graph),
        )
        if runner is not None:
            self.runner = runner
            self.engine_config = runner.config
        elif model is not None:
            self.runner = ModelRunner.from_folder(model, self.engine_config, hf_overrides, device=device)
        else:
            raise ValueError("LLM needs a model folder (or a prepared runner)")
        self.model_dir = None if model is None else Path(model)
        stops = set(stop_token_ids or ())
        if self.model_dir is not None:
            stops |= load_stop_token_ids(self.model_dir)
        self.stop_token_ids = stops
        self.tokenizer = self._load_tokenizer(tokenizer or self.model_dir)
        self.executor = DeviceExecutor(self.runner)
        self.scheduler = Scheduler(
            self.executor, self.engine_config, self.stop_token_ids,
            detokenize=self._decode if self.tokenizer is not None else None,
        )

    @classmethod
    def from_runner(cls, runner: ModelRunner, stop_token_ids: Sequence[int] | None = None) -> "LLM":
        return cls(runner=runner, stop_token_ids=stop_token_ids)

    @staticmethod
    def _load_tokenizer(folder):
        if folder is None or not (Path(folder) / "tokenizer.json").is_file():
            return None
        from tokenizers import Tokenizer

        return Tokenizer.from_file(str(Path(folder) / "tokenizer.json"))

    # ------------------------------------------------------------------------------ #
    def _encode(self, prompt) -> tuple[str | None, list[int]]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer.json in the model folder; pass token ids instead")
            return prompt, self.tokenizer.encode(prompt, add_special_tokens=True).ids
        return None, [int(t) for t in prompt]

    def _decode(self, token_ids: list[int]) -> str:
        return "" if self.tokenizer is None else self.tokenizer.decode(token_ids)

    def _submit(self, prompts, sampling_params):
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None:
            sampling_params = SamplingParams()
        per_prompt = (
            [sampling_params] * len(prompts) if isinstance(sampling_params, SamplingParams) else list(sampling_params)
        )
        if len(per_prompt) != len(prompts):
            raise ValueError("one SamplingParams for all prompts, or one per prompt")
        encoded = [self._encode(p) for p in prompts]
        requests = []
        try:
            for (_, ids), params in zip(encoded, per_prompt):
                requests.append(self.scheduler.add_request(ids, params))
        except Exception:
            for request in requests:          # a refused prompt takes the call's earlier ones with it
                self.scheduler.abort(request)
            raise
        return encoded, requests

    def stream(self, prompts, sampling_params: SamplingParams | Sequence[SamplingParams] | None = None):
        """Yield, after every step that brought something, what each prompt gained since the last
        yield: one entry per prompt, a piece of text when the model folder has a tokenizer, else
        the list of new token ids (``rapid_llm/engine/llm.py:197-222`` yields text pieces the
        same way).  Tokens that are still only on the device (the scheduler runs a step ahead)
        are reported once the host has read them."""
        _, requests = self._submit(prompts, sampling_params)
        reported = [0] * len(requests)
        texts = [""] * len(requests)
        while True:
            gained, anything = [], False
            for index, request in enumerate(requests):
                tokens = request.output_token_ids
                known = next((i for i, token in enumerate(tokens) if token < 0), len(tokens))
                new = list(tokens[reported[index]:known])
                reported[index] = max(reported[index], known)
                anything = anything or bool(new)
                if self.tokenizer is None:
                    gained.append(new)
                else:
                    text = self._decode(list(tokens[:known]))
                    gained.append(text[len(texts[index]):])
                    texts[index] = text
            if anything:
                yield gained
            if not self.scheduler.has_unfinished():
                return
            self.scheduler.step()

    def generate(self, prompts, sampling_params: SamplingParams | Sequence[SamplingParams] | None = None) -> list[RequestOutput]:
        """Generate for every prompt; returns one ``RequestOutput`` per prompt, in order.

        ``prompts``: a string, a list of strings, one list of token ids, or a list of them.
        ``sampling_params``: one set for all prompts, or one per prompt.
        """
        encoded, requests = self._submit(prompts, sampling_params)
        self.scheduler.run_to_completion()
        outputs = []
        for (text, ids), request in zip(encoded, requests):
            completion = CompletionOutput(0, self._decode(request.output_token_ids), list(request.output_token_ids), request.finish_reason)
            metrics = {
                "arrival": request.arrival_time, "first_scheduled": request.first_scheduled_time,
                "first_token": request.first_token_time, "finished": request.finish_time,
                "preemptions": request.num_preemptions,
            }
            outputs.append(RequestOutput(text, ids, [completion], metrics))
        return outputs
