"""A B200-native inference engine for the Qwen3 dense decoder.

``LLM(model_dir).generate(prompts, SamplingParams(...))`` is the Python entry point;
``bin/trace_run`` replays given token ids and writes logits; ``python -m rapid_llm_b200.cli``
is the command line.
"""

__version__ = "0.1.0"

from .config import EngineConfig, Qwen3Config, load_config
from .sampling.params import SamplingParams


def __getattr__(name):  # the engine imports lazily: configuration and weights work without a GPU
    if name in ("LLM", "RequestOutput", "CompletionOutput"):
        from .engine import llm, outputs

        return {"LLM": llm.LLM, "RequestOutput": outputs.RequestOutput, "CompletionOutput": outputs.CompletionOutput}[name]
    if name == "ModelRunner":
        from .engine.runner import ModelRunner

        return ModelRunner
    if name == "Scheduler":
        from .engine.scheduler import Scheduler

        return Scheduler
    raise AttributeError(name)


__all__ = ["EngineConfig", "LLM", "ModelRunner", "Qwen3Config", "SamplingParams", "Scheduler", "load_config"]
