"""Step function, scheduler and the Python entry point.

``from rapid_llm_b200.engine import Scheduler, LLM`` works as it does in the reference
(``rapid_llm/engine/__init__.py``); the classes are imported on first use.
"""


def __getattr__(name):
    if name == "Scheduler":
        from .scheduler import Scheduler

        return Scheduler
    if name == "LLM":
        from .llm import LLM

        return LLM
    if name == "ModelRunner":
        from .runner import ModelRunner

        return ModelRunner
    raise AttributeError(name)
