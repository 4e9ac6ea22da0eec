from .params import PositionLogprobs, SamplingParams

__all__ = ["PositionLogprobs", "SamplingParams"]
