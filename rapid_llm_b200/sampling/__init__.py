from .params import SamplingParams

__all__ = ["SamplingParams"]
