from .causal_lm import CausalLM

__all__ = ["CausalLM"]
