"""Sampling: parameters and the batched selector."""
from .params import SamplingParams, TokenLogprob, mix_seed, uniform_from

__all__ = ["SamplingParams", "TokenLogprob", "mix_seed", "uniform_from"]
