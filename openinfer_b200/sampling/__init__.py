"""Sampling: parameters and the batched selector."""
from .params import SamplingParams, mix_seed, uniform_from

__all__ = ["SamplingParams", "mix_seed", "uniform_from"]
