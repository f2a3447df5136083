"""Sampling parameters, with the reference's names, meanings and defaults
(pegainfer-frontend/src/sampler.rs:2-38)."""
from __future__ import annotations

import dataclasses
import math
from typing import List, Optional, Tuple

GREEDY_TEMPERATURE = 1e-5  # below this the temperature -> 0 limit (argmax) is taken


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1          # <= 0 or >= vocab: off; 1: greedy
    top_p: float = 1.0       # nucleus mass in (0, 1]
    min_p: float = 0.0       # mask p < min_p * p_max; 0: off
    seed: Optional[int] = None   # per request: its draws depend only on (seed, its own step, its distribution)
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if not (self.temperature >= 0.0) or not math.isfinite(self.temperature):
            raise ValueError(f"temperature must be finite and >= 0, got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if not (0.0 <= self.min_p < 1.0):
            raise ValueError(f"min_p must be in [0, 1), got {self.min_p}")

    def is_greedy(self) -> bool:
        """sampler.rs:33-37: temperature below the epsilon, or a single surviving token."""
        return self.temperature < GREEDY_TEMPERATURE or self.top_k == 1

    def effectively_greedy(self, vocab_size: int) -> bool:
        """Also greedy when top_p <= 1/vocab: only the argmax is in the nucleus
        (pegainfer-sample/src/lib.rs:297-303)."""
        return self.is_greedy() or (vocab_size > 0 and self.top_p <= 1.0 / vocab_size)


@dataclasses.dataclass
class TokenLogprob:
    """log-softmax (of the raw logits, no temperature) of a token, and the request's top-k
    (id, log-probability) pairs in descending order (pegainfer-frontend/src/engine.rs:55-58)."""

    logprob: float
    top_logprobs: List[Tuple[int, float]] = dataclasses.field(default_factory=list)


def mix_seed(seed: int, step: int) -> int:
    """SplitMix64 over (seed, step) (pegainfer-sample/src/lib.rs:283-288)."""
    m = (1 << 64) - 1
    z = (seed ^ ((step * 0x9E3779B97F4A7C15) & m)) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def uniform_from(seed: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32) from (seed, step)."""
    return (mix_seed(seed, step) >> 40) / float(1 << 24)
