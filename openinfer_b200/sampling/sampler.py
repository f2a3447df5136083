"""Token selection for a batch of logits rows: greedy rows through the argmax kernel,
the others through the sampling kernel; one device-to-host copy of the chosen ids.

The split follows the reference's ``select_batch`` (pegainfer-sample/src/lib.rs:148-276):
rows that are effectively greedy take the argmax path; a seeded row's draw is a function
of (its seed, its own step) only, so it does not depend on what else is in the batch; an
unseeded row draws from the engine's per-step seed and its row number.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams, mix_seed, uniform_from


class PendingTokens:
    """Token ids chosen on the device and on their way to the host (a copy into pinned memory
    and an event behind it); ``device`` may feed the next step before the host has looked."""

    def __init__(self, device: Optional[torch.Tensor], host: Optional[torch.Tensor], event) -> None:
        self.device, self._host, self._event = device, host, event

    def result(self) -> List[int]:
        if self.device is None:
            return []
        self._event.synchronize()
        return [int(t) for t in self._host.tolist()]


class Sampler:
    def __init__(self, vocab_size: int, device: torch.device) -> None:
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self._probs: Optional[torch.Tensor] = None
        self._pinned: List[torch.Tensor] = []   # a small ring of pinned buffers for the copies to the host
        self._turn = 0
        # the rows' parameters travel the other way through a ring of pinned buffers too: a kernel reads them
        # into one device buffer, so the host never waits for the stream (a copy from pageable memory does)
        self._param_pinned: List[torch.Tensor] = []
        self._param_turn = 0
        self._param_dev: Optional[torch.Tensor] = None

    def _host_buffer(self, n: int) -> torch.Tensor:
        if not self._pinned or self._pinned[0].numel() < n:
            self._pinned = [torch.empty(max(256, 2 * n), dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._turn = (self._turn + 1) % len(self._pinned)
        return self._pinned[self._turn][:n]

    def _param_buffers(self, words: int):
        if not self._param_pinned or self._param_pinned[0].numel() < words:
            torch.cuda.current_stream().synchronize()     # nothing reads the old buffers any more
            size = max(1024, 2 * words)
            self._param_pinned = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._param_dev = torch.empty(size, dtype=torch.int32, device=self.device)
        self._param_turn = (self._param_turn + 1) % len(self._param_pinned)
        return self._param_pinned[self._param_turn], self._param_dev

    def select(self, logits: torch.Tensor, params: Sequence[SamplingParams], steps: Sequence[int],
               step_seed: int) -> List[int]:
        """``logits`` float32 [rows, vocab]; ``steps[i]`` is row i's request-local step
        (how many tokens that request has drawn so far). Returns one token id per row."""
        return self.select_async(logits, params, steps, step_seed).result()

    def select_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], steps: Sequence[int],
                     step_seed: int) -> PendingTokens:
        """As ``select``, without waiting: the ids stay on the device and travel to the host behind an event."""
        n = len(params)
        if n == 0:
            return PendingTokens(None, None, None)
        if logits.shape[0] != n or logits.shape[1] != self.vocab_size:
            raise ValueError(f"logits {tuple(logits.shape)} do not match {n} rows of vocab {self.vocab_size}")
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        sampled = [i for i, p in enumerate(params) if not p.effectively_greedy(self.vocab_size)]
        if len(sampled) < n:
            ops.argmax(out, logits)  # every row; sampled rows are overwritten below
        if sampled:
            k = len(sampled)
            # [temperature | top_p | min_p | uniform] as float32 bit patterns, then top_k and the rows' numbers
            pinned, dev = self._param_buffers(6 * k)
            words = pinned.numpy()
            host = words[: 4 * k].view(np.float32).reshape(4, k)
            topk = words[4 * k: 5 * k]
            which = words[5 * k: 6 * k]
            for j, i in enumerate(sampled):
                p = params[i]
                host[0, j] = p.temperature
                host[1, j] = p.top_p
                host[2, j] = p.min_p
                host[3, j] = (uniform_from(p.seed, steps[i]) if p.seed is not None
                              else uniform_from(mix_seed(step_seed, i), steps[i]))
                topk[j] = p.top_k if 0 < p.top_k < self.vocab_size else 0
                which[j] = i
            ops.copy_words(dev, pinned, 6 * k)
            fl = dev[: 4 * k].view(torch.float32).view(4, k)
            tk = dev[4 * k: 5 * k]
            idx = dev[5 * k: 6 * k]
            rows = logits if k == n else logits.index_select(0, idx)
            if self._probs is None or self._probs.numel() < k * self.vocab_size:
                self._probs = torch.empty(k * self.vocab_size, dtype=torch.float32, device=self.device)
            picked = torch.empty(k, dtype=torch.int32, device=self.device)
            ops.sample(picked, rows.contiguous(), self._probs, fl[0], tk, fl[1], fl[2], fl[3])
            if k == n:
                out = picked
            else:
                out.index_copy_(0, idx.to(torch.int64), picked)   # greedy rows keep their argmax
        host = self._host_buffer(n)
        ops.copy_words(host, out, n)     # a kernel writes the ids into pinned host memory: no copy-engine operation
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(out, host, event)
