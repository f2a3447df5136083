"""Sizing the page pool from a memory budget.

As the reference does (pegainfer-qwen3/src/weights.rs:662-841): run one worst-case step
(``max_prefill_tokens`` prompt tokens) against a small temporary cache, take the peak
memory it needed beside the cache, and give the pool
``total * gpu_memory_utilization - that peak - margin``.
"""
from __future__ import annotations

import torch

from ..cache.manager import CacheManager
from .runner import ModelRunner, StepEntry, _dtype_of


def pages_from_memory_budget(config, weights_seed, folder, dtype, device, page_size: int,
                             utilization: float, margin_mib: int, max_prefill_tokens: int, prefix_cache: bool = False,
                             max_requests: int = 256, strict_weights: bool = False):
    """Build the runner with a pool sized from free memory. Returns (runner, num_pages).
    ``max_requests``: how many requests may be open at once (state slots)."""
    if not (0.0 < utilization <= 1.0):
        raise ValueError(f"gpu_memory_utilization must be in (0, 1], got {utilization}")
    tdtype = _dtype_of(dtype)
    probe_tokens = max(1, min(max_prefill_tokens, config.max_position_embeddings
                              if hasattr(config, "max_position_embeddings") else max_prefill_tokens))
    probe_pages = -(-probe_tokens // page_size) + 1
    runner = ModelRunner.build(config, weights_seed, dtype=dtype, device=device, page_size=page_size,
                               num_pages=probe_pages, max_requests=8, folder=folder, strict_weights=strict_weights)
    dev = torch.device(device)
    esize = 4 if tdtype == torch.float32 else 2
    probe_bytes = sum(runner.cache.bytes_per_page(g, esize) for g in range(len(runner.cache.groups))) * probe_pages
    torch.cuda.synchronize(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    runner.step([StepEntry("__probe__", [0] * probe_tokens, [probe_tokens - 1])])
    runner.end("__probe__")
    torch.cuda.synchronize(dev)
    peak_other = torch.cuda.max_memory_allocated(dev) - probe_bytes
    _, total = torch.cuda.mem_get_info(dev)
    budget = int(total * utilization) - peak_other - margin_mib * (1 << 20)
    per_page = sum(runner.cache.bytes_per_page(g, esize) for g in range(len(runner.cache.groups)))
    num_pages = budget // max(per_page, 1)
    if num_pages < 4:
        raise RuntimeError(
            f"memory budget leaves room for {num_pages} cache pages "
            f"(total {total >> 20} MiB, utilization {utilization}, other peak {peak_other >> 20} MiB)")
    # replace the probe cache by the real one
    model, ignored = runner.model, runner.ignored_tensors
    del runner
    torch.cuda.empty_cache()
    cache = CacheManager(page_size=page_size, prefix_cache=prefix_cache)
    model.bind_cache(cache)
    cache.allocate(int(num_pages), int(max_requests), device=dev, dtype=tdtype)
    runner = ModelRunner(model, cache, dev)
    runner.ignored_tensors = ignored
    return runner, int(num_pages)
