"""The generation engine: model runner + sampler as the scheduler's executor, and the
Python entry point ``LLM.generate`` (token ids in, token ids out; tokenizers live outside).

The reference has no Python API (it serves HTTP); its programmatic surface is the
executor plus ``EngineHandle::submit`` (pegainfer-qwen3/src/lib.rs:199-213,
pegainfer-frontend/src/engine.rs:67-95). Option names and defaults follow its command
line (pegainfer-frontend/src/model_line.rs:85-187, pegainfer-qwen3/src/model_line.rs:32-118).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config.base import ModelConfig, load_config
from ..kernels import ops
from ..sampling.params import SamplingParams, TokenLogprob
from ..sampling.sampler import Sampler
from .runner import ModelRunner, StepEntry
from .scheduler import (DEFAULT_ENGINE_SEED, DEFAULT_MAX_DECODE_BATCH, DEFAULT_MAX_PREFILL_TOKENS, DecodeItem,
                        Event, Executor, PrefillItem, Request, Scheduler)

DEFAULT_GPU_MEMORY_UTILIZATION = 0.90   # pegainfer-qwen3/src/weights.rs:31-36
DEFAULT_KV_MARGIN_MIB = 150
DEFAULT_KV_PAGE_SIZE = 16
# rows of a mixed step are made a multiple of the widest row tile of the prompt products: the kernels say how wide
from ..kernels.gemm_tcgen05 import ROW_TILE as DEFAULT_ROW_ALIGNMENT  # noqa: E402


class RunnerExecutor(Executor):
    """Executes the scheduler's batches on the model runner and samples the wanted rows."""

    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self.page_size = runner.cache.page_size
        self.total_pages = runner.cache.num_pages
        self.sampler = Sampler(runner.spec.vocab_size, runner.device)
        self.last_logprobs: Dict[Hashable, dict] = {}

    def free_pages(self) -> int:
        return self.runner.cache.min_free_pages()

    def free_slots(self) -> int:
        return self.runner.cache.slot_pool.free_count

    supports_lookahead = True

    def execute(self, prefill: List[PrefillItem], decode: List[DecodeItem], step_seed: int) -> Dict[Hashable, int]:
        return self.collect(self.launch(prefill, decode, step_seed))

    def launch(self, prefill: List[PrefillItem], decode: List[DecodeItem], step_seed: int, previous=None):
        """Start one batch on the GPU. Returns (request ids of the sampled rows, their pending tokens,
        request id -> place among the sampled rows, pending log-probabilities or None)."""
        entries, rows = [], []
        sample_at: List[int] = []       # which row of the returned logits each sampled row is
        echo: List[tuple] = []          # (request id, first prompt position, first logits row, targets, top-k)
        at = 0                          # logits rows so far
        for p in prefill:
            n = len(p.tokens)
            if p.targets is not None:   # prompt log-probabilities: the logits of every position of the portion
                entries.append(StepEntry(p.request_id, p.tokens, list(range(n))))
                echo.append((p.request_id, p.first_position, at, list(p.targets), p.logprobs))
                if p.is_last:
                    sample_at.append(at + n - 1)
                    rows.append(p)
                at += n
            else:
                entries.append(StepEntry(p.request_id, p.tokens, [n - 1] if p.is_last else []))
                if p.is_last:
                    sample_at.append(at)
                    rows.append(p)
                    at += 1
        feed = None
        for d in decode:
            if d.token is None:
                # the token comes from the batch launched before this one, which the host has not read yet
                if previous is None or d.request_id not in previous[2]:
                    raise ValueError(f"request {d.request_id!r} has a token in flight but no batch that draws it")
                feed = previous[1].device
                entries.append(StepEntry(d.request_id, [0], [0], token_from=previous[2][d.request_id]))
            else:
                entries.append(StepEntry(d.request_id, [d.token], [0]))
            sample_at.append(at)
            rows.append(d)
            at += 1
        logits = self.runner.step(entries, device_tokens=feed)
        ids = [r.request_id for r in rows]
        pending = None
        if rows:
            picked_rows = logits if sample_at == list(range(logits.shape[0])) else \
                logits[torch.tensor(sample_at, device=logits.device)]
            pending = self.sampler.select_async(picked_rows, [r.sampling for r in rows], [r.step_index for r in rows], step_seed)
        lp = self._launch_logprobs(logits, rows, sample_at, pending, echo)
        return ids, pending, {rid: i for i, rid in enumerate(ids)}, lp

    def _launch_logprobs(self, logits, rows, sample_at, pending, echo):
        """One kernel for every log-probability the batch's requests asked for: of the drawn tokens (ids still
        on the device) and, for echo, of the prompt's tokens. Returns what collect() needs, or None."""
        want_tok = [(i, r) for i, r in enumerate(rows) if r.logprobs > 0]
        if not want_tok and not echo:
            return None
        dev = logits.device
        lrows = [sample_at[i] for i, _ in want_tok]
        ks = [r.logprobs for _, r in want_tok]
        picked = pending.device[torch.tensor([i for i, _ in want_tok], device=dev)].to(torch.int32) if want_tok else \
            torch.empty(0, dtype=torch.int32, device=dev)
        spans = []
        for rid, first_pos, row0, targets, k in echo:
            spans.append((rid, first_pos, len(lrows), len(targets)))
            lrows.extend(range(row0, row0 + len(targets)))
            ks.extend([k] * len(targets))
            picked = torch.cat([picked, torch.tensor(targets, dtype=torch.int32, device=dev)])
        k_max = max(ks) if ks else 0
        lpv, vals, tids = ops.token_logprobs(logits, torch.tensor(lrows, dtype=torch.int32, device=dev), picked,
                                             torch.tensor(ks, dtype=torch.int32, device=dev), k_max)
        return [r.request_id for _, r in want_tok], spans, ks, lpv, vals, tids

    def collect(self, handle) -> Dict[Hashable, int]:
        ids, pending, _, lp = handle
        self.last_logprobs = {}
        tokens = dict(zip(ids, pending.result())) if pending is not None else {}
        if lp is not None:
            tok_ids, spans, ks, lpv, vals, tids = lp
            lpv, vals, tids = lpv.cpu().tolist(), vals.cpu().tolist(), tids.cpu().tolist()

            def entry(i):
                return TokenLogprob(lpv[i], [(tids[i][j], vals[i][j]) for j in range(ks[i]) if tids[i][j] >= 0])

            for i, rid in enumerate(tok_ids):
                self.last_logprobs.setdefault(rid, {})["token"] = entry(i)
            for rid, first_pos, at, n in spans:
                got = [entry(at + j) for j in range(n)]
                # position 0 of the prompt has nothing in front of it
                self.last_logprobs.setdefault(rid, {})["prompt"] = ([None] if first_pos == 0 else []) + got
        return tokens

    def drop(self, request_id: Hashable) -> None:
        self.runner.end(request_id)

    def begin(self, request_id: Hashable, prompt_tokens: Sequence[int]) -> int:
        return self.runner.begin(request_id, prompt_tokens)


@dataclasses.dataclass
class GenerationResult:
    request_id: Hashable
    token_ids: List[int]
    finish_reason: str   # "stop" | "length" | "rejected:<why>" | "error:<message>"
    logprobs: Optional[List[Optional[TokenLogprob]]] = None          # one per generated token, when asked for
    prompt_logprobs: Optional[List[Optional[TokenLogprob]]] = None   # one per prompt token (None for the first), with echo


class LLM:
    """Load a model folder (or build a random model from a config and a seed) and generate.

    >>> llm = LLM("/path/to/model")                        # config.json + safetensors
    >>> llm.generate([[1, 2, 3]], max_tokens=8)            # greedy
    [[...8 token ids...]]
    """

    def __init__(self, model_path: Optional[str] = None, *, config: Optional[ModelConfig] = None,
                 seed: Optional[int] = None, dtype: str = "bfloat16", device_ordinal: int = 0,
                 kv_page_size: int = DEFAULT_KV_PAGE_SIZE, num_pages: Optional[int] = None,
                 max_cache_tokens: Optional[int] = None,
                 gpu_memory_utilization: float = DEFAULT_GPU_MEMORY_UTILIZATION,
                 kv_cache_memory_margin_mib: int = DEFAULT_KV_MARGIN_MIB,
                 max_prefill_tokens: int = DEFAULT_MAX_PREFILL_TOKENS,
                 max_decode_batch: int = DEFAULT_MAX_DECODE_BATCH, engine_seed: int = DEFAULT_ENGINE_SEED,
                 cuda_graph: bool = True, lookahead: bool = True, prefix_cache: Optional[bool] = None,
                 batch_invariant: Optional[bool] = None, runner: Optional[ModelRunner] = None,
                 row_alignment: int = DEFAULT_ROW_ALIGNMENT, strict_weights: bool = False) -> None:
        from ..kernels import policy
        if batch_invariant is not None:
            policy.set_batch_invariant(batch_invariant)   # process-wide: which kernels take which step shapes
        batch_invariant = policy.batch_invariant()
        # A hit in the prefix cache moves a prompt's portions off the request's own grid (they then start where
        # the cached pages end), and a position's bits depend on the portion it is computed in: the two do not go
        # together, as in the reference (pegainfer-qwen3/src/lib.rs:549-554: --batch-invariant requires
        # --no-prefix-cache). Left open, the prefix cache is on unless the policy is.
        if prefix_cache is None:
            prefix_cache = not batch_invariant
        if batch_invariant and (prefix_cache or (runner is not None and runner.cache.prefix_cache)):
            raise ValueError("batch_invariant requires prefix_cache=False: a prefix-cache hit moves a prompt's portions "
                             "off the request's own grid, so bit-identical results cannot be promised")
        device = f"cuda:{device_ordinal}"
        weights_seed = None
        if runner is not None:
            pass  # model, weights and cache already stand
        elif model_path is not None:
            config = load_config(model_path)
            weights_seed = None
        elif config is not None and seed is not None:
            weights_seed = seed
        else:
            raise ValueError("give model_path, or config and seed for random weights")
        if runner is not None:
            self.runner = runner
        elif num_pages is None and max_cache_tokens is None:
            from .memory import pages_from_memory_budget

            self.runner, _ = pages_from_memory_budget(
                config, weights_seed, model_path, dtype, device, kv_page_size, gpu_memory_utilization,
                kv_cache_memory_margin_mib, max_prefill_tokens, prefix_cache=prefix_cache,
                max_requests=max_decode_batch, strict_weights=strict_weights)
        else:
            self.runner = ModelRunner.build(
                config, weights_seed, dtype=dtype, device=device, page_size=kv_page_size, num_pages=num_pages,
                max_tokens=max_cache_tokens, max_requests=max_decode_batch, folder=model_path,
                prefix_cache=prefix_cache, strict_weights=strict_weights)
        self.runner.cuda_graph = cuda_graph
        self.config = config
        self.executor = RunnerExecutor(self.runner)
        max_context = self.runner.spec.max_positions or (1 << 30)
        self.scheduler = Scheduler(
            self.executor, max_context_tokens=max_context, stop_token_ids=self.runner.spec.stop_token_ids,
            max_prefill_tokens=max_prefill_tokens, max_decode_batch=max_decode_batch, seed=engine_seed,
            lookahead=lookahead, batch_invariant=batch_invariant, row_alignment=row_alignment)
        self._next_id = 0

    # ---- step-wise use: submit requests, then call step() until has_work() is false
    def submit(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None,
               max_tokens: int = 16, logprobs: int = 0, echo: bool = False) -> Hashable:
        rid = self._next_id
        self._next_id += 1
        self.scheduler.submit(Request(rid, list(prompt_token_ids), int(max_tokens), sampling_params or SamplingParams(),
                                      int(logprobs), bool(echo)))
        return rid

    def step(self) -> List[Event]:
        """One scheduler iteration: host tokens in, one batch on the GPU, sampled tokens out. With
        ``lookahead`` (the default) the batch launched by this call is collected by the next one: its
        events arrive one call later, and the GPU runs on while the host reads and plans."""
        return self.scheduler.step()

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def cancel(self, request_id: Hashable) -> bool:
        """Take a submitted request back, in whatever state it is: waiting, in the middle of its prompt, or
        decoding. Its pages are free at once; no further token of it is reported. False if it is not alive."""
        return self.scheduler.cancel(request_id) is not None

    def generate_detailed(self, prompt_token_ids: Sequence[Sequence[int]],
                          sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                          max_tokens: Union[int, Sequence[int]] = 16, logprobs: int = 0,
                          echo: bool = False) -> List[GenerationResult]:
        """``logprobs`` = k > 0: every generated token comes with its log-probability and the k most likely
        tokens' (raw logits, no temperature); with ``echo`` also the prompt's tokens (the reference's request
        options of the same names, pegainfer-frontend/src/engine.rs:67-95)."""
        n = len(prompt_token_ids)
        if sampling_params is None:
            sampling_params = SamplingParams()
        sp = [sampling_params] * n if isinstance(sampling_params, SamplingParams) else list(sampling_params)
        mt = [max_tokens] * n if isinstance(max_tokens, int) else list(max_tokens)
        if len(sp) != n or len(mt) != n:
            raise ValueError("sampling_params / max_tokens must be single values or one per prompt")
        ids = []
        for i in range(n):
            rid = self._next_id
            self._next_id += 1
            ids.append(rid)
            self.scheduler.submit(Request(rid, list(prompt_token_ids[i]), int(mt[i]), sp[i], int(logprobs), bool(echo)))
        out: Dict[Hashable, GenerationResult] = {
            rid: GenerationResult(rid, [], "", [] if logprobs > 0 else None, [] if (logprobs > 0 and echo) else None)
            for rid in ids}
        for ev in self.scheduler.run():
            r = out.get(ev.request_id)
            if r is None:
                continue
            if ev.kind == "token":
                r.token_ids.append(ev.token)
                if r.logprobs is not None:
                    r.logprobs.append(ev.logprob)
            elif ev.kind == "prompt_logprobs":
                if r.prompt_logprobs is not None:
                    r.prompt_logprobs.extend(ev.prompt_logprobs)
            elif ev.kind == "finished":
                r.finish_reason = ev.reason
            elif ev.kind in ("rejected", "error"):
                r.finish_reason = f"{ev.kind}:{ev.reason}"
        return [out[rid] for rid in ids]

    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 max_tokens: Union[int, Sequence[int]] = 16) -> List[List[int]]:
        """Generated token ids per prompt (host lists in, host lists out)."""
        results = self.generate_detailed(prompt_token_ids, sampling_params, max_tokens)
        for r in results:
            if r.finish_reason.startswith(("rejected", "error")):
                raise RuntimeError(f"request {r.request_id} did not run: {r.finish_reason}")
        return [r.token_ids for r in results]


def generate(model_path: str, prompt_token_ids: Sequence[Sequence[int]], max_tokens: int = 16,
             sampling_params: Optional[SamplingParams] = None, **engine_options) -> List[List[int]]:
    """One-call form: load ``model_path``, generate, return token ids per prompt."""
    return LLM(model_path, **engine_options).generate(prompt_token_ids, sampling_params, max_tokens)
