"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step`` takes portions of prompts and single decoded tokens side by side,
cut anywhere, runs only the rows it is given against what earlier steps left in the
cache, and returns float32 logits at the wanted rows. It is the one path by which
tokens reach the model: generation, the scheduler and trace replay all call it. The
reference's three entry points (execute_prefill / execute_decode / execute_unified,
pegainfer-qwen3/src/executor.rs:2549-2857) are special cases of this one.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import RELEASED, CacheManager
from ..cache.pool import OutOfPages
from ..config.base import load_config, resolve_architecture
from ..kernels import lib as kernel_lib
from ..kernels import ops
from ..parts.model import Model
from ..weights.loader import load_tensors
from ..weights.random import random_tensors
from .context import GroupStep, StepContext


class StepError(ValueError):
    """A step that cannot run as given (bad token id, position beyond the model's range, ...)."""


@dataclasses.dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()   # places among ``tokens`` whose logits are asked for
    token_from: Optional[int] = None   # a single token that is not known to the host yet: element
                                       # ``token_from`` of the ``device_tokens`` given to step()


def _dtype_of(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if name not in table:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")
    return table[name]


def _align4(n: int) -> int:
    return (n + 3) & ~3


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, device: torch.device) -> None:
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        self.spec = model.spec
        self._staging: List[torch.Tensor] = []
        self._staging_events: List[Optional[torch.cuda.Event]] = []
        self._staging_turn = 0
        self._device_tokens: Optional[torch.Tensor] = None
        self.steps_run = 0
        self.cuda_graph = False          # record decode-only steps as CUDA graphs and replay them
        # the largest batch a recorded step is made for: every request that can be open at once
        self.max_graph_batch = int(getattr(cache, "max_requests", 0) or 256)
        self._graphs: Dict[tuple, tuple] = {}
        self._graph_pool = None
        self._graph_safe: Optional[bool] = None
        self.ignored_tensors: List[str] = []   # names in the model folder that the model did not ask for

    # ------------------------------------------------------------------ construction
    @classmethod
    def build(cls, config, tensors_or_seed, dtype="bfloat16", device="cuda:0", *, page_size: int = 16,
              num_pages: Optional[int] = None, max_tokens: Optional[int] = None,
              max_requests: int = 256, folder: Optional[str] = None, prefix_cache: bool = False,
              strict_weights: bool = False) -> "ModelRunner":
        """Assemble model + cache on the device.

        ``tensors_or_seed``: None to load ``folder``'s safetensors, or an int seed for
        random weights drawn on the device. The pool holds ``num_pages`` pages per group,
        or enough for ``max_tokens`` positions (rounded up to whole pages). Tensors of the
        folder that the model does not name are left unread and listed in
        ``runner.ignored_tensors`` (an error only with ``strict_weights``)."""
        dtype = _dtype_of(dtype)
        device = torch.device(device)
        if device.type != "cuda":
            raise kernel_lib.KernelError(
                f"device {device} is not a CUDA device; this engine has no CPU path")
        if not torch.cuda.is_available():
            raise kernel_lib.KernelError("no CUDA device is available; this engine has no CPU path")
        kernel_lib.load()  # build / load now: a missing extension fails here, loudly
        torch.cuda.set_device(device)
        # the true 32-bit path must not use a reduced-precision matrix mode anywhere
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        # library products of bfloat16 operands add up in float32 throughout, as the reference's do
        # (cublasGemmEx with CUBLAS_COMPUTE_32F, pegainfer-kernels/csrc/shared/linear.cu:312-362): no
        # partial sums of a split K rounded to bfloat16
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        entry = resolve_architecture(config.to_dict())
        spec = entry.build_spec(config)
        model = Model(spec, dtype)
        expected = model.expected_tensors()
        ignored: List[str] = []
        if tensors_or_seed is None:
            if folder is None:
                raise ValueError("either a folder or a seed is needed")
            tensors = load_tensors(folder, expected, dtype, device, strict=strict_weights, ignored=ignored)
        else:
            tensors = random_tensors(expected, int(tensors_or_seed), dtype=dtype, device=device)
        model.load(tensors, device)
        del tensors
        cache = CacheManager(page_size=page_size, prefix_cache=prefix_cache)
        model.bind_cache(cache)
        if num_pages is None:
            if max_tokens is None:
                raise ValueError("give num_pages or max_tokens")
            num_pages = max(1, -(-int(max_tokens) // page_size))
        cache.allocate(num_pages, max_requests, device=device, dtype=dtype)
        runner = cls(model, cache, device)
        runner.ignored_tensors = ignored
        return runner

    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **kw) -> "ModelRunner":
        config = load_config(folder)
        return cls.build(config, None, dtype=dtype, device=device, folder=folder, **kw)

    # ------------------------------------------------------------------ helpers
    def _pinned(self, host: np.ndarray) -> torch.Tensor:
        """The step's metadata in pinned host memory (a ring of buffers, so that the host can write the
        next step's while the device has not read this one's yet)."""
        n = host.size
        if not self._staging or self._staging[0].numel() < n:
            if self._staging:
                torch.cuda.current_stream().synchronize()   # kernels in flight may still read the old buffers
            self._staging = [torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._staging_events = [None] * 4
            self._staging_turn = 0
        self._staging_turn = (self._staging_turn + 1) % len(self._staging)
        event = self._staging_events[self._staging_turn]
        if event is not None:
            event.synchronize()   # the step that used this buffer four steps ago has read it
        buf = self._staging[self._staging_turn]
        buf[:n].numpy()[:] = host
        self._staging_last_bytes = n * 4
        return buf

    def _upload(self, dev: torch.Tensor, host: np.ndarray, sections: Dict[str, int], T: int, entries, fence: bool = True) -> None:
        """Metadata to the device by a KERNEL that reads the pinned buffer (no copy-engine operation between
        the steps' kernels); the same kernel puts in the token ids that the host does not know yet. ``fence``:
        the step's kernels are launched one by one behind it and read the metadata before their own wait, so the
        first of them gets plain stream order (a recorded graph is ordered behind the copy as a whole)."""
        buf = self._pinned(host)
        feed = any(e.token_from is not None for e in entries)
        ops.copy_words(dev, buf, host.size, ids_off=sections["token_ids"] if feed else -1, src_off=sections["token_src"],
                       n_ids=T if feed else 0, tokens=self._device_tokens if feed else None, fence=fence)
        event = torch.cuda.Event()
        event.record()
        self._staging_events[self._staging_turn] = event

    def validate(self, entries: Sequence[StepEntry]) -> None:
        vocab, max_pos = self.spec.vocab_size, self.spec.max_positions
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            lo, hi = (min(e.tokens), max(e.tokens)) if n > 1 else (e.tokens[0], e.tokens[0])
            if not (0 <= int(lo) and int(hi) < vocab):
                bad = next(t for t in e.tokens if not 0 <= int(t) < vocab)
                raise StepError(f"request {e.request_id!r}: token id {bad} outside [0, {vocab})")
            if len(e.want) and not (0 <= int(min(e.want)) and int(max(e.want)) < n):
                bad = next(w for w in e.want if not 0 <= int(w) < n)
                raise StepError(f"request {e.request_id!r}: wanted place {bad} outside its {n} tokens")
            held = self.cache.num_tokens(e.request_id) if self.cache.has(e.request_id) else 0
            if max_pos and held + n > max_pos:
                raise StepError(
                    f"request {e.request_id!r}: {held + n} positions exceed max_position_embeddings {max_pos}")

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch. Returns float32 logits [wanted rows, vocab] on the device, rows in
        the order of the entries and of each entry's ``want`` (None when nothing is wanted).
        ``device_tokens`` (int32, on the device): where entries with ``token_from`` take their token.

        The returned tensor is valid until the next call of ``step``: a step that is replayed as a recorded
        graph returns a view of that graph's output buffer, which the next replay overwrites (work queued on
        the same stream before the next call, like the sampler's, reads it safely; keep ``logits.clone()``
        to hold it longer).

        Raises ``OutOfPages`` with nothing changed if the cache cannot hold the new rows."""
        entries = list(entries)
        if not entries:
            return None
        self.validate(entries)
        self._device_tokens = device_tokens
        if any(e.token_from is not None for e in entries):
            if device_tokens is None or device_tokens.dtype != torch.int32 or not device_tokens.is_cuda:
                raise StepError("entries with token_from need int32 device_tokens")
            for e in entries:
                if e.token_from is not None and (len(e.tokens) != 1 or not 0 <= e.token_from < device_tokens.numel()):
                    raise StepError(f"request {e.request_id!r}: token_from {e.token_from} needs one token and an index "
                                    f"below {device_tokens.numel()}")
        cache = self.cache
        opened, reserved = [], []
        try:
            starts = []
            for e in entries:
                if not cache.has(e.request_id):
                    cache.open(e.request_id)
                    opened.append(e.request_id)
                starts.append(cache.reserve(e.request_id, len(e.tokens)))
                reserved.append(e.request_id)
        except OutOfPages:
            for rid in reserved:
                cache.rollback(rid)
            for rid in opened:
                cache.close(rid)
            raise
        try:
            if (self.graphs_usable() and len(entries) <= self.max_graph_batch
                    and all(len(e.tokens) == 1 for e in entries)):
                logits = self._step_decode_graph(entries, starts)
            else:
                ctx, row_idx = self._build_context(entries, starts)
                logits = self.model.run(ctx, row_idx)
        except Exception:
            for rid in reserved:
                cache.rollback(rid)
            for rid in opened:
                cache.close(rid)
            raise
        for e in entries:     # token ids the host knows let the prefix cache register full pages of them
            cache.commit(e.request_id, tokens=None if e.token_from is not None else e.tokens)
        self.steps_run += 1
        return logits

    def begin(self, request_id: Hashable, prompt_tokens: Sequence[int]) -> int:
        """Open a request ahead of its first step and let it share registered pages that match the front
        of its prompt (the prefix cache). Returns how many prompt tokens are already in the cache: the first
        step of the request brings the tokens behind them."""
        return self.cache.begin(request_id, [int(t) for t in prompt_tokens])

    def end(self, request_id: Hashable) -> None:
        """The request is finished: its pages and state slot go back to the pools."""
        if self.cache.has(request_id):
            self.cache.close(request_id)

    # ------------------------------------------------------------------ metadata
    @staticmethod
    def _layout(T: int, B: int, max_pages: int, G: int, n_want: int):
        """Sections of the packed int32 metadata buffer (each starts on a 16-byte boundary)."""
        sections: Dict[str, int] = {}
        off = 0
        for name, size in (("token_ids", T), ("token_src", T), ("positions", T), ("token_req", T), ("cu_seqlens", B + 1),
                           ("state_slots", B)):
            sections[name] = off
            off += _align4(size)
        for g in range(G):
            for name, size in ((f"slots{g}", T), (f"table{g}", B * max_pages), (f"kv_lens{g}", B)):
                sections[name] = off
                off += _align4(size)
        sections["want"] = off
        off += _align4(max(n_want, 1))
        return sections, off

    def _fill(self, host: np.ndarray, sections: Dict[str, int], entries: List[StepEntry], starts: List[int],
              T: int, B: int, max_pages: int) -> List[int]:
        """Write one step's metadata into ``host``. ``T`` and ``B`` may exceed the real row and
        request counts (a padded decode batch): the extra rows belong to no request (token_req -1),
        store nothing (slot -1) and see one key of page 0. Returns the wanted row numbers."""
        cache = self.cache
        P = cache.page_size
        G = len(cache.groups)

        def view(name, size):
            return host[sections[name]: sections[name] + size]

        tok, pos, req = view("token_ids", T), view("positions", T), view("token_req", T)
        src = view("token_src", T)
        cu = view("cu_seqlens", B + 1)
        slots_host = view("state_slots", B)
        tok[:] = 0
        src[:] = -1
        pos[:] = 0
        req[:] = -1
        slots_host[:] = 0
        want_rows: List[int] = []
        row = 0
        for b, e in enumerate(entries):
            n = len(e.tokens)
            tok[row: row + n] = np.asarray(e.tokens, dtype=np.int32)
            pos[row: row + n] = np.arange(starts[b], starts[b] + n, dtype=np.int32)
            req[row: row + n] = b
            if e.token_from is not None:
                src[row] = e.token_from
            cu[b] = row
            slots_host[b] = cache.state_slot(e.request_id)
            want_rows.extend(row + int(w) for w in e.want)
            row += n
        for b in range(len(entries), B + 1):   # padding requests bring one row each
            cu[b] = row + (b - len(entries))
        for g in range(G):
            sl = view(f"slots{g}", T)
            tb = view(f"table{g}", B * max_pages).reshape(B, max_pages)
            kl = view(f"kv_lens{g}", B)
            sl[:] = -1
            tb[:] = 0
            kl[:] = 1
            row = 0
            for b, e in enumerate(entries):
                table = np.asarray(cache.block_table(e.request_id, g), dtype=np.int32)
                n = len(e.tokens)
                p = np.arange(starts[b], starts[b] + n)
                sl[row: row + n] = table[p // P] * P + (p % P)
                shown = np.where(table == RELEASED, 0, table)  # never read: behind the window
                tb[b, : len(shown)] = shown[:max_pages]
                kl[b] = starts[b] + n
                row += n
        return want_rows

    def _context(self, dev: torch.Tensor, sections: Dict[str, int], T: int, B: int, max_pages: int,
                 q_lens: List[int], starts: List[int], kv_lens: List[int], slots: List[int]) -> StepContext:
        cache = self.cache

        def dview(name, size):
            return dev[sections[name]: sections[name] + size]

        groups = [
            GroupStep(slot_mapping=dview(f"slots{g}", T),
                      block_table=dview(f"table{g}", B * max_pages).view(B, max_pages),
                      kv_lens=dview(f"kv_lens{g}", B), window=cache.groups[g].window)
            for g in range(len(cache.groups))
        ]
        return StepContext(
            num_tokens=T, num_requests=B, token_ids=dview("token_ids", T), positions=dview("positions", T),
            token_req=dview("token_req", T), cu_seqlens=dview("cu_seqlens", B + 1),
            state_slots=dview("state_slots", B), groups=groups, cache=cache,
            q_lens_host=q_lens, starts_host=list(starts), kv_lens_host=kv_lens, state_slots_host=slots,
            decode_only=all(n == 1 for n in q_lens), max_q_len=max(q_lens), max_kv_len=max(kv_lens))

    def _build_context(self, entries: List[StepEntry], starts: List[int]):
        cache = self.cache
        P = cache.page_size
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        kv_lens = [s + n for s, n in zip(starts, q_lens)]
        max_pages = max(1, max(-(-kv // P) for kv in kv_lens))
        n_want = sum(len(e.want) for e in entries)
        sections, total = self._layout(T, B, max_pages, len(cache.groups), n_want)
        host = np.zeros(total, dtype=np.int32)
        want_rows = self._fill(host, sections, entries, starts, T, B, max_pages)
        if n_want:
            host[sections["want"]: sections["want"] + n_want] = np.asarray(want_rows, dtype=np.int32)
        dev = torch.empty(total, dtype=torch.int32, device=self.device)
        self._upload(dev, host, sections, T, entries)
        slots = [cache.state_slot(e.request_id) for e in entries]
        ctx = self._context(dev, sections, T, B, max_pages, q_lens, starts, kv_lens, slots)
        row_idx = dev[sections["want"]: sections["want"] + n_want] if n_want else None
        return ctx, row_idx

    # ------------------------------------------------------------------ decode through CUDA graphs
    def graphs_usable(self) -> bool:
        """Recorded decode steps are used when asked for and every mixer reads the step's
        metadata from device tensors only."""
        if not getattr(self, "cuda_graph", False):
            return False
        if getattr(self, "_graph_safe", None) is None:
            self._graph_safe = all(b.mixer is None or getattr(b.mixer, "graph_safe", False)
                                   for b in self.model.blocks)
        return self._graph_safe

    def _decode_graph(self, bucket: int, cap: int):
        """The recorded decode step for a padded batch of ``bucket`` rows whose block tables
        hold ``cap`` pages (the reference keeps one graph per batch bucket too,
        pegainfer-qwen3/src/batch_decode.rs:69-182, pegainfer-core/src/cuda_graph.rs:42-231)."""
        key = (bucket, cap)
        entry = self._graphs.get(key)
        if entry is not None:
            return entry
        G = len(self.cache.groups)
        sections, total = self._layout(bucket, bucket, cap, G, bucket)
        meta = torch.zeros(total, dtype=torch.int32, device=self.device)
        host = np.zeros(total, dtype=np.int32)
        self._fill(host, sections, [], [], bucket, bucket, cap)
        host[sections["want"]: sections["want"] + bucket] = np.arange(bucket, dtype=np.int32)
        meta.copy_(torch.from_numpy(host))
        ctx = self._context(meta, sections, bucket, bucket, cap, [1] * bucket, [0] * bucket, [1] * bucket,
                            [0] * bucket)
        ctx.static_decode = True
        row_idx = meta[sections["want"]: sections["want"] + bucket]

        def run():
            return self.model.run(ctx, row_idx)

        # warm-up on a side stream (plans and workspaces are made here, outside the recording)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run()
            run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = kernel_lib.launch_count()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = run()
        recorded = kernel_lib.launch_count() - before   # kernels one replay stands for
        kernel_lib.replayed -= recorded                 # the recording itself ran none of them
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        entry = (graph, meta, sections, total, logits, (ctx, recorded))
        self._graphs[key] = entry
        return entry

    def _step_decode_graph(self, entries: List[StepEntry], starts: List[int]) -> Optional[torch.Tensor]:
        B = len(entries)
        P = self.cache.page_size
        bucket = 1
        while bucket < B:
            bucket *= 2
        need_pages = max(-(-(s + 1) // P) for s in starts)
        cap = 16
        while cap < need_pages:
            cap *= 2
        graph, meta, sections, total, logits, (_, recorded) = self._decode_graph(bucket, cap)
        host = np.zeros(total, dtype=np.int32)
        want_rows = self._fill(host, sections, entries, starts, bucket, bucket, cap)
        host[sections["want"]: sections["want"] + bucket] = np.arange(bucket, dtype=np.int32)
        self._upload(meta, host, sections, bucket, entries, fence=False)
        graph.replay()
        kernel_lib.replayed += recorded
        if not want_rows:
            return None
        if want_rows == list(range(len(want_rows))):
            return logits[: len(want_rows)]
        return logits[torch.tensor(want_rows, device=self.device)]
