"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a
token budget, decodes, finishes and frees.

Decisions follow the reference's scheduler (pegainfer-qwen3/src/scheduler.rs):

* three queues, ``deferred`` (waiting for room) -> ``prefilling`` (admitted, prompt not
  done, first come first served) -> ``active`` (decoding) (scheduler.rs:540-555);
* admission reserves a request's WHOLE lifetime in pages, ceil((prompt + max_tokens) / P)
  (or ceil(prompt / P) when max_tokens <= 1), against the free pages minus what admitted
  requests will still draw, and needs a free decode slot (scheduler.rs:1094-1119,
  1172-1258). So an admitted request never runs out of pages; there is no preemption and
  no swapping. A request that cannot fit now stays deferred (later, smaller requests may
  pass it); one that could never fit, or whose prompt + max_tokens exceeds the context
  limit, is rejected at once;
* an admitted request is announced to the executor (``begin``), which may answer that the front of its
  prompt is in the cache already (the reference's prefix cache, on by default there); its portions then
  start behind that;
* every step forwards at most ``max_prefill_tokens`` prompt tokens in total, taken from the
  front of ``prefilling`` (scheduler.rs:145-179), beside one token of every active request
  (plan.rs:56-87): prompt portions always ride along with decoding;
* a stop token ends a request without being emitted (unless ignore_eos); reaching
  max_tokens emits the token and ends it (scheduler/resolve.rs:148-170, 203-230);
* if a step fails all the same (the executor raises, e.g. pages ran out because the pool is
  smaller than reported), every request the step touched ends with an error and is
  dropped, and the scheduler goes on with the rest (scheduler.rs:1354-1378).

One step ahead (not in the reference, whose loop waits for every step's tokens): with an executor
that can ``launch`` a batch and ``collect`` its tokens later, ``step()`` launches batch n + 1 BEFORE it
collects batch n. A decoding request's next input is then "the token batch n draws for it", which
stays on the device, so the GPU goes from one step into the next while the host reads tokens, resolves
stops and plans. What the host cannot know in time is a stop token: a request that batch n ends with a
stop token has already been given a row in batch n + 1; that row's result is thrown away (its cache
pages are free for reuse at once: work on the device is ordered). Ends by length are known in advance
and get no such row. Events therefore arrive one call later; the tokens are the same.

The scheduler is host code only: it talks to an *executor* (the model runner plus
sampler, or a fake in tests).
"""
from __future__ import annotations

import dataclasses
import random
from typing import Dict, Hashable, List, Optional, Sequence

from ..sampling.params import SamplingParams, TokenLogprob

DEFAULT_MAX_PREFILL_TOKENS = 1024   # scheduler.rs:1170
DEFAULT_MAX_DECODE_BATCH = 256      # batch_decode_buffers.rs:25-28
DEFAULT_ENGINE_SEED = 42            # lib.rs:292


@dataclasses.dataclass
class Request:
    request_id: Hashable
    prompt_tokens: Sequence[int]
    max_tokens: int = 16
    sampling: SamplingParams = SamplingParams()
    logprobs: int = 0      # how many top log-probabilities to report beside each token's own (0: none)
    echo: bool = False     # with logprobs > 0: also the log-probabilities of the prompt's tokens


@dataclasses.dataclass
class Event:
    """What the scheduler reports: kind is "token", "finished", "rejected", "error" or "prompt_logprobs"."""

    request_id: Hashable
    kind: str
    token: Optional[int] = None
    reason: str = ""   # finished: "stop" | "length" | "cancelled"; rejected: "context_length" | "kv_budget" | "empty_prompt"; error: message
    logprob: Optional[TokenLogprob] = None              # with kind "token", when the request asked for logprobs
    prompt_logprobs: Optional[List[Optional[TokenLogprob]]] = None   # with kind "prompt_logprobs": one per prompt
                                                                      # position of a portion (None: the very first)


@dataclasses.dataclass
class PrefillItem:
    request_id: Hashable
    tokens: Sequence[int]     # this step's portion of the prompt
    is_last: bool             # the portion ends the prompt: its last row is sampled
    sampling: SamplingParams = SamplingParams()
    step_index: int = 0       # request-local count of tokens drawn so far
    logprobs: int = 0
    # echo with logprobs: the prompt token that follows each token of the portion (one fewer than tokens on
    # the last portion, whose last row is sampled); None otherwise
    targets: Optional[Sequence[int]] = None
    first_position: int = 0   # position of tokens[0] in the prompt


@dataclasses.dataclass
class DecodeItem:
    request_id: Hashable
    token: Optional[int]      # the last generated token, fed back; None: the one the batch in flight draws for it
    sampling: SamplingParams = SamplingParams()
    step_index: int = 0
    logprobs: int = 0


class Executor:
    """What the scheduler needs from below (the reference's ModelExecutor trait,
    pegainfer-qwen3/src/executor.rs:838-974)."""

    page_size: int
    total_pages: int

    def free_pages(self) -> int:
        raise NotImplementedError

    def free_slots(self) -> Optional[int]:
        """How many more requests the cache can hold open (per-request state slots); None: no such limit."""
        return None

    def execute(self, prefill: List[PrefillItem], decode: List[DecodeItem], step_seed: int) -> Dict[Hashable, int]:
        """Run one batch; returns the sampled token of every last portion and every decode item."""
        raise NotImplementedError

    def drop(self, request_id: Hashable) -> None:
        raise NotImplementedError

    def begin(self, request_id: Hashable, prompt_tokens: Sequence[int]) -> int:
        """A request has been admitted. Returns how many tokens at the front of its prompt are in the
        cache already (a prefix cache; 0 without one): its portions start behind them."""
        return 0

    # Optional, for running one step ahead: launch() starts a batch and returns a handle; a decode item
    # whose token is None takes the token that the batch of ``previous`` (a handle not collected yet)
    # draws for the same request. collect() waits for a launched batch and returns its tokens.
    supports_lookahead = False

    def launch(self, prefill: List[PrefillItem], decode: List[DecodeItem], step_seed: int, previous=None):
        raise NotImplementedError

    def collect(self, handle) -> Dict[Hashable, int]:
        raise NotImplementedError

    # After execute() / collect(): what the batch's requests asked for beside tokens.
    # request id -> {"token": TokenLogprob, "prompt": [TokenLogprob or None, ...]} (either may be missing)
    last_logprobs: Dict[Hashable, dict] = {}


@dataclasses.dataclass
class _Pending:
    req: Request
    done: int = 0        # prompt tokens already in the cache
    step_chunk: int = 0


@dataclasses.dataclass
class _Active:
    req: Request
    generated: List[int]
    last_token: int
    inflight: int = 0       # tokens drawn for it by batches that are launched and not collected yet
    ended: bool = False


@dataclasses.dataclass
class _Launched:
    handle: object
    rows: List[_Active]     # who gets a token from this batch


def lifetime_pages(prompt_len: int, max_tokens: int, page_size: int) -> int:
    """Pages a request can draw over its life (scheduler.rs:1094-1101)."""
    tokens = prompt_len if max_tokens <= 1 else prompt_len + max_tokens
    return max(1, -(-tokens // page_size))


def pages_for(tokens: int, page_size: int) -> int:
    return -(-tokens // page_size)


class Scheduler:
    def __init__(self, executor: Executor, *, max_context_tokens: int, stop_token_ids: Sequence[int] = (),
                 max_prefill_tokens: int = DEFAULT_MAX_PREFILL_TOKENS,
                 max_decode_batch: int = DEFAULT_MAX_DECODE_BATCH, seed: int = DEFAULT_ENGINE_SEED,
                 lookahead: Optional[bool] = None, batch_invariant: bool = False, row_alignment: int = 1) -> None:
        if max_prefill_tokens <= 0 or max_decode_batch <= 0:
            raise ValueError("max_prefill_tokens and max_decode_batch must be positive")
        self.executor = executor
        self.page_size = executor.page_size
        self.max_context_tokens = max_context_tokens
        self.stop_token_ids = set(int(t) for t in stop_token_ids)
        self.max_prefill_tokens = max_prefill_tokens
        self.max_decode_batch = max_decode_batch
        self.rng = random.Random(seed)
        # request-local portions (the reference's --batch-invariant, scheduler.rs:137-179): a request takes
        # min(what is left of its prompt, max_prefill_tokens) whole or waits, so where its prompt is cut
        # depends on its own length only
        self.batch_invariant = bool(batch_invariant)
        # A prompt that the token budget cuts anyway is cut so that the step's rows (portions + decoded
        # tokens) are a multiple of this: the products' row tiles are then all full. 1: no such trimming.
        self.row_alignment = max(1, int(row_alignment))
        self.deferred: List[Request] = []
        self.prefilling: List[_Pending] = []
        self.active: List[_Active] = []
        self.steps = 0
        can = bool(getattr(executor, "supports_lookahead", False))
        if lookahead and not can:
            raise ValueError("this executor cannot run one step ahead")
        self.lookahead = can if lookahead is None else bool(lookahead)
        self._inflight: Optional[_Launched] = None

    # ------------------------------------------------------------------ public
    def submit(self, req: Request) -> None:
        self.deferred.append(req)

    def has_work(self) -> bool:
        return bool(self.deferred or self.prefilling or self.active or self._inflight is not None)

    def cancel(self, request_id: Hashable) -> Optional[Event]:
        """Take a submitted request back (its client is gone). The reference retires a request as soon as
        its receiver has hung up and frees its pages at once (scheduler/effects.rs:209-224,
        pegainfer-qwen3/tests/scheduler_robustness.rs); here the caller says so.

        A request that still waits simply disappears; one whose prompt is being computed, or that decodes,
        is dropped and its pages, shared prefix pages and state slot go back now. With one step ahead a row
        of it may be in flight: that row's token is thrown away when it arrives, like the row behind a stop
        token (work on the device is ordered, so whoever gets the pages next writes them after that row has
        read them). Returns the event ``finished`` / ``cancelled``, or None if no such request is alive."""
        for i, req in enumerate(self.deferred):
            if req.request_id == request_id:
                del self.deferred[i]
                return Event(request_id, "finished", reason="cancelled")
        for i, p in enumerate(self.prefilling):
            if p.req.request_id == request_id:
                del self.prefilling[i]
                self.executor.drop(request_id)
                return Event(request_id, "finished", reason="cancelled")
        for a in self.active:
            if a.req.request_id == request_id and not a.ended:
                a.ended = True
                self.executor.drop(request_id)
                self.active = [x for x in self.active if x is not a]
                return Event(request_id, "finished", reason="cancelled")
        return None

    def load(self) -> Dict[str, int]:
        """Snapshot like the reference's LoadSnapshot (scheduler.rs:513-526)."""
        return {"kv_used_pages": self.executor.total_pages - self.executor.free_pages(),
                "kv_total_pages": self.executor.total_pages,
                "running": len(self.active) + len(self.prefilling), "waiting": len(self.deferred)}

    # ------------------------------------------------------------------ admission
    def _future_pages(self) -> int:
        P = self.page_size
        fut = 0
        for a in self.active:
            held = len(a.req.prompt_tokens) + len(a.generated) + a.inflight - 1  # the last token has no keys yet
            fut += max(0, lifetime_pages(len(a.req.prompt_tokens), a.req.max_tokens, P) - pages_for(held, P))
        for p in self.prefilling:
            fut += max(0, lifetime_pages(len(p.req.prompt_tokens), p.req.max_tokens, P) - pages_for(p.done, P))
        return fut

    def _admit(self) -> List[Event]:
        events: List[Event] = []
        budget = max(0, self.executor.free_pages() - self._future_pages())
        slots = max(0, self.max_decode_batch - len(self.active) - len(self.prefilling))
        open_slots = self.executor.free_slots()
        if open_slots is not None:      # a request that finds no state slot waits, like one that finds no pages
            slots = min(slots, max(0, int(open_slots)))
        still: List[Request] = []
        for req in self.deferred:
            n = len(req.prompt_tokens)
            if n == 0:
                events.append(Event(req.request_id, "rejected", reason="empty_prompt"))
                continue
            if n + req.max_tokens > self.max_context_tokens:
                events.append(Event(req.request_id, "rejected", reason="context_length"))
                continue
            need = lifetime_pages(n, req.max_tokens, self.page_size)
            if need > self.executor.total_pages:
                events.append(Event(req.request_id, "rejected", reason="kv_budget"))
                continue
            if need <= budget and slots > 0:
                budget -= need
                slots -= 1
                try:
                    # prompt log-probabilities need the logits of every prompt position: nothing is taken from a prefix cache
                    cached = 0 if (req.echo and req.logprobs > 0) else int(self.executor.begin(req.request_id, req.prompt_tokens))
                except Exception as e:
                    events.append(Event(req.request_id, "error", reason=f"{type(e).__name__}: {e}"))
                    continue
                self.prefilling.append(_Pending(req, done=min(max(cached, 0), n - 1)))
            else:
                still.append(req)
        self.deferred = still
        return events

    # ------------------------------------------------------------------ portions
    def _take_prefill(self, other_rows: int = 0) -> List[_Pending]:
        """The prompt portions of the next step; ``other_rows``: the rows that decoding requests add to it."""
        budget = self.max_prefill_tokens
        taken: List[_Pending] = []
        i = 0
        while i < len(self.prefilling) and budget > 0:
            p = self.prefilling[i]
            left = len(p.req.prompt_tokens) - p.done
            if self.batch_invariant:
                chunk = min(left, self.max_prefill_tokens)
                if chunk > budget:      # whole or not at all: a later, shorter request may still fit
                    i += 1
                    continue
            else:
                chunk = min(left, budget)
            p.step_chunk = chunk
            budget -= chunk
            taken.append(self.prefilling.pop(i))
        if taken and self.row_alignment > 1 and not self.batch_invariant:
            last = taken[-1]
            rows = other_rows + sum(p.step_chunk for p in taken)
            over = rows % self.row_alignment
            # only a prompt that is cut here anyway gives up tokens, and only if whole tiles remain
            if (over and last.step_chunk < len(last.req.prompt_tokens) - last.done and rows > self.row_alignment
                    and last.step_chunk > over):
                last.step_chunk -= over
        return taken

    def _prefill_item(self, p: "_Pending") -> PrefillItem:
        req = p.req
        lo, hi = p.done, p.done + p.step_chunk
        targets = None
        if req.echo and req.logprobs > 0:
            targets = req.prompt_tokens[lo + 1: hi + 1]      # the last portion has one target fewer than tokens
        return PrefillItem(req.request_id, req.prompt_tokens[lo:hi], is_last=hi == len(req.prompt_tokens),
                           sampling=req.sampling, step_index=0, logprobs=req.logprobs, targets=targets, first_position=lo)

    # ------------------------------------------------------------------ one iteration
    def step(self) -> List[Event]:
        """Admit, build one batch, run it, resolve. Returns this iteration's events."""
        if self.lookahead:
            return self._step_ahead()
        events = self._admit()
        decoding = list(self.active)
        taken = self._take_prefill(len(decoding))
        if not taken and not decoding:
            return events
        prefill_items = [self._prefill_item(p) for p in taken]
        decode_items = [DecodeItem(a.req.request_id, a.last_token, a.req.sampling, len(a.generated), a.req.logprobs)
                        for a in decoding]
        step_seed = self.rng.getrandbits(64)
        self.steps += 1
        try:
            tokens = self.executor.execute(prefill_items, decode_items, step_seed)
        except Exception as e:  # the step failed: everyone it touched fails, the rest goes on
            for p in taken:
                events.append(Event(p.req.request_id, "error", reason=f"{type(e).__name__}: {e}"))
                self.executor.drop(p.req.request_id)
            for a in decoding:
                events.append(Event(a.req.request_id, "error", reason=f"{type(e).__name__}: {e}"))
                self.executor.drop(a.req.request_id)
            self.active = []
            return events

        extra = getattr(self.executor, "last_logprobs", None) or {}
        self._report_prompt_logprobs(extra, events)
        # decode rows first (they are older), then the requests whose prompt just ended
        for a in decoding:
            self._resolve(a, tokens[a.req.request_id], events, extra.get(a.req.request_id, {}).get("token"))
        unfinished: List[_Pending] = []
        for p in taken:
            p.done += p.step_chunk
            if p.done < len(p.req.prompt_tokens):
                unfinished.append(p)
                continue
            a = _Active(p.req, [], -1)
            self.active.append(a)
            self._resolve(a, tokens[p.req.request_id], events, extra.get(p.req.request_id, {}).get("token"))
        self.prefilling = unfinished + self.prefilling  # back to the front (effects.rs:318-406)
        return events

    # ------------------------------------------------------------------ one iteration, one step ahead
    def _step_ahead(self) -> List[Event]:
        """Launch the next batch, then collect the one launched by the previous call."""
        events = self._admit()
        previous = self._inflight
        self._inflight, failed = self._launch_next(previous)
        if previous is not None:
            try:
                tokens = self.executor.collect(previous.handle)
            except Exception as e:
                self._fail(previous.rows, e, events)
                tokens = None
            extra = (getattr(self.executor, "last_logprobs", None) or {}) if tokens is not None else {}
            self._report_prompt_logprobs(extra, events)
            for a in previous.rows:
                a.inflight -= 1
                if tokens is not None and not a.ended:   # ended meanwhile (a stop token one step earlier): the row is void
                    self._resolve(a, tokens[a.req.request_id], events, extra.get(a.req.request_id, {}).get("token"))
        if failed is not None:   # the launch failed: everyone it touched fails, after what was in flight has arrived
            e, taken, decoding = failed
            for p in taken:
                events.append(Event(p.req.request_id, "error", reason=f"{type(e).__name__}: {e}"))
                self.executor.drop(p.req.request_id)
            self._fail(decoding, e, events)
        return events

    def _launch_next(self, previous: Optional[_Launched]):
        # who decodes: everyone who is still alive once the tokens in flight have arrived (a stop token
        # among those cannot be known yet)
        decoding = [a for a in self.active if len(a.generated) + a.inflight < max(1, a.req.max_tokens)]
        taken = self._take_prefill(len(decoding))
        if not taken and not decoding:
            return None, None
        prefill_items = [self._prefill_item(p) for p in taken]
        decode_items = [DecodeItem(a.req.request_id, a.last_token if a.inflight == 0 else None, a.req.sampling,
                                   len(a.generated) + a.inflight, a.req.logprobs) for a in decoding]
        step_seed = self.rng.getrandbits(64)
        self.steps += 1
        try:
            handle = self.executor.launch(prefill_items, decode_items, step_seed,
                                          previous.handle if previous is not None else None)
        except Exception as e:
            return None, (e, taken, decoding)
        rows = list(decoding)
        unfinished: List[_Pending] = []
        for p in taken:
            p.done += p.step_chunk
            if p.done < len(p.req.prompt_tokens):
                unfinished.append(p)
                continue
            a = _Active(p.req, [], -1)
            self.active.append(a)
            rows.append(a)
        self.prefilling = unfinished + self.prefilling
        for a in rows:
            a.inflight += 1
        return _Launched(handle, rows), None

    def _fail(self, rows: List[_Active], e: Exception, events: List[Event]) -> None:
        for a in rows:
            if a.ended:
                continue
            a.ended = True
            events.append(Event(a.req.request_id, "error", reason=f"{type(e).__name__}: {e}"))
            self.executor.drop(a.req.request_id)
        self.active = [x for x in self.active if not x.ended]

    @staticmethod
    def _report_prompt_logprobs(extra: Dict[Hashable, dict], events: List[Event]) -> None:
        for rid, what in extra.items():
            if what.get("prompt") is not None:
                events.append(Event(rid, "prompt_logprobs", prompt_logprobs=what["prompt"]))

    def _resolve(self, a: _Active, token: int, events: List[Event], logprob: Optional[TokenLogprob] = None) -> None:
        req = a.req
        if token in self.stop_token_ids and not req.sampling.ignore_eos:
            self._finish(a, events, "stop")
            return
        a.generated.append(token)
        a.last_token = token
        events.append(Event(req.request_id, "token", token=token, logprob=logprob))
        if len(a.generated) >= max(1, req.max_tokens):
            self._finish(a, events, "length")

    def _finish(self, a: _Active, events: List[Event], reason: str) -> None:
        events.append(Event(a.req.request_id, "finished", reason=reason))
        a.ended = True
        self.executor.drop(a.req.request_id)
        self.active = [x for x in self.active if x is not a]

    def run(self) -> List[Event]:
        """Iterate until every submitted request has ended."""
        events: List[Event] = []
        idle = 0
        while self.has_work():
            got = self.step()
            events.extend(got)
            idle = idle + 1 if not got else 0
            if idle > 3 and not self.prefilling and not self.active:
                # nothing runs and nothing was admitted: the deferred requests can never fit
                for req in self.deferred:
                    events.append(Event(req.request_id, "rejected", reason="kv_budget"))
                self.deferred = []
        return events
