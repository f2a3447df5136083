"""The scheduler's decisions with a fake executor (no GPU)."""
from typing import Dict, List

import pytest

from openinfer_b200.engine.scheduler import (DecodeItem, Event, Executor, PrefillItem, Request, Scheduler,
                                             lifetime_pages)
from openinfer_b200.sampling.params import SamplingParams


class FakeExecutor(Executor):
    """Counts pages like the real cache does and 'generates' token = (last input token + 1) % 100."""

    def __init__(self, total_pages=64, page_size=4, fail_on_step=None, real_pages=None):
        self.page_size, self.total_pages = page_size, total_pages
        self.real_pages = total_pages if real_pages is None else real_pages  # what there really is
        self.tokens: Dict[object, int] = {}
        self.batches: List[tuple] = []
        self.dropped: List[object] = []
        self.fail_on_step = fail_on_step

    def used(self):
        return sum(-(-n // self.page_size) for n in self.tokens.values())

    def free_pages(self):
        return self.total_pages - self.used()

    def execute(self, prefill, decode, step_seed):
        self.batches.append(([(p.request_id, len(p.tokens), p.is_last) for p in prefill],
                             [d.request_id for d in decode]))
        if self.fail_on_step is not None and len(self.batches) - 1 == self.fail_on_step:
            raise RuntimeError("injected failure")
        out = {}
        grow = {p.request_id: len(p.tokens) for p in prefill}
        grow.update({d.request_id: 1 for d in decode})
        need = sum(-(-(self.tokens.get(r, 0) + n) // self.page_size) - -(-self.tokens.get(r, 0) // self.page_size)
                   for r, n in grow.items())
        if need > self.real_pages - self.used():
            raise RuntimeError("OutOfPages")
        for p in prefill:
            self.tokens[p.request_id] = self.tokens.get(p.request_id, 0) + len(p.tokens)
            if p.is_last:
                out[p.request_id] = (p.tokens[-1] + 1) % 100
        for d in decode:
            self.tokens[d.request_id] += 1
            out[d.request_id] = (d.token + 1) % 100
        return out

    def drop(self, rid):
        self.dropped.append(rid)
        self.tokens.pop(rid, None)


def sched(ex, **kw):
    kw.setdefault("max_context_tokens", 1000)
    return Scheduler(ex, **kw)


def collect(events):
    toks, fin = {}, {}
    for e in events:
        if e.kind == "token":
            toks.setdefault(e.request_id, []).append(e.token)
        else:
            fin[e.request_id] = (e.kind, e.reason)
    return toks, fin


def test_lifetime_pages():
    assert lifetime_pages(5, 3, 4) == 2 and lifetime_pages(5, 1, 4) == 2 and lifetime_pages(8, 1, 4) == 2
    assert lifetime_pages(8, 2, 4) == 3 and lifetime_pages(1, 0, 4) == 1


def test_generates_and_frees():
    ex = FakeExecutor()
    s = sched(ex)
    s.submit(Request("a", [1, 2, 3], max_tokens=4))
    toks, fin = collect(s.run())
    assert toks["a"] == [4, 5, 6, 7] and fin["a"] == ("finished", "length")
    assert ex.dropped == ["a"] and ex.used() == 0
    # the first token comes from the prompt's last step; three decode steps follow
    assert ex.batches[0] == ([("a", 3, True)], []) and all(b == ([], ["a"]) for b in ex.batches[1:]) and len(ex.batches) == 4


def test_prompt_cut_under_token_budget_fifo_and_mixed_with_decode():
    ex = FakeExecutor(total_pages=200)
    s = sched(ex, max_prefill_tokens=10)
    s.submit(Request("a", list(range(4)), max_tokens=8))
    s.submit(Request("b", list(range(23)), max_tokens=2))
    s.submit(Request("c", list(range(5)), max_tokens=2))
    s.run()
    pre = [b[0] for b in ex.batches]
    assert pre[0] == [("a", 4, True), ("b", 6, False)]          # budget 10: a whole, b's first 6
    assert pre[1] == [("b", 10, False)]                          # b stays at the front
    assert pre[2] == [("b", 7, True), ("c", 3, False)]
    assert pre[3] == [("c", 2, True)]
    assert ex.batches[1][1] == ["a"] and ex.batches[2][1] == ["a"]  # a decodes beside b's portions
    assert sum(n for step in pre for _, n, _ in step) == 4 + 23 + 5


def test_stop_token_not_emitted_and_ignore_eos():
    ex = FakeExecutor()
    s = sched(ex, stop_token_ids=[6])
    s.submit(Request("a", [3], max_tokens=10))                                   # 4, 5, then 6 = stop
    s.submit(Request("b", [3], max_tokens=5, sampling=SamplingParams(ignore_eos=True)))
    s.submit(Request("c", [5], max_tokens=5))                                    # first token is the stop token
    toks, fin = collect(s.run())
    assert toks["a"] == [4, 5] and fin["a"] == ("finished", "stop")
    assert toks["b"] == [4, 5, 6, 7, 8] and fin["b"] == ("finished", "length")
    assert "c" not in toks and fin["c"] == ("finished", "stop")
    assert sorted(ex.dropped) == ["a", "b", "c"]


def test_max_tokens_one_finishes_after_prompt():
    ex = FakeExecutor()
    s = sched(ex)
    s.submit(Request("a", [1, 2], max_tokens=1))
    toks, fin = collect(s.run())
    assert toks["a"] == [3] and fin["a"] == ("finished", "length") and len(ex.batches) == 1


def test_rejections():
    ex = FakeExecutor(total_pages=4, page_size=4)
    s = sched(ex, max_context_tokens=50)
    s.submit(Request("long", list(range(45)), max_tokens=10))   # 55 > 50
    s.submit(Request("big", list(range(20)), max_tokens=4))     # 6 pages > 4 in total
    s.submit(Request("empty", [], max_tokens=4))
    s.submit(Request("ok", [1, 2, 3], max_tokens=4))
    toks, fin = collect(s.run())
    assert fin["long"] == ("rejected", "context_length") and fin["big"] == ("rejected", "kv_budget")
    assert fin["empty"] == ("rejected", "empty_prompt") and fin["ok"] == ("finished", "length")
    assert all(rid == "ok" for b in ex.batches for rid, _, _ in b[0])


def test_admission_reserves_whole_lifetime_so_pages_never_run_out():
    """Three requests of 3 pages each in a pool of 7: two run, the third waits until one ends."""
    ex = FakeExecutor(total_pages=7, page_size=4)
    s = sched(ex)
    for rid in "abc":
        s.submit(Request(rid, list(range(6)), max_tokens=6))     # ceil(12 / 4) = 3 pages
    events = []
    seen_c_start = None
    while s.has_work():
        events += s.step()
        assert ex.used() <= 7
        if seen_c_start is None and any(rid == "c" for rid, _, _ in ex.batches[-1][0]):
            seen_c_start = len(ex.batches)
            assert ex.dropped, "c was admitted before anyone finished"
    toks, fin = collect(events)
    assert all(len(toks[r]) == 6 and fin[r] == ("finished", "length") for r in "abc")
    assert ex.used() == 0 and seen_c_start is not None


def test_later_smaller_request_may_pass_a_deferred_one():
    ex = FakeExecutor(total_pages=5, page_size=4)
    s = sched(ex)
    s.submit(Request("a", list(range(8)), max_tokens=4))    # 3 pages
    s.submit(Request("b", list(range(8)), max_tokens=4))    # 3 pages: does not fit beside a
    s.submit(Request("c", list(range(2)), max_tokens=2))    # 1 page: fits
    s.step()
    assert {rid for rid, _, _ in ex.batches[0][0]} == {"a", "c"}
    assert [r.request_id for r in s.deferred] == ["b"]
    toks, fin = collect(s.run())
    assert fin["b"] == ("finished", "length")


def test_decode_slots_limit():
    ex = FakeExecutor(total_pages=100)
    s = sched(ex, max_decode_batch=2)
    for rid in "abc":
        s.submit(Request(rid, [1], max_tokens=3))
    s.step()
    assert len(ex.batches[0][0]) == 2 and len(s.deferred) == 1
    s.run()
    assert max(len(b[1]) for b in ex.batches) <= 2


def test_failed_step_fails_everyone_it_touched_and_the_rest_goes_on():
    ex = FakeExecutor(fail_on_step=2)
    s = sched(ex)
    s.submit(Request("a", [1, 2], max_tokens=5))
    s.submit(Request("b", [1, 2], max_tokens=5))
    ev = s.step() + s.step() + s.step()
    toks, fin = collect(ev)
    assert fin["a"][0] == "error" and fin["b"][0] == "error" and "injected" in fin["a"][1]
    assert sorted(ex.dropped) == ["a", "b"] and not s.active and ex.used() == 0
    s.submit(Request("c", [7], max_tokens=2))
    toks, fin = collect(s.run())
    assert toks["c"] == [8, 9] and fin["c"] == ("finished", "length")


def test_pages_run_out_when_the_pool_is_smaller_than_reported():
    """The decided behaviour when a step cannot get its pages: the step's requests fail with an
    error and are dropped; nothing hangs, the scheduler stays usable."""
    ex = FakeExecutor(total_pages=12, page_size=4, real_pages=2)
    s = Scheduler(ex, max_context_tokens=1000)
    s.submit(Request("a", list(range(12)), max_tokens=4))
    toks, fin = collect(s.run())
    assert fin["a"][0] == "error" and "OutOfPages" in fin["a"][1]
    assert ex.dropped == ["a"] and not s.has_work()


def test_per_step_seed_is_reproducible():
    seeds = []

    class Rec(FakeExecutor):
        def execute(self, prefill, decode, step_seed):
            seeds.append(step_seed)
            return super().execute(prefill, decode, step_seed)

    for _ in range(2):
        s = sched(Rec(), seed=42)
        s.submit(Request("a", [1], max_tokens=3))
        s.run()
    assert seeds[:3] == seeds[3:] and len(set(seeds[:3])) == 3


# ---------------------------------------------------------------------------
# one step ahead: batch n + 1 is launched before batch n's tokens are read
# ---------------------------------------------------------------------------
class AheadExecutor(FakeExecutor):
    """The fake with launch/collect: a decode item without a token takes the one the batch before
    drew for it. Keeps at most one batch uncollected, as the scheduler promises."""

    supports_lookahead = True

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.uncollected = 0

    def launch(self, prefill, decode, step_seed, previous=None):
        assert self.uncollected <= 1, "two batches were in flight before this launch"
        resolved = []
        for d in decode:
            if d.token is None:
                assert previous is not None and d.request_id in previous, "a token in flight that nobody draws"
                resolved.append(DecodeItem(d.request_id, previous[d.request_id], d.sampling, d.step_index))
            else:
                resolved.append(d)
        out = self.execute(prefill, resolved, step_seed)
        self.uncollected += 1
        return out

    def collect(self, handle):
        self.uncollected -= 1
        return handle


def run_both(make_requests, **kw):
    results = []
    for cls in (FakeExecutor, AheadExecutor):
        ex = cls(**kw.get("ex", {}))
        s = sched(ex, **kw.get("sched", {}))
        assert s.lookahead == (cls is AheadExecutor)
        for r in make_requests():
            s.submit(r)
        results.append((collect(s.run()), ex))
    return results


def test_one_step_ahead_gives_the_same_tokens_and_ends():
    def reqs():
        return [Request("a", [1, 2, 3], max_tokens=6), Request("b", list(range(10, 30)), max_tokens=1),
                Request("c", [50], max_tokens=3), Request("d", [7, 8], max_tokens=40)]
    (sync, ex0), (ahead, ex1) = run_both(reqs, sched={"max_prefill_tokens": 8, "stop_token_ids": [20]})
    assert sync == ahead
    assert sync[1]["d"] == ("finished", "stop") and sync[1]["a"] == ("finished", "length")
    assert ex1.used() == 0 and sorted(ex1.dropped) == sorted(ex0.dropped)
    # d drew its stop token while it already had a row in the next batch: one row more, thrown away
    rows_of_d = [sum("d" in dec for _, dec in ex.batches) for ex in (ex0, ex1)]
    assert rows_of_d[1] == rows_of_d[0] + 1 and ex1.uncollected == 0
    # a, b and c end by length, which is known in advance: no row more
    for r in "ac":
        assert sum(r in dec for _, dec in ex0.batches) == sum(r in dec for _, dec in ex1.batches)


def test_one_step_ahead_never_launches_a_row_past_max_tokens():
    ex = AheadExecutor(total_pages=4, page_size=4)   # room for exactly prompt + max_tokens
    s = sched(ex)
    s.submit(Request("a", list(range(8)), max_tokens=8))
    toks, fin = collect(s.run())
    assert len(toks["a"]) == 8 and fin["a"] == ("finished", "length")
    assert all(len(d) <= 1 for _, d in ex.batches)


def test_one_step_ahead_failed_launch_fails_who_it_touched():
    ex = AheadExecutor(fail_on_step=3)
    s = sched(ex)
    s.submit(Request("a", [1, 2, 3], max_tokens=10))
    events = s.run()
    toks, fin = collect(events)
    assert fin["a"][0] == "error" and "injected failure" in fin["a"][1]
    assert toks["a"] == [4, 5, 6]       # the three batches before the failing one were collected
    assert ex.dropped == ["a"] and not s.has_work()
    s.submit(Request("b", [1], max_tokens=2))
    toks, fin = collect(s.run())
    assert toks["b"] == [2, 3] and fin["b"] == ("finished", "length")


def test_one_step_ahead_is_refused_without_an_executor_for_it():
    with pytest.raises(ValueError):
        sched(FakeExecutor(), lookahead=True)
    assert not sched(AheadExecutor(), lookahead=False).lookahead


def test_portions_start_behind_what_the_executor_already_has():
    """An executor with a prefix cache answers `begin` with the tokens it already holds."""
    class Prefixed(FakeExecutor):
        def begin(self, rid, prompt):
            n = 8 if list(prompt[:8]) == list(range(8)) else 0
            self.tokens[rid] = n
            return n

    ex = Prefixed()
    s = sched(ex, max_prefill_tokens=5)
    s.submit(Request("a", list(range(12)), max_tokens=2))     # 8 cached: portions of 4 tokens in all
    s.submit(Request("b", [9, 9, 9], max_tokens=1))
    toks, fin = collect(s.run())
    assert ex.batches[0][0] == [("a", 4, True), ("b", 1, False)]
    assert toks["a"] == [12, 13] and fin["a"] == ("finished", "length") and toks["b"] == [10]
    assert ex.used() == 0


def test_request_local_portions_take_whole_or_wait():
    """With batch_invariant a request takes min(left, max_prefill_tokens) whole or not at all, so where its
    prompt is cut depends on its own length only (and a later, shorter request may pass a waiting one)."""
    def cuts(batch_invariant, others):
        ex = FakeExecutor(total_pages=200)
        s = sched(ex, max_prefill_tokens=8, batch_invariant=batch_invariant)
        if others:
            s.submit(Request("x", list(range(5)), max_tokens=1))
        s.submit(Request("a", list(range(20)), max_tokens=1))
        if others:
            s.submit(Request("y", list(range(3)), max_tokens=1))
        s.run()
        return [n for pre, _ in ex.batches for rid, n, _ in pre if rid == "a"], ex.batches

    alone, _ = cuts(True, False)
    with_others, batches = cuts(True, True)
    assert alone == with_others == [8, 8, 4]
    # step 0: x takes 5, a's 8 do not fit and wait, y's 3 fit behind
    assert batches[0][0] == [("x", 5, True), ("y", 3, True)]
    assert cuts(False, True)[0] != alone          # the default fills the budget: a is cut by what x left over


def test_a_cut_portion_fills_whole_row_tiles():
    """With a row alignment, a prompt that the budget cuts anyway gives up as many tokens as make the step's
    rows (portions + decoded tokens) a multiple of it; a prompt that ends in the step is never shortened."""
    ex = FakeExecutor(total_pages=4000, page_size=4)
    s = sched(ex, max_prefill_tokens=64, row_alignment=16, lookahead=False, max_context_tokens=100000)
    for rid, n in (("a", 5), ("b", 7), ("c", 9)):
        s.submit(Request(rid, list(range(n)), 50, SamplingParams()))
    s.step()                                        # 21 prompt tokens end here: nothing to trim
    assert [x[1] for x in ex.batches[-1][0]] == [5, 7, 9]
    s.submit(Request("long", list(range(300)), 4, SamplingParams()))
    s.step()                                        # 3 decoded tokens + a cut of 64 -> 61 (64 rows)
    pre, dec = ex.batches[-1]
    assert len(dec) == 3 and [x[1] for x in pre] == [61]
    s.step()
    assert [x[1] for x in ex.batches[-1][0]] == [61]
    # without alignment the budget is filled
    ex2 = FakeExecutor(total_pages=4000, page_size=4)
    s2 = sched(ex2, max_prefill_tokens=64, lookahead=False, max_context_tokens=100000)
    s2.submit(Request("a", list(range(5)), 50, SamplingParams()))
    s2.step()
    s2.submit(Request("long", list(range(300)), 4, SamplingParams()))
    s2.step()
    assert [x[1] for x in ex2.batches[-1][0]] == [64]
    # the last portion of a prompt is taken whole even if it leaves a ragged tile
    ex3 = FakeExecutor(total_pages=4000, page_size=4)
    s3 = sched(ex3, max_prefill_tokens=64, row_alignment=16, lookahead=False, max_context_tokens=100000)
    s3.submit(Request("a", list(range(5)), 50, SamplingParams()))
    s3.step()
    s3.submit(Request("p", list(range(40)), 4, SamplingParams()))
    s3.step()
    assert [x[1] for x in ex3.batches[-1][0]] == [40]


@pytest.mark.parametrize("ahead", [False, True])
def test_cancel_in_every_state(ahead):
    """A request is taken back while it waits, in the middle of its prompt, while it decodes and (one step
    ahead) with a row in flight: it reports `finished / cancelled` once, nothing more of it arrives, its
    pages come back at once, and the other requests' tokens are what they are without it."""
    def others():
        return [Request("keep", [1, 2, 3], max_tokens=8), Request("keep2", [40, 41], max_tokens=5)]

    ex0 = (AheadExecutor if ahead else FakeExecutor)()
    s0 = sched(ex0, max_prefill_tokens=4)
    for r in others():
        s0.submit(r)
    want, _ = collect(s0.run())

    for state in ("deferred", "prefilling", "decoding", "never"):
        ex = (AheadExecutor if ahead else FakeExecutor)(total_pages=64, page_size=4)
        s = sched(ex, max_prefill_tokens=4, max_decode_batch=3 if state != "deferred" else 2)
        for r in others():
            s.submit(r)
        s.submit(Request("gone", list(range(10, 22)), max_tokens=30))
        events = []
        if state == "deferred":
            events += s.step()
            assert [r.request_id for r in s.deferred] == ["gone"]       # no decode slot for it
        elif state == "prefilling":
            while not any(p.req.request_id == "gone" and p.done > 0 for p in s.prefilling):
                events += s.step()
        elif state == "decoding":
            while not any(a.req.request_id == "gone" and (a.generated or a.inflight) for a in s.active):
                events += s.step()
            if ahead:
                assert any(a.req.request_id == "gone" and a.inflight for a in s.active)   # a row of it is in flight
        ev = s.cancel("gone" if state != "never" else "nobody")
        if state == "never":
            assert ev is None
            ev = s.cancel("gone")
        assert ev.kind == "finished" and ev.reason == "cancelled"
        assert s.cancel("gone") is None                        # only once
        assert ("gone" in ex.tokens) is False                  # its pages are back already
        n_before = sum(1 for e in events if e.request_id == "gone" and e.kind == "token")
        rest = s.run()
        assert not [e for e in rest if e.request_id == "gone"], "a cancelled request reported something"
        toks, fin = collect(events + rest)
        assert {k: v for k, v in toks.items() if k != "gone"} == want
        assert len(toks.get("gone", [])) == n_before
        assert ex.used() == 0 and not s.has_work()
        if ahead:
            assert ex.uncollected == 0


def test_state_slots_are_a_limit_of_admission_not_an_error():
    """When the cache can hold fewer requests open than max_decode_batch allows, the ones that find no slot
    wait for one (they are not failed)."""
    class Slotted(FakeExecutor):
        slots = 2

        def free_slots(self):
            return self.slots - len(self.tokens)

        def begin(self, rid, prompt):
            assert self.free_slots() > 0, "admitted without a state slot"
            self.tokens[rid] = 0
            return 0

    ex = Slotted()
    s = sched(ex, max_decode_batch=8)
    for i in range(5):
        s.submit(Request(i, [i, i + 1], max_tokens=3))
    first = s.step()
    assert len(s.prefilling) + len(s.active) == 2 and len(s.deferred) == 3
    toks, fin = collect(first + s.run())
    assert all(fin[i] == ("finished", "length") and len(toks[i]) == 3 for i in range(5))
    assert max(len(p) + len(d) for p, d in ex.batches) <= 2


def test_batch_invariant_and_prefix_cache_do_not_go_together(tmp_path):
    """As in the reference (pegainfer-qwen3/src/lib.rs:549-554): a prefix-cache hit moves a prompt's portions off the
    request's own grid, so the command line refuses --batch-invariant without --no-prefix-cache (before anything is
    built), and so does the Python entry point when both are asked for."""
    import json
    import subprocess
    import sys

    from helpers import ROOT, TINY
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(TINY["A"][0]))
    out = subprocess.run([sys.executable, "-m", "openinfer_b200", "--random-config", str(cfg_file), "--prompt-ids", "1,2,3",
                          "--batch-invariant"], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 2 and "--no-prefix-cache" in out.stderr, (out.returncode, out.stderr[-300:])

    from openinfer_b200.engine.engine import LLM
    from openinfer_b200.kernels import policy
    try:
        with pytest.raises(ValueError, match="prefix_cache"):
            LLM(str(tmp_path), batch_invariant=True, prefix_cache=True)
    finally:
        policy.set_batch_invariant(False)
