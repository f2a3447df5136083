"""Generation through the Python entry point and the command line."""
import json
import os
import random
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
from helpers import ROOT, TINY, make_model_folder, random_tokens, oracle_logits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_model_folder(str(tmp_path_factory.mktemp(f"g{n}")), cfg, seed) for n, (cfg, seed) in list(TINY.items())[:2]}


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(folders, name):
    """Config A: prompts of 5/11/17 tokens, 8 greedy tokens; B: 1/9/33/70 in portions of 13."""
    from openinfer_b200 import LLM
    cfg, w = plain.read_model_folder(folders[name])
    rng = random.Random(11)
    lens = [5, 11, 17] if name == "A" else [1, 9, 33, 70]
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in lens]
    n_new = 8 if name == "A" else 12
    want = [plain.greedy_generate(cfg, w, p, n_new) for p in prompts]
    llm = LLM(folders[name], dtype="float32", max_cache_tokens=1024, max_prefill_tokens=13,
              kv_page_size=8 if name == "A" else 16)
    assert llm.generate(prompts, max_tokens=n_new) == want
    assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages
    # the same requests one at a time give the same tokens (batching does not change results)
    assert [llm.generate([p], max_tokens=n_new)[0] for p in prompts] == want


def test_bf16_greedy_follows_plain_where_the_margin_is_clear(folders):
    from openinfer_b200 import LLM
    cfg, w = plain.read_model_folder(folders["B"])
    rng = random.Random(4)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (9, 33)]
    got = LLM(folders["B"], dtype="bfloat16", max_cache_tokens=512).generate(prompts, max_tokens=6)
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = oracle_logits(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 0.05 * float(logits.abs().max()):
                assert tok == int(logits.argmax())
            seq.append(tok)


def test_sampled_generation_is_reproducible_and_seed_dependent(folders):
    from openinfer_b200 import LLM, SamplingParams
    llm = LLM(folders["B"], dtype="bfloat16", max_cache_tokens=1024, max_prefill_tokens=13)
    rng = random.Random(8)
    prompts = [random_tokens(rng, n, 384) for n in (1, 9, 33, 70)]
    sp = SamplingParams(temperature=0.8, seed=1234)
    a = llm.generate(prompts, sp, max_tokens=12)
    b = llm.generate(prompts, sp, max_tokens=12)
    assert a == b and all(len(x) == 12 for x in a)
    # a seeded request's tokens do not depend on what else is in the batch
    assert llm.generate([prompts[2]], sp, max_tokens=12)[0] == a[2]
    c = llm.generate(prompts, SamplingParams(temperature=0.8, seed=99), max_tokens=12)
    assert c != a
    # top_k = 1 and a tiny top_p collapse to greedy (pegainfer-qwen3/tests/sampling_behavior.rs:1-15)
    g = llm.generate(prompts, max_tokens=6)
    assert llm.generate(prompts, SamplingParams(temperature=1.0, top_k=1), max_tokens=6) == g
    assert llm.generate(prompts, SamplingParams(temperature=1.0, top_p=1e-6, seed=5), max_tokens=6) == g
    # temperature gives diversity across seeds
    outs = {tuple(llm.generate([prompts[1]], SamplingParams(temperature=1.5, seed=s), max_tokens=8)[0]) for s in range(6)}
    assert len(outs) > 1


def test_stop_tokens_and_rejection(folders, tmp_path):
    from openinfer_b200 import LLM
    import shutil
    f = str(tmp_path / "m")
    shutil.copytree(folders["A"], f)
    cfg, w = plain.read_model_folder(f)
    prompt = [3, 1, 4, 1, 5]
    free = plain.greedy_generate(cfg, w, prompt, 8)
    stop = free[3]
    first = free.index(stop)
    raw = json.load(open(os.path.join(f, "config.json")))
    raw["eos_token_id"] = stop
    json.dump(raw, open(os.path.join(f, "config.json"), "w"))
    llm = LLM(f, dtype="float32", max_cache_tokens=512)
    res = llm.generate_detailed([prompt, list(range(600))], max_tokens=8)
    assert res[0].token_ids == free[:first] and res[0].finish_reason == "stop"   # the stop token is not emitted
    assert res[1].finish_reason == "rejected:context_length" and res[1].token_ids == []


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_step_ahead_gives_the_tokens_of_waiting_for_every_step(folders, dtype):
    """The engine launches step n + 1 before it has read step n's tokens (they are fed on the device);
    the generated ids are those of the loop that waits, stop tokens, ends by length and prompts cut
    into portions beside decoding included, and every page comes back."""
    from openinfer_b200 import LLM
    cfg, _ = plain.read_model_folder(folders["B"])
    rng = random.Random(5)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (1, 9, 33, 70, 4)]
    max_tokens = [12, 1, 7, 20, 16]
    outs = []
    for ahead in (False, True):
        llm = LLM(folders["B"], dtype=dtype, max_cache_tokens=1024, max_prefill_tokens=13, lookahead=ahead)
        assert llm.scheduler.lookahead == ahead
        free = llm.generate(prompts, max_tokens=max_tokens)
        # make some token that the longest request draws in mid-course a stop token
        llm.scheduler.stop_token_ids = {free[3][9]}
        res = llm.generate_detailed(prompts, max_tokens=max_tokens)
        outs.append((free, [(r.token_ids, r.finish_reason) for r in res]))
        assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages and not llm.has_work()
    assert outs[0] == outs[1]
    assert outs[1][1][3][1] == "stop" and len(outs[1][1][3][0]) <= 9


def test_command_line(folders):
    cfg, w = plain.read_model_folder(folders["A"])
    want = plain.greedy_generate(cfg, w, [7, 8, 9], 5)
    out = subprocess.run([sys.executable, "-m", "openinfer_b200", "--model-path", folders["A"], "--dtype", "float32",
                          "--prompt-ids", "7,8,9", "--max-tokens", "5", "--num-pages", "32", "--kv-page-size", "8"],
                         cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["token_ids"] == want and line["finish_reason"] == "length"


def test_memory_budget_sizes_the_pool(folders):
    from openinfer_b200 import LLM
    llm = LLM(folders["A"], dtype="bfloat16", gpu_memory_utilization=0.05)
    assert llm.runner.cache.num_pages > 100
    assert len(llm.generate([[1, 2, 3]], max_tokens=4)[0]) == 4


def test_no_cpu_path(folders):
    from openinfer_b200.engine.runner import ModelRunner
    from openinfer_b200.kernels import KernelError
    with pytest.raises(KernelError, match="no CPU path"):
        ModelRunner.from_folder(folders["A"], device="cpu", max_tokens=64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_cache_gives_the_same_tokens_and_is_used(folders, dtype):
    """Requests whose prompts share a front reuse its pages (registered when the first of them was computed);
    the generated ids are those of an engine without the prefix cache, and every page comes back."""
    from openinfer_b200 import LLM
    cfg, _ = plain.read_model_folder(folders["B"])
    rng = random.Random(9)
    stem = random_tokens(rng, 50, cfg["vocab_size"])
    prompts = [stem + random_tokens(rng, n, cfg["vocab_size"]) for n in (1, 7, 20)] + [stem[:33], stem, random_tokens(rng, 9, cfg["vocab_size"])]
    outs = []
    for on in (False, True):
        llm = LLM(folders["B"], dtype=dtype, max_cache_tokens=2048, max_prefill_tokens=24, kv_page_size=16, prefix_cache=on)
        first = llm.generate(prompts[:1], max_tokens=6)            # computes and registers the stem's three full pages
        rest = llm.generate(prompts[1:], max_tokens=6)             # five more requests at once
        again = llm.generate(prompts[:1], max_tokens=6)
        outs.append((first, rest, again))
        hits = llm.runner.cache.prefix_hits
        # stem + n shares 48 tokens; stem[:33] 32; stem itself 48; the unrelated prompt none; the repeat 48
        assert hits == ((48 + 48 + 32 + 48 + 0 + 48) if on else 0), hits
        assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages and not llm.has_work()
        llm.runner.cache.check()
    if dtype == "float32":
        assert outs[0] == outs[1]
    else:
        same = sum(a == b for a, b in zip(sum(outs[0], []), sum(outs[1], [])))
        assert same >= len(sum(outs[0], [])) - 1       # bfloat16: a near-tie may fall the other way
    assert outs[1][0] == outs[1][2]


@pytest.mark.parametrize("lookahead", [True, False])
def test_logprobs_and_echo(folders, lookahead):
    """The request options `logprobs` and `echo` of the reference: each generated token with its log-probability
    and the k most likely tokens, and with echo the same for the prompt's tokens, portions and decoding mixed."""
    from openinfer_b200 import LLM
    cfg, w = plain.read_model_folder(folders["A"])
    rng = random.Random(3)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (9, 30, 4)]
    llm = LLM(folders["A"], dtype="float32", max_cache_tokens=1024, max_prefill_tokens=7, kv_page_size=8, lookahead=lookahead)
    res = llm.generate_detailed(prompts, max_tokens=5, logprobs=3, echo=True)
    plain_tokens = llm.generate(prompts, max_tokens=5)
    for p, r, toks in zip(prompts, res, plain_tokens):
        assert r.token_ids == toks and r.finish_reason == "length"
        full = torch.log_softmax(oracle_logits(cfg, w, p + r.token_ids).double(), dim=-1)
        assert len(r.logprobs) == 5 and len(r.prompt_logprobs) == len(p) and r.prompt_logprobs[0] is None
        for t in range(1, len(p)):          # the prompt: token t under the distribution after t - 1
            e = r.prompt_logprobs[t]
            assert abs(e.logprob - float(full[t - 1, p[t]])) < 1e-3
            assert [i for i, _ in e.top_logprobs] == torch.topk(full[t - 1], 3).indices.tolist()
        for j, e in enumerate(r.logprobs):  # generated token j under the distribution after what precedes it
            at = len(p) - 1 + j
            assert abs(e.logprob - float(full[at, r.token_ids[j]])) < 1e-3
            assert e.top_logprobs[0][0] == r.token_ids[j]        # greedy: the drawn token is the most likely one
            assert all(abs(v - float(full[at, i])) < 1e-3 for i, v in e.top_logprobs)
    # without echo only the generated tokens carry log-probabilities; without logprobs nothing does
    r = llm.generate_detailed(prompts[:1], max_tokens=3, logprobs=2)[0]
    assert r.prompt_logprobs is None and len(r.logprobs) == 3 and len(r.logprobs[0].top_logprobs) == 2
    r = llm.generate_detailed(prompts[:1], max_tokens=3)[0]
    assert r.logprobs is None and r.prompt_logprobs is None
    assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages


@pytest.mark.parametrize("lookahead", [True, False])
def test_many_requests_arriving_over_time_with_few_pages(folders, lookahead):
    """Thirty requests of random lengths (some sharing a front, so the prefix cache lends pages) arrive while
    others run, in a pool that holds about five of them: requests wait for pages, pages are used again many
    times, prompts are cut into portions beside decoded tokens. In float32 every request gets the tokens it
    gets alone in a fresh engine, a third of them are also checked against the plain implementation, and
    in the end every page is back."""
    from openinfer_b200 import LLM
    cfg, w = plain.read_model_folder(folders["B"])
    rng = random.Random(31 + int(lookahead))
    stem = random_tokens(rng, 40, cfg["vocab_size"])
    reqs = []
    for i in range(30):
        body = random_tokens(rng, rng.choice([1, 2, 5, 17, 30, 63, 90]), cfg["vocab_size"])
        prompt = (stem[: rng.choice([16, 32, 40])] + body) if i % 3 == 0 else body
        reqs.append((prompt, rng.randint(1, 20)))
    llm = LLM(folders["B"], dtype="float32", max_cache_tokens=640, max_prefill_tokens=24, max_decode_batch=6,
              kv_page_size=16, lookahead=lookahead, prefix_cache=True)
    got = {}
    reasons = {}
    ids = []
    waiting = list(reqs)
    steps = 0
    while waiting or llm.has_work():
        for _ in range(rng.randint(0, 3)):          # zero to three arrivals before every step
            if waiting:
                prompt, n_new = waiting.pop(0)
                ids.append(llm.submit(prompt, max_tokens=n_new))
        for ev in llm.step():
            assert ev.kind in ("token", "finished"), (ev.kind, ev.reason)
            if ev.kind == "token":
                got.setdefault(ev.request_id, []).append(ev.token)
            else:
                reasons[ev.request_id] = ev.reason
        steps += 1
        assert steps < 5000
    assert len(ids) == 30 and set(reasons) == set(ids)
    cache = llm.runner.cache
    cache.check()
    assert cache.min_free_pages() == cache.num_pages
    assert cache.prefix_hits > 0
    solo = LLM(folders["B"], dtype="float32", max_cache_tokens=640, prefix_cache=False, runner=None)
    for k, (rid, (prompt, n_new)) in enumerate(zip(ids, reqs)):
        assert len(got[rid]) == n_new and reasons[rid] == "length"
        assert got[rid] == solo.generate([prompt], max_tokens=n_new)[0], f"request {k}"
        if k % 3 == 1:
            assert got[rid] == plain.greedy_generate(cfg, w, prompt, n_new), f"request {k} against the plain implementation"


def _splitmix(seed: int, step: int) -> int:
    """SplitMix64 over (seed, step), restated from pegainfer-sample/src/lib.rs:283-288."""
    m = (1 << 64) - 1
    z = (seed ^ ((step * 0x9E3779B97F4A7C15) & m)) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def _uniform(seed: int, step: int) -> float:
    return (_splitmix(seed, step) >> 40) / float(1 << 24)     # the top 24 bits: exact in float32


@pytest.mark.parametrize("ahead", [False, True])
def test_sampled_tokens_are_the_plain_draws(folders, ahead):
    """Configuration B's workload: prompts of 1/9/33/70 tokens in portions of 13 beside decoding, 12 tokens at
    temperature 0.8 (one request also with top-k and top-p), seeded and unseeded requests mixed, in float32.
    Every token must be the plain implementation's inverse-CDF pick from the plain distribution at the uniform
    number that belongs to the draw: SplitMix64(the request's seed, its own count of tokens so far) for a seeded
    request; for an unseeded one SplitMix64(SplitMix64(the step's seed, its row among the rows the step hands to
    the sampler), its own count), the step's seed being the next 64 bits of Random(engine seed). A draw whose uniform
    number lies within 1e-4 of an edge of the cumulative distribution is not checked. A fifth request is greedy and
    runs in the same steps: its rows keep the argmax while the others' are drawn."""
    from openinfer_b200 import LLM, SamplingParams
    cfg, w = plain.read_model_folder(folders["B"])
    rng = random.Random(8)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (1, 9, 33, 70, 20)]
    params = [SamplingParams(temperature=0.8, seed=1234), SamplingParams(temperature=0.8),
              SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=77), SamplingParams(temperature=0.8),
              SamplingParams()]      # and a greedy request in the same steps: its rows keep the argmax
    n_new = 12
    engine_seed = 4242
    llm = LLM(folders["B"], dtype="float32", max_cache_tokens=1024, max_prefill_tokens=13, lookahead=ahead,
              engine_seed=engine_seed)
    # which rows each step samples, in the order the executor hands them to the sampler: the requests whose
    # prompt ends in the step, then the decoding ones (recorded from the scheduler's calls, nothing else)
    batches = []
    inner = llm.executor.launch

    def launch(prefill, decode, step_seed, previous=None):
        batches.append((step_seed, [p.request_id for p in prefill if p.is_last] + [d.request_id for d in decode]))
        return inner(prefill, decode, step_seed, previous)

    llm.executor.launch = launch
    got = llm.generate(prompts, params, max_tokens=n_new)
    seeds = random.Random(engine_seed)
    drawn = {i: 0 for i in range(5)}
    where = {}                           # (request, its k-th token) -> (step seed, row)
    for step_seed, rows in batches:
        assert step_seed == seeds.getrandbits(64)
        for row, rid in enumerate(rows):
            where[(rid, drawn[rid])] = (step_seed, row)
            drawn[rid] += 1
    ids = sorted(drawn)
    checked = 0
    for i, rid in enumerate(ids):
        assert len(got[i]) == n_new
        sp, seq = params[i], list(prompts[i])
        for k, tok in enumerate(got[i]):
            logits = oracle_logits(cfg, w, seq)[-1]
            if sp.temperature == 0:
                top = torch.topk(logits, 2).values
                if float(top[0] - top[1]) > 1e-4:
                    assert tok == int(logits.argmax()), f"request {i}, token {k}: not the argmax"
                    checked += 1
                seq.append(tok)
                continue
            dist = plain.sampling_distribution(logits, sp.temperature, sp.top_k, sp.top_p, sp.min_p)
            if sp.seed is not None:
                u = _uniform(sp.seed, k)
            else:
                step_seed, row = where[(rid, k)]
                u = _uniform(_splitmix(step_seed, row), k)
            edges = torch.cumsum(dist, 0)
            if float((edges - u).abs().min()) > 1e-4:
                assert tok == plain.inverse_cdf_pick(dist, u), f"request {i}, token {k}: not the plain draw"
                checked += 1
            seq.append(tok)
    assert checked >= 50


@pytest.mark.parametrize("ahead", [False, True])
def test_cancel_leaves_the_others_alone_and_frees_its_pages(folders, ahead):
    """Requests are taken back in the middle of a prompt that is computed in portions and in the middle of
    decoding (one step ahead: with a row in flight): nothing more of them is reported, the other requests' tokens
    are what they are without any cancelling, and every page and state slot is back at the end."""
    from openinfer_b200 import LLM
    cfg, w = plain.read_model_folder(folders["B"])
    rng = random.Random(21)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (9, 70, 33, 5, 60)]
    keep = [0, 2, 3]
    want = {i: plain.greedy_generate(cfg, w, prompts[i], 10) for i in keep}
    llm = LLM(folders["B"], dtype="float32", max_cache_tokens=1024, max_prefill_tokens=13, lookahead=ahead)
    ids = [llm.submit(p, max_tokens=10) for p in prompts]
    tokens = {rid: [] for rid in ids}
    finished = {}
    cancelled_at = {}

    def take(events):
        for ev in events:
            assert ev.request_id not in cancelled_at, f"request {ev.request_id} reported {ev.kind} after it was cancelled"
            if ev.kind == "token":
                tokens[ev.request_id].append(ev.token)
            elif ev.kind == "finished":
                finished[ev.request_id] = ev.reason
            else:
                raise AssertionError(f"unexpected event {ev}")

    steps = 0
    while llm.has_work():
        take(llm.step())
        steps += 1
        # request 1 (70 tokens, portions of 13): taken back while its prompt is half computed
        if ids[1] not in cancelled_at and any(p.req.request_id == ids[1] and p.done >= 13 for p in llm.scheduler.prefilling):
            assert llm.cancel(ids[1])
            cancelled_at[ids[1]] = steps
        # request 4: taken back after its third token
        if ids[4] not in cancelled_at and len(tokens[ids[4]]) >= 3:
            assert llm.cancel(ids[4])
            cancelled_at[ids[4]] = steps
            assert not llm.cancel(ids[4])
        assert steps < 500
    assert set(cancelled_at) == {ids[1], ids[4]} and tokens[ids[1]] == [] and 3 <= len(tokens[ids[4]]) <= 4
    for i in keep:
        assert tokens[ids[i]] == want[i] and finished[ids[i]] == "length"
    cache = llm.runner.cache
    cache.check()
    assert cache.min_free_pages() == cache.num_pages and cache.slot_pool.used_count == 0
