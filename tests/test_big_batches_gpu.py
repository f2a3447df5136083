"""Steps with many live requests against the plain implementation: decode batches of 9 to 100 rows at
unequal lengths (every batch bucket of the recorded graphs, the padded 17-32-row products, the path of
33 and more rows, decode attention in one and in two waves, key slices that shrink with the batch) and
mixed steps of 8 prompt portions beside 56 decoded tokens, with so few pages that they are used again;
then the same scale through the scheduler, one step ahead."""
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import (TINY_C, TINY_E, TINY_F, assert_close, count_page_handouts, make_model_folder,
                     random_tokens, oracle_logits)

pytestmark = pytest.mark.gpu

CONFIGS = {"C": (TINY_C, 2), "E": (TINY_E, 4), "F": (TINY_F, 5)}
PAGE = 16
DECODE_SIZES = [9, 17, 32, 33, 64, 100]      # graph buckets 16, 32, 32, 64, 64, 128
N_FIRST = 100                                 # requests of the first wave
N_KEEP = 56                                   # of them decode on beside the second wave's portions
SECOND = [150, 71, 129, 200, 64, 97, 256, 33]  # prompts of the 8 requests of the second wave


def _plan(vocab, seed):
    """Every request's whole token sequence (prompt + the tokens later fed one by one) and the steps."""
    rng = random.Random(seed)
    prompt_len = {f"a{r}": (300 if r == 0 else 3 + (r * 7) % 61) for r in range(N_FIRST)}
    decodes = {f"a{r}": sum(1 for n in DECODE_SIZES if r < n) + (2 if r < N_KEEP else 0) for r in range(N_FIRST)}
    for i, n in enumerate(SECOND):
        prompt_len[f"b{i}"], decodes[f"b{i}"] = n, 0
    seqs = {rid: random_tokens(rng, prompt_len[rid] + decodes[rid], vocab) for rid in prompt_len}
    fed = {rid: 0 for rid in seqs}
    steps = []

    def entry(rid, n, want_all=False):
        toks = seqs[rid][fed[rid]: fed[rid] + n]
        assert len(toks) == n
        fed[rid] += n
        return {"id": rid, "tokens": toks, "want": list(range(n)) if want_all else [n - 1]}

    first = [f"a{r}" for r in range(N_FIRST)]
    for at in range(0, N_FIRST, 20):          # whole prompts, 20 requests a step
        steps.append({"entries": [entry(rid, prompt_len[rid]) for rid in first[at: at + 20]], "end": []})
    for n in DECODE_SIZES:                    # single tokens of the first n requests
        steps.append({"entries": [entry(rid, 1) for rid in first[:n]], "end": []})
    steps[-1]["end"] = first[N_KEEP:]         # 44 requests end: their pages go to the second wave
    second = [f"b{i}" for i in range(len(SECOND))]
    halves = {rid: prompt_len[rid] // 2 for rid in second}
    for part in range(2):                     # 8 portions beside 56 decoded tokens, twice
        entries = [entry(rid, 1) for rid in first[:N_KEEP]]
        for rid in second:
            n = halves[rid] if part == 0 else prompt_len[rid] - halves[rid]
            entries.append(entry(rid, n, want_all=True))
        rng.shuffle(entries)
        steps.append({"entries": entries, "end": []})
    steps[-1]["end"] = first[:N_KEEP] + second
    assert all(fed[rid] == len(seqs[rid]) for rid in seqs)
    # the fewest pages with which this runs: the larger of the two waves' needs
    pages = lambda rid: -(-len(seqs[rid]) // PAGE)
    need1 = sum(pages(rid) for rid in first)
    need2 = sum(pages(rid) for rid in first[:N_KEEP]) + sum(pages(rid) for rid in second)
    return seqs, steps, max(need1, need2), need1, need2


@pytest.fixture(scope="module")
def workloads(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in CONFIGS.items():
        folder = make_model_folder(str(tmp_path_factory.mktemp(f"big{name}")), cfg, seed)
        pcfg, w = plain.read_model_folder(folder)
        seqs, steps, num_pages, need1, need2 = _plan(cfg["vocab_size"], 40 + seed)
        ref = {rid: oracle_logits(pcfg, w, toks) for rid, toks in seqs.items()}
        out[name] = (folder, pcfg, w, seqs, steps, num_pages, ref)
    return out


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E", "F"])
def test_large_decode_batches_and_mixed_steps_match_plain(workloads, name, dtype, graphs):
    from openinfer_b200.engine.runner import ModelRunner, StepEntry
    from openinfer_b200.kernels import attention as A, gemm_tcgen05 as G, linear as LN
    folder, _, _, seqs, steps, num_pages, ref = workloads[name]
    runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=PAGE, num_pages=num_pages,
                                     max_requests=128)
    runner.cuda_graph = graphs
    handed_out = count_page_handouts(runner.cache)
    at = {rid: 0 for rid in seqs}
    for i, st in enumerate(steps):
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]])
        row = 0
        for e in st["entries"]:
            n = len(e["tokens"])
            pos = [at[e["id"]] + w for w in e["want"]]
            assert_close(logits[row: row + len(pos)], ref[e["id"]][pos], dtype,
                         f"{name}/{dtype}/step {i} ({len(st['entries'])} requests) request {e['id']}")
            row += len(pos)
            at[e["id"]] += n
        for rid in st["end"]:
            runner.end(rid)
    runner.cache.check()
    assert runner.cache.min_free_pages() == runner.cache.num_pages, "pages were not all given back"
    assert max(handed_out.values()) >= 2, "no page was used again"
    if graphs:
        assert {k[0] for k in runner._graphs} == {16, 32, 64, 128}, f"graph buckets {sorted(runner._graphs)}"
    assert A.tcgen05_status() == 0 and G.status() == 0 and LN.stream_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["E", "F"])
def test_a_hundred_requests_through_the_scheduler_one_step_ahead(workloads, name, dtype):
    """100 requests through LLM.generate with one step ahead and recorded graphs for the decode-only steps:
    prompts cut by a budget of 256 tokens ride beside up to 100 decoding requests, the pool holds about
    two thirds of what all requests need, so requests wait and pages are used again. float32: the tokens of the
    plain implementation; bfloat16: its token wherever its two best logits are clearly apart."""
    from openinfer_b200 import LLM
    folder, pcfg, w, _, _, _, _ = workloads[name]
    rng = random.Random(9)
    lens = [2 + (r * 13) % 90 for r in range(100)]
    lens[7], lens[50] = 400, 300
    prompts = [random_tokens(rng, n, pcfg["vocab_size"]) for n in lens]
    new = 5
    need = sum(-(-(n + new) // PAGE) for n in lens)
    llm = LLM(folder, dtype=dtype, kv_page_size=PAGE, num_pages=(2 * need) // 3, max_prefill_tokens=256,
              max_decode_batch=128, lookahead=True, cuda_graph=True, prefix_cache=False)
    handed_out = count_page_handouts(llm.runner.cache)
    got = llm.generate(prompts, max_tokens=new)
    assert llm.runner._graphs, "no decode step went through a graph"
    assert max(handed_out.values()) >= 2, "no page was used again"
    assert llm.runner.cache.min_free_pages() == llm.runner.cache.num_pages
    for p, g in zip(prompts, got):
        assert len(g) == new
        seq = list(p)
        for tok in g:
            logits = oracle_logits(pcfg, w, seq)[-1]
            if dtype == "float32":
                assert tok == int(logits.argmax()), f"prompt of {len(p)} tokens: token {len(seq) - len(p)} differs"
            else:
                top2 = torch.topk(logits, 2).values
                if float(top2[0] - top2[1]) > 0.05 * float(logits.abs().max()):
                    assert tok == int(logits.argmax())
            seq.append(tok)
