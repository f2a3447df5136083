"""The engine against the plain implementation under every way of cutting the work,
in float32 and in bfloat16, for both tiny configurations."""
import os
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import (TINY, assert_close, count_page_handouts, make_model_folder, random_tokens, replay_in_process,
                     replay_trace_run, round64, trace_mixed, trace_portions, trace_tail, trace_whole, oracle_logits)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 47, 130, 200, 77, 33], "B": [1, 9, 70, 150, 261, 40], "C": [3, 64, 129, 300, 65], "D": [2, 100, 257, 33],
           "E": [400, 130, 1, 260, 17]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in TINY.items():
        out[name] = make_model_folder(str(tmp_path_factory.mktemp(f"tiny{name}")), cfg, seed)
    return out


@pytest.fixture(scope="module")
def workloads(folders):
    """Per config: the requests and the plain implementation's logits at every position."""
    out = {}
    for name, folder in folders.items():
        cfg, w = plain.read_model_folder(folder)
        rng = random.Random(100 + len(name))
        reqs = {f"r{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate(LENGTHS[name])}
        ref = {rid: oracle_logits(cfg, w, toks) for rid, toks in reqs.items()}
        out[name] = (cfg, reqs, ref)
    return out


def _runner(folder, dtype, max_tokens, page_size=16, cuda_graph=False):
    from openinfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=page_size,
                                max_tokens=max_tokens, max_requests=8)
    r.cuda_graph = cuda_graph
    return r


def _check(got, ref, dtype, what):
    assert set(got) == set(ref)
    for rid in ref:
        assert_close(got[rid], ref[rid], dtype, f"{what} request {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cuttings_match_plain(folders, workloads, name, dtype, mode):
    cfg, reqs, ref = workloads[name]
    biggest = max(round64(len(t)) for t in reqs.values())
    if mode == "whole":
        steps, max_tokens = trace_whole(reqs), biggest
    elif mode == "tail":
        steps, max_tokens = trace_tail(reqs), biggest
    elif mode == "portions":
        steps, max_tokens = trace_portions(reqs), biggest
    else:
        # room for the largest request plus two more blocks of 64: pages must be reused
        max_tokens = biggest + 128
        steps = trace_mixed(reqs, max_tokens, seed=7)
        assert max(len(s["entries"]) for s in steps) >= 2
    page = {"A": 8, "B": 16, "C": 16, "D": 32, "E": 16}[name]
    runner = _runner(folders[name], dtype, max_tokens, page_size=page)
    handed_out = count_page_handouts(runner.cache)
    got = replay_in_process(runner, steps)
    _check(got, ref, dtype, f"{name}/{dtype}/{mode}")
    runner.cache.check()
    if mode == "mixed":
        assert max(handed_out.values()) >= 2, "no page was used again: the pool is too large for this test"
    assert runner.cache.min_free_pages() == runner.cache.num_pages, "pages were not all given back"
    from openinfer_b200.kernels import attention as A, gemm_tcgen05 as G
    assert A.tcgen05_status() == 0 and G.status() == 0, "a bounded wait ran out in a tcgen05 kernel"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, workloads, tmp_path, dtype):
    """The bin/trace_run program itself, fed line by line, mixed trace with page reuse."""
    name = "B"
    cfg, reqs, ref = workloads[name]
    max_tokens = max(round64(len(t)) for t in reqs.values()) + 128
    steps = trace_mixed(reqs, max_tokens, seed=3)
    got = replay_trace_run(folders[name], dtype, steps, str(tmp_path / "out"), max_tokens, cfg["vocab_size"])
    _check(got, ref, dtype, f"trace_run/{dtype}")


def test_trace_run_writes_no_file_for_a_step_in_which_nothing_is_wanted(folders, tmp_path):
    """Steps may bring tokens whose logits nobody asks for (``want`` empty, or absent): the tokens still go through the
    model and into the cache, ``done`` is printed, and no file is written; later steps' logits are right."""
    name = "A"
    cfg, w = plain.read_model_folder(folders[name])
    rng = random.Random(9)
    a, b = random_tokens(rng, 9, cfg["vocab_size"]), random_tokens(rng, 5, cfg["vocab_size"])
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:6], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[6:7], "want": [0]}, {"id": "b", "tokens": b[:3], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[3:4], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[7:], "want": [1]}, {"id": "b", "tokens": b[4:], "want": [0]}], "end": ["a", "b"]},
    ]
    out = str(tmp_path / "out")
    got = replay_trace_run(folders[name], "float32", steps, out, 256, cfg["vocab_size"])   # asserts which files exist
    assert sorted(os.listdir(out)) == ["1.f32", "3.f32"]
    ra, rb = oracle_logits(cfg, w, a), oracle_logits(cfg, w, b)
    assert_close(got["a"], ra[[6, 8]], "float32", "request a")
    assert_close(got["b"], rb[[4]], "float32", "request b")


def test_first_tokens_and_long_decode(folders, workloads):
    """The first tokens of a sequence one by one from an empty cache, then a long decode."""
    name = "A"
    cfg, w = plain.read_model_folder(folders[name])
    rng = random.Random(5)
    toks = random_tokens(rng, 300, cfg["vocab_size"])
    ref = oracle_logits(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        runner = _runner(folders[name], dtype, round64(len(toks)), page_size=8)
        steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []}
                 for i, t in enumerate(toks)]
        steps[-1]["end"] = ["x"]
        got = replay_in_process(runner, steps)
        assert_close(got["x"], ref, dtype, f"token by token {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "D", "E"])
def test_decode_steps_replayed_as_cuda_graphs(folders, workloads, name, dtype):
    """Steps that bring one token per request run as recorded CUDA graphs (padded to a batch
    bucket, key slices fixed by the bucket); the logits must not notice."""
    cfg, reqs, ref = workloads[name]
    biggest = max(round64(len(t)) for t in reqs.values())
    for mode in ("tail", "mixed"):
        max_tokens = biggest if mode == "tail" else biggest + 192
        steps = trace_tail(reqs) if mode == "tail" else trace_mixed(reqs, max_tokens, seed=11)
        runner = _runner(folders[name], dtype, max_tokens, page_size=16, cuda_graph=True)
        got = replay_in_process(runner, steps)
        assert runner._graphs, "no step went through a graph"
        _check(got, ref, dtype, f"graphs {name}/{dtype}/{mode}")
        runner.cache.check()


def test_without_programmatic_dependent_launch(folders, workloads):
    """Every kernel is launched so that it may start under its predecessor and waits before touching
    what that one writes; with the attribute switched off (plain stream order) the logits are the same
    bit for bit, with and without recorded graphs."""
    from openinfer_b200.kernels import lib as klib
    name = "A"
    cfg, reqs, ref = workloads[name]
    biggest = max(round64(len(t)) for t in reqs.values())
    steps = trace_mixed(reqs, biggest + 192, seed=3)
    L = klib.load()
    outs = {}
    try:
        for pdl in (1, 0):
            for graphs in (False, True):
                klib.check(L.oi_set_pdl(pdl), "set_pdl")
                runner = _runner(folders[name], "bfloat16", biggest + 192, page_size=16, cuda_graph=graphs)
                outs[(pdl, graphs)] = replay_in_process(runner, steps)
    finally:
        klib.check(L.oi_set_pdl(1), "set_pdl")
    for graphs in (False, True):
        a, b = outs[(1, graphs)], outs[(0, graphs)]
        assert a.keys() == b.keys()
        for k in a:
            assert torch.equal(torch.as_tensor(a[k]), torch.as_tensor(b[k])), f"step {k} differs without the attribute (graphs {graphs})"
    _check(outs[(1, True)], ref, "bfloat16", "with dependent launches")


@pytest.mark.parametrize("name", ["C", "E"])
def test_batch_invariant_mode_is_bitwise(folders, workloads, name):
    """With the batch-invariant numeric policy a request's logits are the same BIT FOR BIT whether it runs
    alone or beside others (prompt portions of its own fixed size, then single tokens), in bfloat16, with
    recorded graphs for the decode steps; and they still agree with the plain implementation."""
    from openinfer_b200.engine.runner import StepEntry
    from openinfer_b200.kernels import policy
    cfg, reqs, ref = workloads[name]          # C: head 64 (mma.sync tiles); E: head 128 (tcgen05 tiles, fused gate/up)
    C = 16 if name == "C" else 96            # request-local portion size
    tail = 6                                 # tokens at the end of every request that are fed one by one
    reqs = {r: t for r, t in reqs.items() if len(t) > tail}
    ids = list(reqs)[:4]

    def schedule(group):
        """Steps for the requests of `group` running together: request-local portions, then single tokens."""
        at = {r: 0 for r in group}
        steps = []
        while any(at[r] < len(reqs[r]) for r in group):
            entries = []
            for r in group:
                n = len(reqs[r])
                if at[r] >= n:
                    continue
                take = min(C, n - tail - at[r]) if at[r] < n - tail else 1
                entries.append((r, reqs[r][at[r]: at[r] + take]))
                at[r] += take
            steps.append(entries)
        return steps

    def run(group):
        runner = _runner(folders[name], "bfloat16", sum(round64(len(reqs[r])) for r in group) + 64, page_size=16, cuda_graph=True)
        rows = {r: [] for r in group}
        for entries in schedule(group):
            logits = runner.step([StepEntry(r, toks, list(range(len(toks)))) for r, toks in entries])
            at = 0
            for r, toks in entries:
                rows[r].append(logits[at: at + len(toks)].float().cpu())
                at += len(toks)
        for r in group:
            runner.end(r)
        return {r: torch.cat(v) for r, v in rows.items()}

    policy.set_batch_invariant(True)
    try:
        together = run(ids)
        alone = {r: run([r])[r] for r in ids}
        pair = run(ids[1:3])
    finally:
        policy.set_batch_invariant(False)
    for r in ids:
        assert torch.equal(together[r], alone[r]), f"request {r}: logits differ between running alone and with three others"
    for r in ids[1:3]:
        assert torch.equal(pair[r], alone[r]), f"request {r}: logits differ in a batch of two"
    _check({r: together[r] for r in ids}, {r: ref[r] for r in ids}, "bfloat16", "batch-invariant policy")


def test_long_context_decode_rows_in_64_and_128_slices_through_the_engine(tmp_path):
    """Two requests with 13,000 and 25,000 tokens of context decode alone: such rows are cut into 64 and 128 key
    slices whose partial results a second kernel merges (recorded graphs and launched steps). The bfloat16 engine's
    logits are compared with the float32 engine's (its general attention kernel visits every key in order) on the
    same weights: whole prompts in portions of 4,096 tokens, then four tokens one by one. (The kernel itself is
    compared with float64 in test_kernels_gpu; the plain implementation cannot hold 25,000 x 25,000 scores.)"""
    from openinfer_b200.engine.runner import ModelRunner, StepEntry
    from openinfer_b200.kernels import attention as A
    cfg = dict(TINY["E"][0], max_position_embeddings=32768)
    folder = make_model_folder(str(tmp_path / "m"), cfg, 11)
    rng = random.Random(2)
    prompts = {"long": random_tokens(rng, 25000, cfg["vocab_size"]), "mid": random_tokens(rng, 13000, cfg["vocab_size"])}
    seen = []
    old = A.decode_splits

    def recording(*a, **k):
        ns = old(*a, **k)
        seen.append(ns)
        return ns

    outs, feed = {}, {}
    for dtype, graphs in (("float32", False), ("bfloat16", True), ("bfloat16", False)):
        runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=16, max_tokens=40000, max_requests=4)
        runner.cuda_graph = graphs
        rows = {r: [] for r in prompts}
        for r, p in prompts.items():
            for at in range(0, len(p), 4096):
                toks = p[at: at + 4096]
                logits = runner.step([StepEntry(r, toks, [len(toks) - 1])])
            rows[r].append(logits[0].float().cpu())
        A.decode_splits = recording
        try:
            for step in range(4):
                for r in prompts:                    # each alone: one row a step leaves SMs idle with 32 slices
                    if dtype == "float32":
                        feed[(step, r)] = int(rows[r][-1].argmax())
                    logits = runner.step([StepEntry(r, [feed[(step, r)]], [0])])
                    rows[r].append(logits[0].float().cpu())
        finally:
            A.decode_splits = old
        outs[(dtype, graphs)] = {r: torch.stack(v) for r, v in rows.items()}
        if graphs:
            assert runner._graphs, "the single-token steps did not go through a graph"
        del runner
        torch.cuda.empty_cache()
    assert 64 in seen and 128 in seen, seen
    for key in (("bfloat16", True), ("bfloat16", False)):
        for r in prompts:
            assert_close(outs[key][r], outs[("float32", False)][r], "bfloat16", f"long context, {r}, graphs {key[1]}")


def test_real_layer_sizes_and_vocabulary(tmp_path):
    """Qwen3-8B layer sizes (hidden 4096, 32/8 heads of 128, intermediate 12288) with the REAL vocabulary
    of 151,936 entries, two layers, random weights written to a folder: the bfloat16 engine (streaming
    products with clusters of 4 and 8, gate/up with the activation, decode attention with rotation and merge
    inside, recorded graphs) against the float32 engine on the same weights, prompts in portions and then
    tokens one by one, three requests; and the float32 engine against the plain implementation on the shortest
    request (43 positions: the plain implementation's head alone is 2.5 GB of float32 on the CPU)."""
    from openinfer_b200.engine.runner import ModelRunner, StepEntry
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
    folder = make_model_folder(str(tmp_path / "m"), cfg, 7)
    rng = random.Random(1)
    prompts = {r: [rng.randrange(151936) for _ in range(n)] for r, n in (("a", 150), ("b", 37), ("c", 260))}
    outs = {}
    feed = {}
    for dtype in ("float32", "bfloat16"):
        runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=16, max_tokens=1024, max_requests=8)
        runner.cuda_graph = dtype == "bfloat16"
        rows = {r: [] for r in prompts}
        # the prompts in two portions each, together; then 6 tokens one by one (the float32 run's argmax is fed to both)
        for part in range(2):
            entries = []
            for r, p in prompts.items():
                cut = len(p) // 2
                toks = p[:cut] if part == 0 else p[cut:]
                entries.append(StepEntry(r, toks, [len(toks) - 1]))
            logits = runner.step(entries)
            for i, r in enumerate(prompts):
                rows[r].append(logits[i].float().cpu())
        for step in range(6):
            if dtype == "float32":
                feed[step] = {r: int(rows[r][-1].argmax()) for r in prompts}
            logits = runner.step([StepEntry(r, [feed[step][r]], [0]) for r in prompts])
            for i, r in enumerate(prompts):
                rows[r].append(logits[i].float().cpu())
        outs[dtype] = {r: torch.stack(v) for r, v in rows.items()}
        if dtype == "bfloat16":
            assert runner._graphs, "the single-token steps did not go through a graph"
        del runner
        torch.cuda.empty_cache()
    _check(outs["bfloat16"], outs["float32"], "bfloat16", "real layer sizes")
    pcfg, w = plain.read_model_folder(folder, dtype=torch.float64)   # an oracle without rounding of its own
    p = prompts["b"]
    seq = p + [feed[s]["b"] for s in range(6)]
    at = [len(p) // 2 - 1, len(p) - 1] + list(range(len(p), len(p) + 6))
    ref = oracle_logits(pcfg, w, seq)[at]
    assert_close(outs["float32"]["b"], ref, "float32", "real layer sizes and vocabulary, float32 engine against plain")
    assert_close(outs["bfloat16"]["b"], ref, "bfloat16", "real layer sizes and vocabulary, bfloat16 engine against plain")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,nq,nkv,hidden", [(48, 4, 2, 80), (80, 6, 3, 144), (96, 2, 1, 176), (112, 5, 5, 208),
                                               (144, 3, 1, 96), (256, 2, 2, 112)])
def test_head_sizes_in_steps_of_16(tmp_path, dtype, hd, nq, nkv, hidden):
    """Head sizes that no tuned kernel covers (48 ... 256), with widths that are no power of two and groups of
    1, 2, 3: the engine takes them through its general kernels. Two requests, mixed with so few pages that they
    are used again, against the plain implementation."""
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=hidden,
               num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd, intermediate_size=hidden + 40,
               vocab_size=257, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=bool(hd % 32),
               max_position_embeddings=512)
    folder = make_model_folder(str(tmp_path / "m"), cfg, hd)
    pcfg, w = plain.read_model_folder(folder)
    rng = random.Random(hd)
    reqs = {f"r{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate((70, 45, 100))}
    ref = {rid: oracle_logits(pcfg, w, toks) for rid, toks in reqs.items()}
    max_tokens = 128 + 128
    steps = trace_mixed(reqs, max_tokens, seed=hd)
    runner = _runner(folder, dtype, max_tokens, page_size=16)
    _check(replay_in_process(runner, steps), ref, dtype, f"head {hd}/{dtype}")
    runner.cache.check()
    assert runner.cache.min_free_pages() == runner.cache.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "E"])
def test_native_step_and_part_by_part_step_give_the_same_bits(folders, workloads, name, dtype):
    """A model made of the package's own parts runs every layer of a step in one native call; with that switched
    off the parts are called one by one from Python (what a model with a registered part of its own does). Both
    launch the same kernels with the same arguments: the logits are equal bit for bit, mixed steps and recorded
    decode steps included. The native step's optional variant without norm kernels in decode-sized steps (the
    products add the residual and scale by the reciprocal root mean square themselves) rounds the residual sum
    once where the norm kernel's input was rounded before: it is compared with the plain implementation."""
    from openinfer_b200.kernels import lib as klib, native
    cfg, reqs, ref = workloads[name]
    max_tokens = max(round64(len(t)) for t in reqs.values()) + 192
    steps = trace_mixed(reqs, max_tokens, seed=13)
    outs = {}
    L = klib.load()
    try:
        for mode in ("native_fused_norms", "native", "parts"):
            klib.check(L.oi_configure(native.OPT_FUSE_NORM, 1 if mode == "native_fused_norms" else 0), "configure")
            runner = _runner(folders[name], dtype, max_tokens, page_size=16, cuda_graph=True)
            runner.model.native_step = mode != "parts"
            outs[mode] = replay_in_process(runner, steps)
            assert (runner.model._native is not None) == (mode != "parts")
    finally:
        klib.check(L.oi_configure(native.OPT_FUSE_NORM, 0), "configure")
    for rid in ref:
        assert torch.equal(outs["native"][rid], outs["parts"][rid]), f"request {rid}: the two step paths differ"
    _check(outs["native_fused_norms"], ref, dtype, f"native step without norm kernels {name}/{dtype}")
    _check(outs["parts"], ref, dtype, f"part by part {name}/{dtype}")


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_bfloat16_engine_against_the_twin_with_the_reference_rounding(folders, workloads, name):
    """The engine rounds once per kernel output where the reference rounds more often (tests/plain_qwen3_bf16.py
    restates where). Against the float32 plain implementation the engine's bfloat16 logits are at least about as
    exact as that scheme of rounding would be (mean error at most 1.25 times the twin's), and the two bfloat16
    computations agree with each other within the bfloat16 tolerance."""
    import plain_qwen3_bf16 as twin
    cfg, reqs, ref = workloads[name]
    pcfg, w = plain.read_model_folder(folders[name])
    rid = max(reqs, key=lambda r: len(reqs[r]))
    toks = reqs[rid]
    runner = _runner(folders[name], "bfloat16", round64(len(toks)), page_size=16)
    got = replay_in_process(runner, trace_whole({rid: toks}))[rid]
    tw = twin.forward_logits(pcfg, w, toks)
    scale = ref[rid].abs().max().item()
    err_engine = (got - ref[rid]).abs().mean().item() / scale
    err_twin = (tw - ref[rid]).abs().mean().item() / scale
    assert err_engine <= 1.25 * err_twin, f"engine {err_engine:.5f} against the reference's rounding {err_twin:.5f}"
    assert_close(got, tw, "bfloat16", f"engine against the bfloat16 twin, {name}")
