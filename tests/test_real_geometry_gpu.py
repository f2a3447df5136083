"""The real layer geometries of the three benchmarked sizes against the plain implementation.

Hidden size, head counts, head size and intermediate size are those of Qwen3-8B, Qwen3-0.6B and
Qwen3-32B; the depth is 2 layers and the vocabulary is cut to 3,001 entries, because this is a
correctness test, not a benchmark: the plain implementation runs on the CPU, here in float64 (sums of
4,096 to 25,600 float32 terms differ between two correct orders of summation by about as much as the
float32 tolerance allows, so the oracle's own rounding is taken out of the comparison). Mixed steps with up to
twelve live requests, nine and more of them decoding at once, so few pages that they are used again,
decode-only steps replayed as recorded graphs, in float32 and in bfloat16."""
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close, count_page_handouts, make_model_folder, random_tokens, replay_in_process, trace_mixed, oracle_logits

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, head_dim=128, vocab_size=3001,
            rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=4096)
GEOMETRY = {
    "8b": dict(BASE, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               tie_word_embeddings=False),
    "0.6b": dict(BASE, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072,
                 tie_word_embeddings=True),
    "32b": dict(BASE, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                tie_word_embeddings=False),
}
LENGTHS = [90, 24, 61, 33, 128, 47, 70, 25, 52, 38, 101, 29, 44, 66]


@pytest.fixture(scope="module", params=list(GEOMETRY))
def workload(request, tmp_path_factory):
    name = request.param
    folder = make_model_folder(str(tmp_path_factory.mktemp(f"geo{name}")), GEOMETRY[name], seed=len(name))
    cfg, w = plain.read_model_folder(folder, dtype=torch.float64)
    rng = random.Random(17)
    reqs = {f"r{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate(LENGTHS)}
    ref = {rid: oracle_logits(cfg, w, toks) for rid, toks in reqs.items()}
    del w
    return name, folder, reqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_geometry_mixed_steps_match_plain(workload, dtype):
    from openinfer_b200.engine.runner import ModelRunner
    from openinfer_b200.kernels import attention as A, gemm_tcgen05 as G, linear as LN
    name, folder, reqs, ref = workload
    max_tokens = 1024                    # never room for all fourteen requests (1,216): pages are used again
    steps = trace_mixed(reqs, max_tokens, seed=1, max_live=12, tail=10)
    assert max(sum(1 for e in s["entries"] if len(e["tokens"]) == 1) for s in steps) >= 9
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), "no mixed step"
    runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", page_size=16, max_tokens=max_tokens,
                                     max_requests=16)
    runner.cuda_graph = True
    handed_out = count_page_handouts(runner.cache)
    got = replay_in_process(runner, steps)
    for rid in ref:
        assert_close(got[rid], ref[rid], dtype, f"{name} geometry/{dtype} request {rid}")
    runner.cache.check()
    assert runner.cache.min_free_pages() == runner.cache.num_pages
    assert max(handed_out.values()) >= 2, "no page was used again"
    assert runner._graphs, "no decode-only step went through a graph"
    assert A.tcgen05_status() == 0 and G.status() == 0 and LN.stream_status() == 0
