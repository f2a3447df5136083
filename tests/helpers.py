"""Shared by the tests: the tiny configurations, model folders, trace builders, comparisons."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Qwen3 configurations that differ in every size and option.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=512)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
    intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=768)
# Two more whose head sizes the tensor-core attention kernel covers (groups of 4 and 3).
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=192, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
    intermediate_size=320, vocab_size=500, rope_theta=500000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=1024)
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=160, num_attention_heads=3, num_key_value_heads=1, head_dim=128,
    intermediate_size=272, vocab_size=300, rope_theta=10000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=1024)
# Real head geometry at reduced depth and vocabulary: head 128 with a group of 2, an intermediate size
# that is a multiple of 128: the shapes the tcgen05 kernels (products, fused gate/up, prompt attention),
# the streaming decode products and the split decode attention take in the engine.
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=512, num_attention_heads=8, num_key_value_heads=4, head_dim=128,
    intermediate_size=1536, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=2048)
# The shape relations of the smallest real model (head 128, a group of 2, queries twice as wide as the
# hidden state) at toy width.
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
    intermediate_size=768, vocab_size=700, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=2048)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4)}

# Stated tolerances (never widened to make a cutting pass; every cutting uses the same).
#  float32: both sides sum in float32 in different orders; logits are O(1).
F32_ATOL, F32_RTOL = 1e-5, 5e-5       # measured: up to 4e-6 absolute on logits up to 2.4
#  bfloat16: activations are rounded to 8 bits of mantissa between kernels; the bound is
#  relative to the largest logit of the reference.
BF16_MAX_REL = 0.02          # measured on the five tiny configurations: 0.2 % to 0.8 %
BF16_MEAN_REL = 0.003        # measured: 0.04 % to 0.13 %


def make_model_folder(path: str, cfg: dict, seed: int) -> str:
    from openinfer_b200.config.base import resolve_architecture
    from openinfer_b200.weights import write_random_model

    config = resolve_architecture(cfg).config_cls.from_dict(cfg)
    write_random_model(config, path, seed)
    return path


def random_tokens(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


_ORACLE_F64 = {}
ORACLE_SELF_TOL = 8e-6    # float32 against float64 evaluation of the plain implementation: 2.5e-6 at most on the tiny models
ORACLE_F64_TOL = 1e-9     # two float64 evaluations with different shapes


def oracle_logits(cfg: dict, w, token_ids) -> torch.Tensor:
    """The plain implementation's logits for one whole sequence, checked against itself, as float32 values of a
    float64 evaluation (an oracle without rounding of its own). Two evaluations must agree: in float64 and in
    float32 (tensors as read), to float32 rounding; or, when the tensors are float64 already, in float64 with
    other shapes (one token more: causal, so the rows in front are the same function of the same tokens). On
    disagreement a third evaluation, on one thread and with yet other shapes, decides which to believe; when
    nothing agrees the ORACLE is reported as broken, not the engine.
    Why: on a many-core host the CPU library behind ``plain_qwen3`` was seen to return, in a few per cent of the
    processes, logits of a 300-token sequence that are off by 2e-5 to 9e-5 (the same wrong values every time within
    that process, in one precision only), which made exact float32 comparisons fail for no fault of the engine."""
    import plain_qwen3 as plain
    toks = [int(t) for t in token_ids]
    n = len(toks)
    if next(iter(w.values())).dtype == torch.float64:
        w64, second_tol = w, ORACLE_F64_TOL
        second = lambda: plain.forward_logits(cfg, w64, toks + toks[:1])[:n]
    else:
        key = id(w)
        if key not in _ORACLE_F64:
            _ORACLE_F64[key] = (w, {k: v.to(torch.float64) for k, v in w.items()})   # w is kept so that its id stays its own
        w64, second_tol = _ORACLE_F64[key][1], ORACLE_SELF_TOL
        second = lambda: plain.forward_logits(cfg, w, toks)

    def agree(x, y, tol):
        return (x.double() - y.double()).abs().max().item() <= tol * max(1.0, y.abs().max().item())

    a = plain.forward_logits(cfg, w64, toks)
    b = second()
    if agree(a, b, second_tol):
        return a.to(torch.float32)
    threads = torch.get_num_threads()
    try:
        torch.set_num_threads(1)
        c = plain.forward_logits(cfg, w64, toks + toks[:2])[:n]
    finally:
        torch.set_num_threads(threads)
    if agree(a, c, ORACLE_F64_TOL):
        return a.to(torch.float32)
    if agree(b, c, second_tol):
        return c.to(torch.float32)
    raise AssertionError("the plain implementation disagrees with itself "
                         f"(max difference between two evaluations {(a.double() - b.double()).abs().max().item():.3e}): "
                         "the CPU oracle is broken here")


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    diff = (got - ref).abs()
    if dtype == "float32":
        bound = F32_ATOL + F32_RTOL * ref.abs()
        bad = diff > bound
        if bad.any():
            idx = torch.nonzero(bad)[0].tolist()
            raise AssertionError(
                f"{what}: float32 mismatch at {idx}: got {got[tuple(idx)].item():.7f} ref {ref[tuple(idx)].item():.7f} "
                f"(max diff {diff.max().item():.3e}; first bad row {idx[0]})")
    else:
        scale = ref.abs().max().item()
        mx, mean = diff.max().item() / scale, diff.mean().item() / scale
        if mx > BF16_MAX_REL or mean > BF16_MEAN_REL:
            row = int(torch.argmax(diff.max(dim=-1).values)) if diff.dim() > 1 else 0
            raise AssertionError(
                f"{what}: bfloat16 error too large: max {mx:.4f} (bound {BF16_MAX_REL}), mean {mean:.5f} "
                f"(bound {BF16_MEAN_REL}); worst row {row}")


# ---------------------------------------------------------------------------
# traces: lists of steps {"step", "entries": [{"id", "tokens", "want"}], "end"}
# ---------------------------------------------------------------------------
def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def trace_tail(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        s += 1
        for i in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 13, 5, 2, 31, 3, 64, 2, 17)) -> List[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps, s, k = [], 0, 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            last = at + n == len(toks)
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[at: at + n], "want": list(range(n))}],
                          "end": [rid] if last else []})
            at += n
            s += 1
    return steps


def round64(n: int) -> int:
    return -(-n // 64) * 64


def trace_mixed(requests: Dict[str, List[int]], max_tokens: int, seed: int = 0, max_live: int = 4,
                tail: int = 32) -> List[dict]:
    """Up to ``max_live`` live requests; portions of some beside single (decoded) tokens of
    others; a request may sit out a step. A request is admitted only while the live
    requests' token counts (each rounded up to 64) fit ``max_tokens``, so pages are reused."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: Dict[str, int] = {}  # id -> tokens fed so far
    steps, s = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting[0]
            held = sum(round64(len(requests[r])) for r in live)
            if held + round64(len(toks)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = 0
        assert live, "max_tokens too small for the next request"
        entries, ended = [], []
        ids = list(live)
        rng.shuffle(ids)
        for rid in ids:
            if len(ids) > 1 and rng.random() < 0.25:
                continue  # sits this step out
            toks, at = requests[rid], live[rid]
            left = len(toks) - at
            if left <= tail:
                n = 1
            else:
                n = min(left - tail, rng.choice([2, 3, 5, 8, 13, 21, 40]))
            entries.append({"id": rid, "tokens": toks[at: at + n], "want": list(range(n))})
            live[rid] = at + n
            if at + n == len(toks):
                ended.append(rid)
        if not entries:
            continue
        steps.append({"step": s, "entries": entries, "end": ended})
        for rid in ended:
            del live[rid]
        s += 1
    return steps


def count_page_handouts(cache) -> Dict[tuple, int]:
    """From now on, count how often each (group, page id) is handed out by the cache's pools. A page that
    was handed out twice has been used again after a request gave it back."""
    counts: Dict[tuple, int] = {}
    for gi, g in enumerate(cache.groups):
        inner = g.pool.allocate

        def allocate(n, _inner=inner, _gi=gi):
            ids = _inner(n)
            for i in ids:
                counts[(_gi, i)] = counts.get((_gi, i), 0) + 1
            return ids

        g.pool.allocate = allocate
    return counts


def replay_in_process(runner, steps: List[dict]) -> Dict[str, torch.Tensor]:
    """Drive the engine's step function with a trace; returns per request the logits rows
    in position order, [tokens, vocab]."""
    from openinfer_b200.engine.runner import StepEntry

    rows: Dict[str, List[torch.Tensor]] = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = runner.step(entries)
        at = 0
        for e in st["entries"]:
            n = len(e["want"])
            if n:
                rows.setdefault(e["id"], []).append(logits[at: at + n].float().cpu())
                at += n
        for rid in st["end"]:
            runner.end(rid)
    return {rid: torch.cat(parts, 0) for rid, parts in rows.items()}


def replay_trace_run(model_dir: str, dtype: str, steps: List[dict], out_dir: str, max_tokens: int,
                     vocab: int, env=None) -> Dict[str, torch.Tensor]:
    """Drive bin/trace_run as a child process, strictly step by step (next line only after 'done')."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    rows: Dict[str, List[torch.Tensor]] = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if not n_want:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
        at = 0
        for e in st["entries"]:
            n = len(e["want"])
            if n:
                rows.setdefault(e["id"], []).append(torch.from_numpy(arr[at: at + n].copy()))
                at += n
    return {rid: torch.cat(parts, 0) for rid, parts in rows.items()}
