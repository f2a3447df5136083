"""The plain implementation itself (no GPU): properties any correct restatement must have."""
import math
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, make_model_folder, random_tokens


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in list(TINY.items())[:2]:
        f = make_model_folder(str(tmp_path_factory.mktemp(f"p{name}")), cfg, seed)
        out[name] = plain.read_model_folder(f)
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_causal_and_shapes(models, name):
    cfg, w = models[name]
    rng = random.Random(3)
    toks = random_tokens(rng, 40, cfg["vocab_size"])
    full = plain.forward_logits(cfg, w, toks)
    assert full.shape == (40, cfg["vocab_size"]) and torch.isfinite(full).all()
    # a position's logits depend only on the tokens up to it
    part = plain.forward_logits(cfg, w, toks[:17])
    assert torch.allclose(full[:17], part, atol=1e-5, rtol=1e-5)
    other = list(toks)
    other[30] = (other[30] + 1) % cfg["vocab_size"]
    changed = plain.forward_logits(cfg, w, other)
    assert torch.allclose(full[:30], changed[:30], atol=1e-6) and not torch.allclose(full[30:], changed[30:], atol=1e-4)


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]])
    out = plain.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 / rms * 2.0, 4 / rms * 0.5]]))
    w = {"gate_proj.weight": torch.tensor([[1.0]]), "up_proj.weight": torch.tensor([[2.0]]),
         "down_proj.weight": torch.tensor([[3.0]])}
    y = plain.swiglu(torch.tensor([[0.7]]), w, "")
    assert torch.allclose(y, torch.tensor([[0.7 / (1 + math.exp(-0.7)) * 1.4 * 3.0]]))


def test_rope_is_a_rotation_and_relative():
    hd, theta = 16, 10000.0
    pos = torch.arange(50)
    cos, sin = plain.rope_tables(hd, theta, pos)
    assert cos.shape == (50, 8) and torch.allclose(cos[0], torch.ones(8)) and torch.allclose(sin[0], torch.zeros(8))
    assert abs(cos[1, 1].item() - math.cos(1.0 / theta ** (2 / 16))) < 1e-6
    q, k = torch.randn(50, 1, hd), torch.randn(50, 1, hd)
    qr, kr = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
    assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-4)
    # <rope(q, m), rope(k, n)> depends on m - n only
    q1, k1 = q[0:1].expand(50, 1, hd), k[0:1].expand(50, 1, hd)
    a = (plain.apply_rope(q1, cos, sin)[10] * plain.apply_rope(k1, cos, sin)[7]).sum()
    b = (plain.apply_rope(q1, cos, sin)[33] * plain.apply_rope(k1, cos, sin)[30]).sum()
    assert abs(a.item() - b.item()) < 1e-3


def test_attention_groups_window_and_softmax():
    T, nq, nkv, hd = 9, 6, 2, 8
    q, k, v = torch.randn(T, nq, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    o = plain.causal_attention(q, k, v, 0.3)
    assert torch.allclose(o[0], v[0].repeat_interleave(3, dim=0), atol=1e-6)  # first token sees only itself
    # heads 0..2 read kv head 0, heads 3..5 kv head 1
    v2 = v.clone()
    v2[:, 1] += 1.0
    o2 = plain.causal_attention(q, k, v2, 0.3)
    assert torch.allclose(o2[:, :3], o[:, :3]) and torch.allclose(o2[:, 3:], o[:, 3:] + 1.0, atol=1e-5)
    # window 1 = only itself; window >= T = full
    assert torch.allclose(plain.causal_attention(q, k, v, 0.3, window=1), v.repeat_interleave(3, dim=1), atol=1e-6)
    assert torch.allclose(plain.causal_attention(q, k, v, 0.3, window=T), o, atol=1e-6)


def test_greedy_generation_is_consistent(models):
    cfg, w = models["A"]
    out = plain.greedy_generate(cfg, w, [5, 9, 200], 5)
    seq = [5, 9, 200]
    for t in out:
        assert int(plain.forward_logits(cfg, w, seq)[-1].argmax()) == t
        seq.append(t)


def test_sampling_distribution_semantics():
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -3.0])
    p = torch.softmax(logits / 0.7, 0).double()
    d = plain.sampling_distribution(logits, 0.7)
    assert torch.allclose(d, p, atol=1e-7)
    d = plain.sampling_distribution(logits, 0.7, top_k=2)
    assert (d > 0).tolist() == [True, True, False, False, False, False] and abs(d.sum().item() - 1) < 1e-9
    d = plain.sampling_distribution(logits, 1.0, top_p=0.8)
    ps = torch.softmax(logits, 0)
    n = int((torch.cumsum(ps, 0) < 0.8).sum()) + 1
    assert int((d > 0).sum()) == n
    d = plain.sampling_distribution(logits, 1.0, min_p=0.3)
    assert (d > 0).tolist() == (ps >= 0.3 * ps.max()).tolist()
    # top-k then top-p works on the renormalised rest
    d = plain.sampling_distribution(logits, 1.0, top_k=3, top_p=0.6)
    r = ps[:3] / ps[:3].sum()
    n = int((torch.cumsum(r, 0) < 0.6).sum()) + 1
    assert int((d > 0).sum()) == n
    assert plain.inverse_cdf_pick(torch.tensor([0.0, 0.25, 0.0, 0.75]), 0.2) == 1
    assert plain.inverse_cdf_pick(torch.tensor([0.0, 0.25, 0.0, 0.75]), 0.25) == 3
    assert plain.inverse_cdf_pick(torch.tensor([0.0, 0.25, 0.0, 0.75]), 0.999) == 3


def test_bfloat16_twin_with_the_reference_rounding_points(tmp_path):
    """The twin restates WHERE the reference rounds (q/k norm twice, every product of the rotation, SiLU before the
    multiply, each residual sum, bfloat16 tables and logits). Its logits are bfloat16 values, stay within the
    bfloat16 tolerance of the float32 plain implementation on all five tiny configurations, and its rounding
    points are live: each differs from the single rounding somewhere."""
    import plain_qwen3_bf16 as twin
    from helpers import BF16_MAX_REL, BF16_MEAN_REL
    for name, (cfg, seed) in TINY.items():
        f = make_model_folder(str(tmp_path / name), cfg, seed)
        c, w = plain.read_model_folder(f)
        toks = random_tokens(random.Random(3), 90, cfg["vocab_size"])
        a, b = plain.forward_logits(c, w, toks), twin.forward_logits(c, w, toks)
        assert torch.equal(b, b.to(torch.bfloat16).float()), "the twin's logits are not bfloat16 values"
        scale = a.abs().max().item()
        err = (a - b).abs()
        assert err.max().item() / scale <= BF16_MAX_REL and err.mean().item() / scale <= BF16_MEAN_REL, name
        assert err.max().item() > 0
    torch.manual_seed(0)
    u, wn = torch.randn(50, 3, 32), 1 + 0.1 * torch.randn(32)
    once = twin.bf(plain.rms_norm(u, wn, 1e-6))
    assert not torch.equal(twin.head_norm(u, wn, 1e-6), once), "two roundings never differ from one"
    pos = torch.arange(50)
    cos, sin = plain.rope_tables(32, 1e4, pos)
    assert not torch.equal(twin.apply_rope(twin.bf(u), pos, 1e4), twin.bf(plain.apply_rope(twin.bf(u), cos, sin)))


def test_oracle_checks_itself_and_survives_one_wrong_evaluation(tmp_path, monkeypatch):
    """``oracle_logits`` evaluates the plain implementation in float32 and float64 and wants them to agree; when one
    evaluation is off (simulated here: the float32 one, by 5e-5 at one place) a third evaluation with other shapes
    decides, and the exact result comes back; when nothing agrees it reports the oracle, not the engine."""
    from helpers import oracle_logits
    f = make_model_folder(str(tmp_path / "m"), TINY["A"][0], TINY["A"][1])
    c, w = plain.read_model_folder(f)
    toks = random_tokens(random.Random(5), 60, c["vocab_size"])
    good = oracle_logits(c, w, toks)
    assert (good - plain.forward_logits(c, w, toks)).abs().max().item() < 5e-6
    real = plain.forward_logits

    def off_in_float32(cfg, ww, t):
        out = real(cfg, ww, t).clone()
        if next(iter(ww.values())).dtype == torch.float32:
            out[5, 7] += 5e-5
        return out

    monkeypatch.setattr(plain, "forward_logits", off_in_float32)
    assert torch.equal(oracle_logits(c, w, toks), good)

    def off_everywhere(cfg, ww, t):
        out = real(cfg, ww, t).clone()
        out[5, 7] += 5e-5 * (1 + len(t) % 3) * (2.0 if out.dtype == torch.float64 else 1.0)
        return out

    monkeypatch.setattr(plain, "forward_logits", off_everywhere)
    with pytest.raises(AssertionError, match="oracle"):
        oracle_logits(c, w, toks)

    # float64 tensors: the second evaluation has other shapes; one wrong evaluation is outvoted
    monkeypatch.setattr(plain, "forward_logits", real)
    _, w64 = plain.read_model_folder(f, torch.float64)
    good64 = oracle_logits(c, w64, toks)
    assert (good64 - good).abs().max().item() < 1e-6
    calls = {"n": 0}

    def first_call_off(cfg, ww, t):
        out = real(cfg, ww, t).clone()
        calls["n"] += 1
        if calls["n"] == 1:
            out[3, 2] += 1e-4
        return out

    monkeypatch.setattr(plain, "forward_logits", first_call_off)
    assert torch.equal(oracle_logits(c, w64, toks), good64) and calls["n"] == 3
