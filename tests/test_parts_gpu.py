"""Each part alone against its plain statement, and the generality of the assembly: a
window, a layer that reads another layer's cache, a layer named twice in the run order, and
a toy mixer with state of its own, a toy feed-forward with routing and a toy position encoding
that are defined here, registered, built and stepped without touching the package."""
import dataclasses
import math
import random
from typing import Dict, List, Optional

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _runner(spec, dtype, tensors, page=4, pages=64):
    from openinfer_b200.cache import CacheManager
    from openinfer_b200.engine.runner import ModelRunner
    from openinfer_b200.parts.model import Model
    model = Model(spec, dtype)
    model.load({k: v.to(DEV).to(dtype) for k, v in tensors.items()}, torch.device(DEV))
    cache = CacheManager(page_size=page)
    model.bind_cache(cache)
    cache.allocate(pages, 8, device=torch.device(DEV), dtype=dtype)
    return ModelRunner(model, cache, torch.device(DEV))


def _random_tensors(spec, seed):
    from openinfer_b200.parts.model import Model
    from openinfer_b200.weights import random_tensors
    return random_tensors(Model(spec, torch.bfloat16).expected_tensors(), seed)


def _mini_spec(window=None, order=None, layers=2, nq=4, nkv=2, hd=16, hidden=40, inter=72, vocab=50,
               rotary_dim=None, qk_norm=True, offset=0.0, activation="silu", embedding_scale=1.0, logit_soft_cap=0.0,
               interleaved=False):
    from openinfer_b200.parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec, PositionSpec)
    norm = NormSpec("rms", hidden, 1e-5, offset)
    pos = PositionSpec("rope", rotary_dim or hd, 777.0, 256, interleaved)
    mixer = AttentionSpec(hidden_size=hidden, num_heads=nq, num_kv_heads=nkv, head_dim=hd,
                          softmax_scale=1 / math.sqrt(hd), position=pos,
                          qk_norm=NormSpec("rms", hd, 1e-5, offset) if qk_norm else None, window=window)
    blocks = tuple(BlockSpec(name=f"L{i}.", mixer=mixer, feed_forward=GatedMlpSpec(hidden_size=hidden, intermediate_size=inter, activation=activation),
                             input_norm=norm, post_norm=norm) for i in range(layers))
    return ModelSpec(vocab_size=vocab, hidden_size=hidden, blocks=blocks, order=tuple(order or range(layers)),
                     final_norm=norm, embedding_name="emb", final_norm_name="fn.", head_name="head", max_positions=256,
                     embedding_scale=embedding_scale, logit_soft_cap=logit_soft_cap)


def _plain_gated_mlp(x, w, prefix, activation):
    """down( act(gate x) * (up x) ); "gelu_tanh": act(g) = 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))."""
    if activation == "silu":
        return plain.swiglu(x, w, prefix)
    g = plain.linear(x, w[prefix + "gate_proj.weight"])
    u = plain.linear(x, w[prefix + "up_proj.weight"])
    act = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    return plain.linear(act * u, w[prefix + "down_proj.weight"])


def _plain_rope(x, cos, sin, interleaved):
    """Rotate-half (the plain implementation's), or the neighbours (2 d, 2 d + 1) by angle d:
    out[2d] = x[2d] cos_d - x[2d+1] sin_d, out[2d+1] = x[2d] sin_d + x[2d+1] cos_d."""
    if not interleaved:
        return plain.apply_rope(x, cos, sin)
    a, b = x[..., 0::2], x[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2)


def _plain_forward(spec, w, toks, window=None, order=None, cache_of=None, rotary_dim=None, qk_norm=True, offset=0.0,
                   activation="silu", embedding_scale=1.0, logit_soft_cap=0.0, interleaved=False):
    """Whole-sequence float32 forward of a mini spec, from the plain part functions."""
    w = {k: v.float() for k, v in w.items()}
    m = spec.blocks[0].mixer
    T = len(toks)
    positions = torch.arange(T)
    h = plain.embedding(torch.tensor(toks), w["emb"]) * embedding_scale
    kv_of_call = {}
    calls = spec.calls()
    for ci, c in enumerate(calls):
        p = f"L{c.layer}."
        x = plain.rms_norm(h, offset + w[p + "input_layernorm.weight"], 1e-5)
        a = p + "self_attn."
        q = plain.linear(x, w[a + "q_proj.weight"]).view(T, m.num_heads, m.head_dim)
        if qk_norm:
            q = plain.rms_norm(q, offset + w[a + "q_norm.weight"], 1e-5)
        rot = rotary_dim or m.head_dim
        cos, sin = plain.rope_tables(rot, 777.0, positions)
        q = torch.cat([_plain_rope(q[..., :rot], cos, sin, interleaved), q[..., rot:]], -1)
        if c.read_cache_of is None:
            k = plain.linear(x, w[a + "k_proj.weight"]).view(T, m.num_kv_heads, m.head_dim)
            if qk_norm:
                k = plain.rms_norm(k, offset + w[a + "k_norm.weight"], 1e-5)
            k = torch.cat([_plain_rope(k[..., :rot], cos, sin, interleaved), k[..., rot:]], -1)
            v = plain.linear(x, w[a + "v_proj.weight"]).view(T, m.num_kv_heads, m.head_dim)
            kv_of_call[ci] = (k, v)
        else:
            k, v = kv_of_call[c.read_cache_of]
        o = plain.causal_attention(q, k, v, m.softmax_scale, window)
        h = h + plain.linear(o.reshape(T, -1), w[a + "o_proj.weight"])
        x = plain.rms_norm(h, offset + w[p + "post_attention_layernorm.weight"], 1e-5)
        h = h + _plain_gated_mlp(x, w, p + "mlp.", activation)
    h = plain.rms_norm(h, offset + w["fn.weight"], 1e-5)
    logits = plain.linear(h, w["head"])
    return logit_soft_cap * torch.tanh(logits / logit_soft_cap) if logit_soft_cap > 0 else logits


def _step_all(runner, toks, cuts):
    from openinfer_b200.engine.runner import StepEntry
    out, at = [], 0
    for n in cuts:
        out.append(runner.step([StepEntry("r", toks[at: at + n], list(range(n)))]).float().cpu())
        at += n
    assert at == len(toks)
    runner.end("r")
    return torch.cat(out)


def _cuts(n, rng):
    cuts = []
    while n:
        c = min(n, rng.choice([1, 2, 3, 7, 11]))
        cuts.append(c)
        n -= c
    return cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["plain", "window", "partial_rotary", "no_qk_norm", "one_plus_w",
                                  "shared_cache", "layer_twice", "interleaved_rotary", "interleaved_partial_rotary"])
def test_assemblies(dtype, case):
    from openinfer_b200.parts.spec import LayerCall
    kw, pkw = {}, {}
    if case == "window":
        kw = dict(window=6)
        pkw = dict(window=6)
    elif case == "partial_rotary":
        kw = dict(rotary_dim=8)
        pkw = dict(rotary_dim=8)
    elif case == "no_qk_norm":
        kw = dict(qk_norm=False)
        pkw = dict(qk_norm=False)
    elif case == "one_plus_w":
        kw = dict(offset=1.0)
        pkw = dict(offset=1.0)
    elif case == "interleaved_rotary":    # the rotation turns neighbouring pairs (2 d, 2 d + 1)
        kw = dict(interleaved=True)
        pkw = dict(interleaved=True)
    elif case == "interleaved_partial_rotary":
        kw = dict(interleaved=True, rotary_dim=8)
        pkw = dict(interleaved=True, rotary_dim=8)
    elif case == "shared_cache":      # the second call reads the keys and values of the first
        kw = dict(order=(0, LayerCall(1, read_cache_of=0)))
    elif case == "layer_twice":       # layer 0 runs twice (with a cache of its own each time), then layer 1
        kw = dict(order=(0, 0, 1))
    spec = _mini_spec(**kw)
    w = _random_tensors(spec, 3)
    rng = random.Random(1)
    toks = [rng.randrange(50) for _ in range(37)]
    ref = _plain_forward(spec, w, toks, **pkw)
    runner = _runner(spec, dtype, w)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    assert_close(_step_all(runner, toks, [len(toks)]), ref, name, f"{case} whole")
    assert_close(_step_all(runner, toks, _cuts(len(toks), rng)), ref, name, f"{case} in portions")
    runner.cache.check()
    assert all(f == runner.cache.num_pages for f in runner.cache.free_pages())
    if case == "window":
        # pages behind the window went back while the request was live
        from openinfer_b200.engine.runner import StepEntry
        for t in toks:
            runner.step([StepEntry("w", [t], [])])
        assert runner.cache.groups[0].pool.used_count <= -(-6 // 4) + 1
        runner.end("w")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_each_part_alone(dtype):
    """Norm, feed-forward and attention parts, each called by itself."""
    from openinfer_b200.parts import build_feed_forward, build_norm
    from openinfer_b200.parts.spec import GatedMlpSpec, NormSpec
    torch.manual_seed(0)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    x = torch.randn(9, 56).to(dtype)
    norm = build_norm(NormSpec("rms", 56, 1e-4))
    wn = (1 + 0.1 * torch.randn(56)).to(dtype)
    norm.load({"weight": wn.to(DEV)})
    got = norm(x.to(DEV))
    assert torch.allclose(got.float().cpu(), plain.rms_norm(x.float(), wn.float(), 1e-4), atol=2e-2 if dtype == torch.bfloat16 else 1e-5)
    ffn = build_feed_forward(GatedMlpSpec(hidden_size=56, intermediate_size=88))
    wf = {k: (torch.randn(s) * 0.1).to(dtype) for k, s in
          {"gate_proj.weight": (88, 56), "up_proj.weight": (88, 56), "down_proj.weight": (56, 88)}.items()}
    ffn.load({k: v.to(DEV) for k, v in wf.items()})
    got = ffn.forward(x.to(DEV), None)
    ref = plain.swiglu(x.float(), {k: v.float() for k, v in wf.items()}, "")
    assert_close(got, ref, name, "gated mlp")


# ---------------------------------------------------------------------------
# a toy mixer with state of its own: a running mean of the inputs of a request
# ---------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class RunningMeanSpec:
    kind: str = "toy_running_mean"
    hidden_size: int = 0


def _register_toy():
    from openinfer_b200.cache import StateNeed
    from openinfer_b200.parts import Mixer, ParamInfo, register_mixer

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """y_t = w * mean(x_0..x_t) of the request; the state is (sum, count). Written with
        torch ops: it is a test double, not a product kernel."""

        def parameters(self):
            return {"scale.weight": ParamInfo((self.spec.hidden_size,), ("one_plus_normal", 0.02))}

        def load(self, tensors):
            self.w = tensors["scale.weight"]

        def state_needs(self):
            return [StateNeed((self.spec.hidden_size + 1,), "float32")]

        def forward(self, x, ctx, binding):
            state = ctx.cache.state_tensor(binding.states[0])
            out = torch.empty_like(x)
            row = 0
            for b, n in enumerate(ctx.q_lens_host):
                slot = ctx.state_slots_host[b]
                s = state[slot]
                xs = x[row: row + n].float()
                csum = torch.cumsum(xs, 0) + s[:-1]
                cnt = torch.arange(1, n + 1, device=x.device, dtype=torch.float32) + s[-1]
                out[row: row + n] = (csum / cnt[:, None] * self.w.float()).to(x.dtype)
                s[:-1] = csum[-1]
                s[-1] = cnt[-1]
                row += n
            return out

    return RunningMean


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation_embedding_scale_and_logit_cap_are_spec_values(dtype):
    """Another gate activation (tanh-GELU), a scale on the embedded rows and a soft cap on the logits are values
    of the spec: the package's own feed-forward and model take them, its kernels get the activation as an argument.
    Sizes at which the bfloat16 path forms the activation in all three places: the streaming product (steps of up
    to 32 rows), the stand-alone kernel (33 to 127 rows) and the epilogue of the tcgen05 product (128 rows and more)."""
    kw = dict(layers=2, nq=4, nkv=2, hd=64, hidden=256, inter=512, vocab=300)
    extra = dict(activation="gelu_tanh", embedding_scale=3.5, logit_soft_cap=2.0)
    spec = _mini_spec(**kw, **extra)
    w = _random_tensors(spec, 21)
    rng = random.Random(6)
    toks = [rng.randrange(300) for _ in range(230)]
    ref = _plain_forward(spec, w, toks, **extra)
    assert float(ref.abs().max()) <= 2.0 and float(ref.abs().max()) > 1.0     # the cap bites
    assert not torch.allclose(ref, _plain_forward(spec, w, toks, embedding_scale=3.5, logit_soft_cap=2.0), atol=1e-3)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    runner = _runner(spec, dtype, w, page=16, pages=32)
    got = _step_all(runner, toks, [130, 40, 7, 1, 1, 33, 18])
    assert_close(got, ref, name, f"gelu_tanh / scaled embedding / capped logits {name}")
    with pytest.raises(Exception, match="no kernel"):
        _runner(_mini_spec(**kw, activation="relu_squared"), dtype, w)


def test_toy_mixer_with_state_registers_builds_and_steps():
    from openinfer_b200.engine.runner import StepEntry
    from openinfer_b200.parts.spec import BlockSpec, GatedMlpSpec, ModelSpec, NormSpec
    _register_toy()
    hidden, vocab = 24, 31
    norm = NormSpec("rms", hidden, 1e-5)
    attn_block = _mini_spec(layers=1, hidden=hidden, nq=2, nkv=1, hd=8, inter=40, vocab=vocab).blocks[0]
    toy_block = BlockSpec(name="T.", mixer=RunningMeanSpec(hidden_size=hidden), mixer_name="mix.",
                          feed_forward=GatedMlpSpec(hidden_size=hidden, intermediate_size=40),
                          input_norm=norm, post_norm=norm)
    # one model with different mixers in different layers
    spec = ModelSpec(vocab_size=vocab, hidden_size=hidden, blocks=(toy_block, attn_block), order=(0, 1),
                     final_norm=norm, embedding_name="emb", final_norm_name="fn.", head_name="head", max_positions=256)
    w = _random_tensors(spec, 5)
    assert "T.mix.scale.weight" in w
    runner = _runner(spec, torch.float32, w)
    assert len(runner.cache.state_needs) == 1 and len(runner.cache.groups) == 1

    def plain_forward(toks):
        wf = {k: v.float() for k, v in w.items()}
        T = len(toks)
        h = plain.embedding(torch.tensor(toks), wf["emb"])
        x = plain.rms_norm(h, wf["T.input_layernorm.weight"], 1e-5)
        mean = torch.cumsum(x, 0) / torch.arange(1, T + 1)[:, None]
        h = h + mean * wf["T.mix.scale.weight"]
        h = h + plain.swiglu(plain.rms_norm(h, wf["T.post_attention_layernorm.weight"], 1e-5), wf, "T.mlp.")
        sub = _mini_spec(layers=1, hidden=hidden, nq=2, nkv=1, hd=8, inter=40, vocab=vocab)
        # the attention block on top, through the same plain functions as the other tests
        m = sub.blocks[0].mixer
        p = "L0."
        x = plain.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-5)
        pos = torch.arange(T)
        cos, sin = plain.rope_tables(8, 777.0, pos)
        q = plain.apply_rope(plain.rms_norm(plain.linear(x, wf[p + "self_attn.q_proj.weight"]).view(T, 2, 8), wf[p + "self_attn.q_norm.weight"], 1e-5), cos, sin)
        k = plain.apply_rope(plain.rms_norm(plain.linear(x, wf[p + "self_attn.k_proj.weight"]).view(T, 1, 8), wf[p + "self_attn.k_norm.weight"], 1e-5), cos, sin)
        v = plain.linear(x, wf[p + "self_attn.v_proj.weight"]).view(T, 1, 8)
        h = h + plain.linear(plain.causal_attention(q, k, v, m.softmax_scale).reshape(T, -1), wf[p + "self_attn.o_proj.weight"])
        h = h + plain.swiglu(plain.rms_norm(h, wf[p + "post_attention_layernorm.weight"], 1e-5), wf, p + "mlp.")
        return plain.linear(plain.rms_norm(h, wf["fn.weight"], 1e-5), wf["head"])

    rng = random.Random(2)
    a = [rng.randrange(vocab) for _ in range(19)]
    b = [rng.randrange(vocab) for _ in range(11)]
    # two requests interleaved, in portions: each keeps a state of its own
    got_a, got_b = [], []
    got_a.append(runner.step([StepEntry("a", a[:5], list(range(5)))]))
    both = runner.step([StepEntry("b", b[:4], list(range(4))), StepEntry("a", a[5:6], [0])])
    got_b.append(both[:4]); got_a.append(both[4:])
    both = runner.step([StepEntry("a", a[6:], list(range(13))), StepEntry("b", b[4:], list(range(7)))])
    got_a.append(both[:13]); got_b.append(both[13:])
    assert_close(torch.cat(got_a), plain_forward(a), "float32", "toy request a")
    assert_close(torch.cat(got_b), plain_forward(b), "float32", "toy request b")
    runner.end("a")
    # a new request in a's slot starts from a cleared state
    again = runner.step([StepEntry("c", a, list(range(len(a))))])
    assert_close(again, plain_forward(a), "float32", "toy request c in a reused slot")
    runner.end("b"); runner.end("c")
    runner.cache.check()


# ---------------------------------------------------------------------------
# a toy feed-forward with routing and a toy position encoding, defined here: one model mixes them
# with the package's own parts, layer by layer, without a change to the package
# ---------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class RoutedToySpec:
    kind: str = "toy_routed"
    hidden_size: int = 0
    inner: int = 0
    experts: int = 0


@dataclasses.dataclass(frozen=True)
class HalvedPositionSpec:
    kind: str = "toy_halved_rope"
    rotary_dim: int = 0
    theta: float = 100.0
    max_positions: int = 0


def _register_toy_ffn_and_position():
    from openinfer_b200.parts import ParamInfo
    from openinfer_b200.parts.base import FeedForward, PositionEncoding
    from openinfer_b200.parts.registry import register_feed_forward, register_position_encoding

    @register_feed_forward("toy_routed")
    class RoutedToy(FeedForward):
        """Every row goes to the ONE expert its router logit (float32) is largest for:
        y = gate_e * relu(x W1_e^T) W2_e^T. torch ops: a test double, not a product kernel."""

        def parameters(self):
            s = self.spec
            return {"router.weight": ParamInfo((s.experts, s.hidden_size)),
                    "w1": ParamInfo((s.experts * s.inner, s.hidden_size)),
                    "w2": ParamInfo((s.experts * s.hidden_size, s.inner))}

        def load(self, tensors):
            s = self.spec
            self.router = tensors["router.weight"]
            self.w1 = tensors["w1"].view(s.experts, s.inner, s.hidden_size)
            self.w2 = tensors["w2"].view(s.experts, s.hidden_size, s.inner)

        def forward(self, x, ctx):
            logits = x.float() @ self.router.float().t()
            prob = torch.softmax(logits, -1)
            top = prob.argmax(-1)
            out = torch.zeros_like(x, dtype=torch.float32)
            for e in range(self.spec.experts):
                rows = (top == e).nonzero().flatten()
                if rows.numel():
                    hmid = torch.relu(x[rows].float() @ self.w1[e].float().t())
                    out[rows] = prob[rows, e, None] * (hmid @ self.w2[e].float().t())
            return out.to(x.dtype)

    @register_position_encoding("toy_halved_rope")
    class HalvedRope(PositionEncoding):
        """Rotation by HALF the position: angle = (pos / 2) * theta^(-2i / rotary_dim). Only the table differs."""

        def rotation_tables(self, device):
            s = self.spec
            half = s.rotary_dim // 2
            inv = 1.0 / torch.pow(torch.tensor(float(s.theta)), torch.arange(half, dtype=torch.float32) * 2.0 / s.rotary_dim)
            ang = (torch.arange(s.max_positions, dtype=torch.float32) / 2.0)[:, None] * inv[None, :]
            return torch.cos(ang).contiguous().to(device), torch.sin(ang).contiguous().to(device)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_toy_position_encoding(dtype_name):
    from openinfer_b200.engine.runner import StepEntry
    from openinfer_b200.parts.spec import AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec
    _register_toy_ffn_and_position()
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    hidden, vocab, nq, nkv, hd, rot = 40, 37, 4, 2, 16, 8
    norm = NormSpec("rms", hidden, 1e-5)
    toy_attn = AttentionSpec(hidden_size=hidden, num_heads=nq, num_kv_heads=nkv, head_dim=hd, softmax_scale=0.3,
                             position=HalvedPositionSpec(rotary_dim=rot, theta=100.0, max_positions=128), qk_norm=None)
    usual = _mini_spec(layers=1, hidden=hidden, nq=nq, nkv=nkv, hd=hd, inter=72, vocab=vocab).blocks[0]
    toy_block = BlockSpec(name="T.", mixer=toy_attn, feed_forward=RoutedToySpec(hidden_size=hidden, inner=24, experts=3),
                          input_norm=norm, post_norm=norm)
    spec = ModelSpec(vocab_size=vocab, hidden_size=hidden, blocks=(toy_block, usual), order=(0, 1), final_norm=norm,
                     embedding_name="emb", final_norm_name="fn.", head_name="head", max_positions=128)
    w = _random_tensors(spec, 9)
    assert {"T.mlp.router.weight", "T.mlp.w1", "T.mlp.w2"} <= set(w)
    w["T.mlp.router.weight"] = w["T.mlp.router.weight"] * 40     # clear routing decisions, all experts in use
    runner = _runner(spec, dtype, w)

    def plain_forward(toks):
        wf = {k: v.float() for k, v in w.items()}
        T = len(toks)
        pos = torch.arange(T)
        h = plain.embedding(torch.tensor(toks), wf["emb"])
        # the toy layer: attention with the halved rotation over the first `rot` dims, no q/k norm
        x = plain.rms_norm(h, wf["T.input_layernorm.weight"], 1e-5)
        inv = 1.0 / torch.pow(torch.tensor(100.0), torch.arange(rot // 2, dtype=torch.float32) * 2.0 / rot)
        ang = (pos.float() / 2.0)[:, None] * inv[None, :]
        cos, sin = torch.cos(ang), torch.sin(ang)
        q = plain.linear(x, wf["T.self_attn.q_proj.weight"]).view(T, nq, hd)
        k = plain.linear(x, wf["T.self_attn.k_proj.weight"]).view(T, nkv, hd)
        v = plain.linear(x, wf["T.self_attn.v_proj.weight"]).view(T, nkv, hd)
        q = torch.cat([plain.apply_rope(q[..., :rot], cos, sin), q[..., rot:]], -1)
        k = torch.cat([plain.apply_rope(k[..., :rot], cos, sin), k[..., rot:]], -1)
        h = h + plain.linear(plain.causal_attention(q, k, v, 0.3).reshape(T, -1), wf["T.self_attn.o_proj.weight"])
        x = plain.rms_norm(h, wf["T.post_attention_layernorm.weight"], 1e-5)
        prob = torch.softmax(x @ wf["T.mlp.router.weight"].t(), -1)
        top = prob.argmax(-1)
        w1 = wf["T.mlp.w1"].view(3, 24, hidden)
        w2 = wf["T.mlp.w2"].view(3, hidden, 24)
        y = torch.stack([prob[t, top[t]] * (torch.relu(x[t] @ w1[top[t]].t()) @ w2[top[t]].t()) for t in range(T)])
        assert len(set(top.tolist())) >= 2, "the test wants rows on different experts"
        h = h + y
        # the usual layer on top
        p = "L0."
        m = usual.mixer
        x = plain.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-5)
        cos, sin = plain.rope_tables(hd, 777.0, pos)
        q = plain.apply_rope(plain.rms_norm(plain.linear(x, wf[p + "self_attn.q_proj.weight"]).view(T, nq, hd), wf[p + "self_attn.q_norm.weight"], 1e-5), cos, sin)
        k = plain.apply_rope(plain.rms_norm(plain.linear(x, wf[p + "self_attn.k_proj.weight"]).view(T, nkv, hd), wf[p + "self_attn.k_norm.weight"], 1e-5), cos, sin)
        v = plain.linear(x, wf[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
        h = h + plain.linear(plain.causal_attention(q, k, v, m.softmax_scale).reshape(T, -1), wf[p + "self_attn.o_proj.weight"])
        h = h + plain.swiglu(plain.rms_norm(h, wf[p + "post_attention_layernorm.weight"], 1e-5), wf, p + "mlp.")
        return plain.linear(plain.rms_norm(h, wf["fn.weight"], 1e-5), wf["head"])

    rng = random.Random(4)
    a = [rng.randrange(vocab) for _ in range(21)]
    b = [rng.randrange(vocab) for _ in range(9)]
    got_a = [runner.step([StepEntry("a", a[:7], list(range(7)))])]
    both = runner.step([StepEntry("b", b, list(range(9))), StepEntry("a", a[7:8], [0])])
    got_b = both[:9]
    got_a.append(both[9:])
    got_a.append(runner.step([StepEntry("a", a[8:], list(range(13)))]))
    if dtype_name == "float32":
        assert_close(torch.cat(got_a), plain_forward(a), dtype_name, "toy routed model, request a")
        assert_close(got_b, plain_forward(b), dtype_name, "toy routed model, request b")
    else:
        # bfloat16 rounding may send a row near a tie to another expert: compare where float32 routing is clear
        ref = plain_forward(a)
        err = (torch.cat(got_a).float().cpu() - ref).abs().max(dim=1).values / ref.abs().max()
        assert (err < 0.05).float().mean() >= 0.8, f"rows within 5 %: {(err < 0.05).float().mean():.2f}"
    runner.end("a"); runner.end("b")
    runner.cache.check()


def _drive_together(runner, seqs, rng):
    """All requests at once through the step function: portions of changing size (a request may sit a step out),
    then the last 30 tokens of each one by one; returns the logits of every position, per request."""
    from openinfer_b200.engine.runner import StepEntry
    at = {r: 0 for r in seqs}
    got = {r: [] for r in seqs}
    live = list(seqs)
    while live:
        entries = []
        for r in list(live):
            left = len(seqs[r]) - at[r]
            n = 1 if left <= 30 else min(left - 30, rng.choice([1, 2, 9, 31, 64, 100]))
            if rng.random() < 0.2 and len(live) > 1:
                continue
            entries.append((r, n))
        if not entries:
            continue
        logits = runner.step([StepEntry(r, seqs[r][at[r]: at[r] + n], list(range(n))) for r, n in entries]).float().cpu()
        row = 0
        for r, n in entries:
            got[r].append(logits[row: row + n])
            row += n
            at[r] += n
            if at[r] == len(seqs[r]):
                runner.end(r)
                live.remove(r)
    return {r: torch.cat(v) for r, v in got.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,nq,nkv,hidden,inter,window", [(128, 8, 2, 256, 384, 40), (64, 6, 3, 192, 320, 100),
                                                           (128, 4, 4, 128, 256, 17)])
def test_windows_through_the_tuned_kernels(dtype, hd, nq, nkv, hidden, inter, window):
    """A mixer with a window at head sizes 64 and 128 and pages of 16 keys, where the tensor-core kernels run (prompt
    tiles, decode rows in recorded graphs): five requests together in portions of changing size and then token by
    token, in a pool smaller than their total length, so that pages behind the window go back while a request lives
    and are used again; against the plain implementation with the same window."""
    spec = _mini_spec(window=window, nq=nq, nkv=nkv, hd=hd, hidden=hidden, inter=inter, vocab=120)
    w = _random_tensors(spec, 3)
    rng = random.Random(window + hd)
    seqs = {f"q{i}": [rng.randrange(120) for _ in range(n)] for i, n in enumerate((250, 131, 64, 199, 33))}
    refs = {r: _plain_forward(spec, w, t, window=window) for r, t in seqs.items()}
    name = "float32" if dtype == torch.float32 else "bfloat16"
    runner = _runner(spec, dtype, w, page=16, pages=40)      # 640 tokens of room for requests of 677 tokens
    runner.cuda_graph = True
    got = _drive_together(runner, seqs, rng)
    for r in seqs:
        assert_close(got[r], refs[r], name, f"head {hd}, window {window}, {name}, request {r}")
    assert runner._graphs, "the single-token steps did not go through a graph"
    runner.cache.check()
    assert all(f == runner.cache.num_pages for f in runner.cache.free_pages())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["partial_rotary", "partial_rotary_16", "no_qk_norm", "one_plus_w", "interleaved_rotary",
                                  "shared_cache", "layer_twice", "gelu_tanh", "window_and_shared_cache"])
def test_assemblies_through_the_tensor_core_kernels(dtype, case):
    """The assemblies of test_assemblies once more at a head size of 128 and pages of 16 keys, where the bfloat16 model
    runs the tensor-core attention kernels, the decode kernel with the rotation inside, the streaming products and
    recorded graphs (the float32 model the general ones): five requests together, portions and single tokens."""
    from openinfer_b200.parts.spec import LayerCall
    kw, pkw = {
        "partial_rotary": (dict(rotary_dim=64), dict(rotary_dim=64)),
        "partial_rotary_16": (dict(rotary_dim=16), dict(rotary_dim=16)),
        "no_qk_norm": (dict(qk_norm=False), dict(qk_norm=False)),
        "one_plus_w": (dict(offset=1.0), dict(offset=1.0)),
        "interleaved_rotary": (dict(interleaved=True), dict(interleaved=True)),
        "shared_cache": (dict(order=(0, LayerCall(1, read_cache_of=0))), {}),
        "layer_twice": (dict(order=(0, 0, 1)), {}),
        "gelu_tanh": (dict(activation="gelu_tanh"), dict(activation="gelu_tanh")),
        "window_and_shared_cache": (dict(window=50, order=(0, LayerCall(1, read_cache_of=0))), dict(window=50)),
    }[case]
    spec = _mini_spec(nq=8, nkv=2, hd=128, hidden=256, inter=384, vocab=120, **kw)
    w = _random_tensors(spec, 3)
    if case == "one_plus_w":     # stored around zero, as such models store them: 1 + w is around one
        w = {k: (v - 1.0 if (k.endswith("norm.weight") or k == "fn.weight") else v) for k, v in w.items()}
    rng = random.Random(len(case))
    seqs = {f"q{i}": [rng.randrange(120) for _ in range(n)] for i, n in enumerate((250, 131, 64, 199, 33))}
    refs = {r: _plain_forward(spec, w, t, **pkw) for r, t in seqs.items()}
    name = "float32" if dtype == torch.float32 else "bfloat16"
    runner = _runner(spec, dtype, w, page=16, pages=64)
    runner.cuda_graph = True
    got = _drive_together(runner, seqs, rng)
    for r in seqs:
        assert_close(got[r], refs[r], name, f"{case}, {name}, request {r}")
    runner.cache.check()
    assert all(f == runner.cache.num_pages for f in runner.cache.free_pages())
