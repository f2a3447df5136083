"""Weight loading errors and the random-weights mode (no GPU: tensors are loaded to the CPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from helpers import TINY_A, TINY_B, make_model_folder
from openinfer_b200.config import Qwen3Config
from openinfer_b200.weights import WeightError, expected_tensors, load_tensors, random_tensors


@pytest.fixture()
def folder(tmp_path):
    return make_model_folder(str(tmp_path / "m"), TINY_B, seed=1)


def _rewrite(folder, fn):
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    fn(t)
    save_file(t, path)


def test_loads_by_name_in_bf16(folder):
    cfg = Qwen3Config.from_dict(TINY_B)
    exp = expected_tensors(cfg)
    assert "lm_head.weight" in exp and "model.layers.2.self_attn.q_norm.weight" in exp
    assert len(exp) == 3 + 3 * 11
    t = load_tensors(folder, exp, torch.bfloat16, "cpu")
    assert set(t) == set(exp)
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    assert t["model.layers.0.self_attn.q_proj.weight"].shape == (192, 96)
    t32 = load_tensors(folder, exp, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.norm.weight"], t["model.norm.weight"].float())  # widened exactly


def test_tied_model_has_no_lm_head(tmp_path):
    f = make_model_folder(str(tmp_path / "a"), TINY_A, seed=0)
    exp = expected_tensors(Qwen3Config.from_dict(TINY_A))
    assert "lm_head.weight" not in exp
    load_tensors(f, exp, torch.bfloat16, "cpu")


def test_one_error_lists_everything(folder):
    def damage(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.extra.weight"] = torch.zeros(3)
        t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 95, dtype=torch.bfloat16)
        t["model.layers.2.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int32)
    _rewrite(folder, damage)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, expected_tensors(Qwen3Config.from_dict(TINY_B)), torch.bfloat16, "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "[64, 95]" in msg and "[64, 96]" in msg
    assert "wrong dtypes (1)" in msg and "I32" in msg


def test_tensor_stored_in_32_bit_stays_32_bit(folder):
    _rewrite(folder, lambda t: t.update({"model.norm.weight": t["model.norm.weight"].float()}))
    exp = expected_tensors(Qwen3Config.from_dict(TINY_B))
    t = load_tensors(folder, exp, torch.bfloat16, "cpu")
    assert t["model.norm.weight"].dtype == torch.float32
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_sharded_checkpoint(folder):
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    names = sorted(t)
    half = len(names) // 2
    save_file({n: t[n] for n in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({n: t[n] for n in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    os.unlink(path)
    wm = {n: "model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors"
          for i, n in enumerate(names)}
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    exp = expected_tensors(Qwen3Config.from_dict(TINY_B))
    got = load_tensors(folder, exp, torch.bfloat16, "cpu")
    assert all(torch.equal(got[n], t[n]) for n in names)


def test_no_checkpoint(tmp_path):
    with pytest.raises(WeightError, match="neither"):
        load_tensors(str(tmp_path), {}, torch.bfloat16, "cpu")


def test_random_weights_are_deterministic_and_seeded(tmp_path):
    exp = expected_tensors(Qwen3Config.from_dict(TINY_A))
    a, b, c = random_tensors(exp, 5), random_tensors(exp, 5), random_tensors(exp, 6)
    assert all(torch.equal(a[n], b[n]) for n in exp)
    assert any(not torch.equal(a[n], c[n]) for n in exp)
    w = a["model.layers.0.mlp.down_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.003 and abs(w.mean().item()) < 0.002
    n = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.02
    # a tensor's values do not depend on which other tensors exist
    sub = {k: exp[k] for k in list(exp)[:3]}
    s = random_tensors(sub, 5)
    assert all(torch.equal(s[k], a[k]) for k in sub)


def test_tensors_nobody_asked_for_are_ignored_unless_strict(tmp_path):
    """A tied model whose file still stores lm_head.weight, and a file with rotary inv_freq buffers, load:
    the reference looks tensors up by name and never reads the rest (pegainfer-core/src/weight_loader.rs:251-269,
    pegainfer-qwen3/src/weights/load.rs:85-91). ``strict`` refuses them; any other fault still names them."""
    f = make_model_folder(str(tmp_path / "a"), TINY_A, seed=0)
    before = {n: v.clone() for n, v in load_file(os.path.join(f, "model.safetensors")).items()}  # the file is rewritten below

    def extras(t):
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    _rewrite(f, extras)
    exp = expected_tensors(Qwen3Config.from_dict(TINY_A))
    ignored = []
    got = load_tensors(f, exp, torch.bfloat16, "cpu", ignored=ignored)
    assert ignored == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert set(got) == set(exp) and all(torch.equal(got[n], before[n]) for n in exp)
    with pytest.raises(WeightError, match=r"unexpected tensors \(2\)"):
        load_tensors(f, exp, torch.bfloat16, "cpu", strict=True)
    _rewrite(f, lambda t: t.pop("model.norm.weight"))
    with pytest.raises(WeightError) as e:
        load_tensors(f, exp, torch.bfloat16, "cpu")
    assert "missing tensors (1)" in str(e.value) and "unexpected tensors (2)" in str(e.value)
