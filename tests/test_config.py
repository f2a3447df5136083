"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from helpers import TINY_A, TINY_B
from openinfer_b200.config import (ConfigError, ModelConfig, Qwen3Config, known_architectures, load_config,
                                   register_architecture, resolve_architecture, unregister_architecture)


def write(tmp_path, cfg, gen=None):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    if gen is not None:
        (tmp_path / "generation_config.json").write_text(json.dumps(gen))
    return str(tmp_path)


def test_reads_every_key(tmp_path):
    cfg = load_config(write(tmp_path, dict(TINY_B, eos_token_id=7)))
    assert isinstance(cfg, Qwen3Config)
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "vocab_size", "rms_norm_eps", "rope_theta",
                "tie_word_embeddings", "max_position_embeddings"):
        assert getattr(cfg, key) == TINY_B[key]
    assert cfg.q_dim == 6 * 32 and cfg.kv_dim == 2 * 32 and cfg.q_dim != cfg.hidden_size
    assert cfg.stop_token_ids == (7,)


def test_default_max_positions_and_unknown_keys_ignored(tmp_path):
    raw = dict(TINY_A, sliding_window=77, rope_scaling={"type": "yarn"}, attention_bias=True)
    raw.pop("max_position_embeddings")
    cfg = load_config(write(tmp_path, raw))
    assert cfg.max_position_embeddings == 40960
    assert not hasattr(cfg, "sliding_window")


@pytest.mark.parametrize("key", ["hidden_size", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings",
                                 "num_key_value_heads", "vocab_size", "intermediate_size"])
def test_missing_required_key(tmp_path, key):
    raw = dict(TINY_A)
    raw.pop(key)
    with pytest.raises(ConfigError, match=key):
        load_config(write(tmp_path, raw))


def test_wrong_types_and_values(tmp_path):
    with pytest.raises(ConfigError, match="hidden_size"):
        load_config(write(tmp_path, dict(TINY_A, hidden_size="64")))
    with pytest.raises(ConfigError, match="tie_word_embeddings"):
        load_config(write(tmp_path, dict(TINY_A, tie_word_embeddings=1)))
    with pytest.raises(ConfigError, match="multiple"):
        load_config(write(tmp_path, dict(TINY_A, num_attention_heads=5)))
    with pytest.raises(ConfigError, match="head_dim"):
        load_config(write(tmp_path, dict(TINY_A, head_dim=15)))
    with pytest.raises(ConfigError, match="positive"):
        load_config(write(tmp_path, dict(TINY_A, num_hidden_layers=0)))


def test_generation_config_stop_ids_win(tmp_path):
    cfg = load_config(write(tmp_path, dict(TINY_A, eos_token_id=3), gen={"eos_token_id": [9, 11, 9]}))
    assert cfg.stop_token_ids == (9, 11)
    cfg = load_config(write(tmp_path, dict(TINY_A, eos_token_id=3), gen={"eos_token_id": 5}))
    assert cfg.stop_token_ids == (5,)


def test_registry_unknown_and_mismatch(tmp_path):
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="no registered architecture"):
        load_config(write(tmp_path, dict(TINY_A, architectures=["LlamaForCausalLM"])))
    with pytest.raises(ConfigError, match="model_type"):
        load_config(write(tmp_path, dict(TINY_A, model_type="llama")))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "nowhere"))


def test_round_trip_and_registration(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_B)
    cfg.save(str(tmp_path))
    assert load_config(str(tmp_path)) == cfg
    raw = json.loads((tmp_path / "config.json").read_text())
    assert raw["architectures"] == ["Qwen3ForCausalLM"] and raw["model_type"] == "qwen3"

    import dataclasses

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "ToyForTests"
        model_type = "toy"
        width: int

    register_architecture("ToyForTests", ToyConfig, lambda c: None)
    try:
        entry = resolve_architecture({"architectures": ["ToyForTests"], "model_type": "toy"})
        assert entry.config_cls is ToyConfig
        with pytest.raises(ConfigError, match="several"):
            resolve_architecture({"architectures": ["ToyForTests", "Qwen3ForCausalLM"]})
    finally:
        unregister_architecture("ToyForTests")


def test_spec_has_no_constants_of_its_own():
    """Every size of the spec comes from the config: two configs give specs that differ everywhere."""
    from openinfer_b200.models.qwen3 import build_spec

    a, b = build_spec(Qwen3Config.from_dict(TINY_A)), build_spec(Qwen3Config.from_dict(TINY_B))
    ma, mb = a.blocks[0].mixer, b.blocks[0].mixer
    for f in ("hidden_size", "num_heads", "head_dim", "softmax_scale"):
        assert getattr(ma, f) != getattr(mb, f)
    assert ma.position.theta != mb.position.theta and ma.qk_norm.eps != mb.qk_norm.eps
    assert a.blocks[0].feed_forward.intermediate_size != b.blocks[0].feed_forward.intermediate_size
    assert a.head_name is None and b.head_name == "lm_head.weight"
    assert len(a.blocks) == 2 and len(b.blocks) == 3 and a.vocab_size != b.vocab_size
