"""Configuration parsing, its errors, and the architecture registry."""

from __future__ import annotations

import pytest

from borrowed_compute_b200.architectures import architecture_names, register_architecture, resolve, unregister_architecture
from borrowed_compute_b200.config import ConfigError, LlamaConfig
from borrowed_compute_b200.engine.model import expected_tensors_for_config, model_for_config
from conftest import TINY_A, TINY_B


def test_defaults_follow_the_format():
    c = LlamaConfig.from_dict({"num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "intermediate_size": 100,
                               "vocab_size": 50})
    assert (c.num_key_value_heads, c.head_dim, c.rope_theta, c.rms_norm_eps, c.max_position_embeddings) == (4, 16, 10000.0, 1e-5, 4096)
    assert c.rope_scaling is None and not c.tie_word_embeddings and c.rope_pairing == "half" and c.eos_token_ids == ()
    assert c.q_dim == 64 and c.kv_dim == 64 and c.kv_bytes_per_token_layer(2) == 256


def test_every_key_is_read():
    a, b = LlamaConfig.from_dict(TINY_A), LlamaConfig.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 4, 1, 32)
    assert b.q_dim == 128 != b.hidden_size
    assert b.rope_scaling.factor == 4.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.tie_word_embeddings and b.rope_pairing == "adjacent" and b.eos_token_ids == (7, 300) and a.eos_token_ids == (255,)
    assert LlamaConfig.from_dict(b.to_dict()) == b and LlamaConfig.from_dict(a.to_dict()) == a


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_hidden_layers": "2"}, "num_hidden_layers"),
    ({"vocab_size": None}, "vocab_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "odd"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"rope_pairing": "spiral"}, "rope_pairing"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"eos_token_id": 9999}, "eos_token_id"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"hidden_size": 66, "head_dim": None}, "head_dim"),
])
def test_errors_name_the_key(change, match):
    cfg = dict(TINY_A)
    cfg.update(change)
    cfg = {k: v for k, v in cfg.items() if v is not None}
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(cfg)


def test_registry_resolves_by_name():
    assert "LlamaForCausalLM" in architecture_names()
    typed, model = model_for_config(TINY_B)
    assert isinstance(typed, LlamaConfig) and len(model.blocks) == 3
    with pytest.raises(ConfigError, match="Mystery"):
        resolve({"architectures": ["MysteryForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve({})
    register_architecture("MysteryForCausalLM", LlamaConfig.from_dict, resolve(TINY_A).model_spec)
    try:
        cfg = dict(TINY_A, architectures=["MysteryForCausalLM"])
        assert len(expected_tensors_for_config(cfg)) == len(expected_tensors_for_config(TINY_A))
    finally:
        unregister_architecture("MysteryForCausalLM")


def test_expected_tensors_follow_the_config():
    a, b = expected_tensors_for_config(TINY_A), expected_tensors_for_config(TINY_B)
    assert a["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert a["model.layers.0.mlp.down_proj.weight"].shape == (64, 176)
    assert a["lm_head.weight"].shape == (256, 64) and not a["lm_head.weight"].optional
    assert b["model.layers.2.self_attn.q_proj.weight"].shape == (128, 96)
    assert b["model.layers.2.self_attn.o_proj.weight"].shape == (96, 128)
    assert b["lm_head.weight"].optional                       # tied: the folder may or may not store it
    assert a["model.norm.weight"].role == "vector" and a["model.embed_tokens.weight"].role == "matrix"
    assert len(a) == 1 + 2 * 9 + 2 and len(b) == 1 + 3 * 9 + 2


def test_generation_config_adds_stop_ids(tmp_path):
    import json

    from borrowed_compute_b200.weights import read_generation_stop_ids

    assert read_generation_stop_ids(str(tmp_path), 100) == ()
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 9], "temperature": 0.6}))
    assert read_generation_stop_ids(str(tmp_path), 100) == (7, 9)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    assert read_generation_stop_ids(str(tmp_path), 100) == (5,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 100}))
    with pytest.raises(ConfigError, match="outside the vocabulary"):
        read_generation_stop_ids(str(tmp_path), 100)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(ConfigError, match="integer"):
        read_generation_stop_ids(str(tmp_path), 100)
