"""Configuration and registry: keys, defaults, refusals (reference: src/safetensors.rs:609-727,
src/model.rs:1272-1420)."""

import json

import pytest

from axon_b200.config import (ConfigError, Qwen2Config, architecture_of, config_from_dict,
                              known_architectures, load_config, qwen2_spec)
from conftest import TINY_A, TINY_B


def test_reads_every_key():
    c = config_from_dict(TINY_B)
    assert isinstance(c, Qwen2Config)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 256, 384)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5
    assert c.tie_word_embeddings is False and c.max_position_embeddings == 256


def test_defaults():
    cfg = {k: v for k, v in TINY_A.items()
           if k not in ("head_dim", "rope_theta", "rms_norm_eps", "tie_word_embeddings", "num_key_value_heads")}
    c = config_from_dict(cfg)
    assert c.head_dim == 64 // 4            # hidden_size / heads (src/model.rs:1297-1305)
    assert c.rope_theta == 10000.0          # src/model.rs:639
    assert c.rms_norm_eps == 1e-6           # src/model.rs:1784
    assert c.tie_word_embeddings is False
    assert c.num_key_value_heads == 4


def test_registry_resolution():
    assert "Qwen2ForCausalLM" in known_architectures()
    assert architecture_of({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    assert architecture_of({"architectures": ["Qwen2ForCausalLM"]}).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="not supported"):
        architecture_of({"model_type": "gemma3", "architectures": ["Qwen2ForCausalLM"]})
    with pytest.raises(ConfigError, match="FooForCausalLM"):
        architecture_of({"architectures": ["FooForCausalLM"]})


@pytest.mark.parametrize("patch,match", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"num_hidden_layers": 2.5}, "whole number"),
    ({"num_hidden_layers": 0}, "whole number"),
    ({"hidden_size": -64}, "whole number"),
    ({"num_attention_heads": True}, "whole number"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "odd"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "RoPE scaling"),
    ({"rope_theta": "big"}, "not a number"),
    ({"rope_theta": -1.0}, "positive"),
    ({"tie_word_embeddings": "yes"}, "true or false"),
    ({"quantization_config": {"quant_method": "fp8"}}, "quantized"),
    ({"num_experts": 8}, "experts"),
])
def test_refusals(patch, match):
    cfg = dict(TINY_A)
    cfg.update(patch)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(cfg)


def test_missing_key_is_named():
    cfg = dict(TINY_A)
    del cfg["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(cfg)


def test_hidden_not_divisible_needs_head_dim():
    cfg = dict(TINY_A, hidden_size=66)
    del cfg["head_dim"]
    with pytest.raises(ConfigError, match="split"):
        config_from_dict(cfg)
    assert config_from_dict(dict(cfg, head_dim=16)).head_dim == 16   # Q may differ from D


def test_rope_parameters_of_newer_configs():
    cfg = dict(TINY_A)
    del cfg["rope_theta"]
    cfg["rope_parameters"] = {"rope_type": "default", "rope_theta": 123456.0}
    assert config_from_dict(cfg).rope_theta == 123456.0


def test_round_trip_through_json(tmp_path):
    c = config_from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError, match="not a JSON object"):
        load_config(str(tmp_path))


def test_spec_is_data_and_layerwise():
    a, b = qwen2_spec(config_from_dict(TINY_A)), qwen2_spec(config_from_dict(TINY_B))
    assert len(a.layers) == 2 and len(b.layers) == 3
    assert [e.layer for e in b.schedule] == [0, 1, 2]
    m = b.layers[1].parts["mixer"]
    assert m.kind == "attention" and m.params["kv_heads"] == 1 and m.params["head_dim"] == 32
    assert m.parts["position"].params["theta"] == 1e6
    assert m.weights["q_bias"] == "model.layers.1.self_attn.q_proj.bias"
    # tied head reads the embedding table, untied one its own tensor
    assert a.head.weights["weight"] == "model.embed_tokens.weight"
    assert b.head.weights["weight"] == "lm_head.weight"
    assert a.final_norm.params["eps"] == 1e-6 and b.final_norm.params["eps"] == 1e-5
