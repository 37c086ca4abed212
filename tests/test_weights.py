"""Weights: the safetensors reader on malformed files, the loader's single error that
lists everything wrong, dtypes kept, and the random-weights mode
(reference cases: src/safetensors_tests.rs:611-806)."""

import json
import os
import struct

import pytest
import torch

from axon_b200.config import config_from_dict, qwen2_spec
from axon_b200.weights import (Checkpoint, SafetensorsError, WeightsError, expected_tensors, load_weights,
                               write_random_model, write_safetensors)
from conftest import TINY_A, TINY_B


def _write_raw(path, header: dict, data: bytes = b""):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)


def test_round_trip_agrees_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(4), "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, t)
    theirs = load_file(p)
    ck = Checkpoint(str(tmp_path))
    for k, v in t.items():
        assert torch.equal(theirs[k], v)
        assert torch.equal(ck.tensor(k), v)
    ck.close()


@pytest.mark.parametrize("header,data,match", [
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 16]}}, b"\0" * 8, "outside the file"),
    ({"x": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8, "do not hold shape"),
    ({"x": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, "dtype"),
    ({"x": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, b"\0" * 8, "shape"),
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}, b"\0" * 8, "outside|offsets"),
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
      "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12, "overlap"),
    ({"x": [1, 2]}, b"", "not an object"),
])
def test_malformed_headers(tmp_path, header, data, match):
    _write_raw(tmp_path / "model.safetensors", header, data)
    with pytest.raises(SafetensorsError, match=match):
        Checkpoint(str(tmp_path))


def test_truncated_and_oversized_header(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        Checkpoint(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        Checkpoint(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not JSON"):
        Checkpoint(str(tmp_path))


def test_no_checkpoint(tmp_path):
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        Checkpoint(str(tmp_path))


def test_shards_and_duplicates(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.zeros(2)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.ones(3)})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    ck = Checkpoint(str(tmp_path))
    assert sorted(ck.names()) == ["a", "b"] and torch.equal(ck.tensor("b"), torch.ones(3))
    ck.close()
    # the index names a tensor its shard lacks
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "zz": "s2.safetensors"}}))
    with pytest.raises(SafetensorsError, match="does not hold"):
        Checkpoint(str(tmp_path))
    # the same tensor in two shards
    write_safetensors(str(tmp_path / "s2.safetensors"), {"a": torch.ones(2), "b": torch.ones(3)})
    (tmp_path / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    with pytest.raises(SafetensorsError, match="is in"):
        Checkpoint(str(tmp_path))


def test_expected_tensors_follow_the_spec():
    a = expected_tensors(qwen2_spec(config_from_dict(TINY_A)))
    b = expected_tensors(qwen2_spec(config_from_dict(TINY_B)))
    assert "lm_head.weight" not in a and b["lm_head.weight"].shape == (384, 96)
    assert a["model.layers.1.self_attn.k_proj.weight"].shape == (2 * 16, 64)
    assert b["model.layers.2.self_attn.q_proj.bias"].shape == (3 * 32,)
    assert b["model.layers.0.mlp.down_proj.weight"].shape == (96, 256)
    assert len(a) == 1 + 2 * 12 + 1 and len(b) == 1 + 3 * 12 + 2


def test_random_model_loads_and_keeps_dtypes(tmp_path):
    cfg = config_from_dict(TINY_B)
    write_random_model(str(tmp_path), cfg, seed=7)
    spec = qwen2_spec(cfg)
    w = load_weights(str(tmp_path), spec, torch.bfloat16, "cpu")
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16     # matrices stay bfloat16
    assert w["model.layers.0.input_layernorm.weight"].dtype == torch.float32  # vectors are widened
    assert w["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    w32 = load_weights(str(tmp_path), spec, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["lm_head.weight"], w["lm_head.weight"].float())   # widening is exact
    # statistics of the init: N(0, 0.02) weights, gains 1 + N(0, 0.1)
    m = w32["model.layers.1.mlp.gate_proj.weight"]
    assert abs(m.std().item() - 0.02) < 0.002 and abs(m.mean().item()) < 0.002
    g = w32["model.layers.1.input_layernorm.weight"]
    assert abs(g.mean().item() - 1.0) < 0.05 and 0.05 < g.std().item() < 0.15
    # same seed, same bytes; another seed, other bytes
    other = tmp_path / "again"
    write_random_model(str(other), cfg, seed=7)
    assert (other / "model.safetensors").read_bytes() == (tmp_path / "model.safetensors").read_bytes()
    write_random_model(str(other), cfg, seed=8)
    assert (other / "model.safetensors").read_bytes() != (tmp_path / "model.safetensors").read_bytes()


def test_a_tensor_stored_in_32_bit_stays_so(tmp_path):
    cfg = config_from_dict(TINY_A)
    write_random_model(str(tmp_path), cfg, seed=3, store_dtype=torch.float32)
    w = load_weights(str(tmp_path), qwen2_spec(cfg), torch.bfloat16, "cpu")
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32


def test_one_error_lists_everything(tmp_path):
    from safetensors.torch import load_file
    cfg = config_from_dict(TINY_A)
    write_random_model(str(tmp_path), cfg, seed=1)
    t = load_file(str(tmp_path / "model.safetensors"))
    del t["model.layers.0.self_attn.q_proj.bias"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)
    t["model.layers.1.mlp.up_proj.weight"] = torch.zeros(64, 192, dtype=torch.bfloat16)
    t["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.ones(8)   # skipped, not an error
    t["model.layers.1.mlp.down_proj.weight"] = torch.zeros(64, 192, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path), qwen2_spec(cfg), torch.bfloat16, "cpu")
    msg = str(e.value)
    assert e.value.missing == ["model.layers.0.self_attn.q_proj.bias", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert "model.layers.1.mlp.up_proj.weight: shape [64, 192] doesn't fit the model (expected [192, 64])" in msg
    assert "model.layers.1.mlp.down_proj.weight: dtype I32" in msg
    assert "inv_freq" not in msg


def test_untied_model_without_a_head_is_an_error(tmp_path):
    from safetensors.torch import load_file
    cfg = config_from_dict(TINY_B)
    write_random_model(str(tmp_path), cfg, seed=1)
    t = load_file(str(tmp_path / "model.safetensors"))
    del t["lm_head.weight"]
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightsError, match="lm_head.weight"):     # src/safetensors.rs:1608-1614
        load_weights(str(tmp_path), qwen2_spec(cfg), torch.bfloat16, "cpu")


def test_random_model_in_shards_reads_back_the_same(tmp_path):
    """A model written as several files with an index holds the bytes of the one-file model, and the
    loader reads both alike (shards and their index: src/safetensors.rs:347-430)."""
    import json
    cfg = config_from_dict(TINY_B)
    one, many = tmp_path / "one", tmp_path / "many"
    write_random_model(str(one), cfg, seed=4)
    write_random_model(str(many), cfg, seed=4, shards=3)
    files = sorted(p.name for p in many.iterdir())
    assert files == ["config.json", "model-00001-of-00003.safetensors", "model-00002-of-00003.safetensors",
                     "model-00003-of-00003.safetensors", "model.safetensors.index.json"]
    index = json.loads((many / "model.safetensors.index.json").read_text())
    spec = qwen2_spec(cfg)
    a = load_weights(str(one), spec, torch.bfloat16, "cpu")
    b = load_weights(str(many), spec, torch.bfloat16, "cpu")
    assert set(index["weight_map"]) == set(a) == set(b)
    assert all(torch.equal(a[k], b[k]) for k in a)
    sizes = [(many / f).stat().st_size for f in files if f.endswith(".safetensors")]
    assert max(sizes) < 2 * min(sizes), f"the shards are of very different sizes: {sizes}"
    assert index["metadata"]["total_size"] == sum(t.numel() * 2 for t in a.values() if t.dtype == torch.bfloat16) + \
        sum(t.numel() * 2 for t in a.values() if t.dtype == torch.float32)
