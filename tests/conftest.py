"""Shared fixtures: the tiny configurations, model folders made in temporary
folders, and the ``gpu`` marker."""

from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations that differ in every size and option: layers, width, heads,
# kv heads (grouped vs. a single kv head), head size, feed-forward width (no multiple of
# the width), vocabulary (no power of two for B), theta, eps, tying, context.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "use_sliding_window": False, "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "use_sliding_window": False, "hidden_act": "silu",
}
# A third one with the head size of the large models (128): 6 heads over 2 kv heads,
# widths and vocabulary that are no powers of two.
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 344, "vocab_size": 1000, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 1024,
    "use_sliding_window": False, "hidden_act": "silu",
}
# A fourth one whose sizes no tuned kernel takes: head size 48, a width that is no multiple of
# 8 (rows that are no whole 16-byte pieces), as many kv heads as heads, a prime vocabulary.
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 132, "vocab_size": 211, "rope_theta": 200000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 160,
    "use_sliding_window": False, "hidden_act": "silu",
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def make_model_folder(path: str, cfg: dict, seed: int, sharpen: float = 6.0) -> str:
    """A seeded random model folder.  With N(0, 0.02) weights every attention score is
    close to zero, softmax is nearly uniform, and faults in positions, rotation, pages or
    windows barely move the logits; so the query and key projections are scaled by
    ``sharpen`` (scores by its square), which makes single keys stand out."""
    from safetensors.torch import load_file

    from axon_b200.config import config_from_dict
    from axon_b200.weights import write_random_model, write_safetensors

    write_random_model(path, config_from_dict(cfg), seed)
    if sharpen != 1.0:
        f = os.path.join(path, "model.safetensors")
        t = load_file(f)
        for k in list(t):
            if ".q_proj." in k or ".k_proj." in k:
                t[k] = (t[k].float() * sharpen).to(t[k].dtype)
        write_safetensors(f, t, {"format": "pt"})
    return path


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """{"A": folder, "B": folder, "C": folder}: seeded random models (bfloat16 weights)."""
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        out[name] = make_model_folder(str(tmp_path_factory.mktemp(f"tiny_{name}")), cfg, 1234 + i)
    return out
