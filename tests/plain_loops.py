"""A second plain statement of the Qwen2 decoder, independent of ``plain_qwen2.py``: numpy
float64, one token at a time with growing lists of keys and values, explicit loops over
heads, positions and rotation pairs, and a reader of its own for ``config.json`` and
``model.safetensors`` (``json`` and ``numpy.frombuffer`` only).  It shares no code with the
product or with the first plain implementation; the two are compared to 1e-10 in
``test_plain.py``, so a slip in either one's reading of the formulas shows.

Written from the reference's formulas in the order its float64 test oracle walks them
(``dense_ref``, src/model.rs:4743-4834: per token, per layer; rms and matrix-vector
products :4614-4622, rotation of pairs (i, i + hd/2) :4644-4659, scores over all earlier
positions, softmax and the weighted sum of values :4768-4790, SwiGLU :4794-4804, final
norm and head :4830-4831) plus the q/k/v biases of the model proper (src/model.rs:2983-2991).
The reference's own code cannot be compiled here (no Rust toolchain), so this file too
rests on the formulas.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Sequence

import numpy as np


def _bf16_to_f64(raw: bytes) -> np.ndarray:
    """bfloat16 is the upper half of a float32."""
    u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32)
    return (u16 << 16).view(np.float32).astype(np.float64)


def read_folder(folder: str):
    """(config dict, {name: float64 array}) from config.json and model.safetensors."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    data = blob[8 + hlen:]
    out: Dict[str, np.ndarray] = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        b, e = rec["data_offsets"]
        raw = data[b:e]
        if rec["dtype"] == "BF16":
            a = _bf16_to_f64(raw)
        elif rec["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif rec["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {rec['dtype']}")
        out[name] = a.reshape(rec["shape"])
    return cfg, out


def _rms(x: np.ndarray, g: np.ndarray, eps: float) -> np.ndarray:
    ss = 0.0
    for v in x:
        ss += v * v
    inv = 1.0 / math.sqrt(ss / len(x) + eps)
    return np.array([v * inv * gi for v, gi in zip(x, g)])


def _mv(w: np.ndarray, x: np.ndarray) -> np.ndarray:
    """y[o] = row_o . x (src/model.rs:2146)."""
    return np.array([float(np.dot(row, x)) for row in w])


def _rotate(v: np.ndarray, pos: int, hd: int, theta: float) -> None:
    """In place, head by head: the pair (i, i + hd/2) turns by pos * theta^(-2i/hd)."""
    half = hd // 2
    for h0 in range(0, len(v), hd):
        for i in range(half):
            ang = pos * theta ** (-2.0 * i / hd)
            c, s = math.cos(ang), math.sin(ang)
            a, b = v[h0 + i], v[h0 + i + half]
            v[h0 + i] = a * c - b * s
            v[h0 + i + half] = a * s + b * c


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    """Logits [T, V] (float64) of the sequence, computed token by token."""
    L, D, H = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads", H)
    hd = cfg.get("head_dim") or D // H
    theta = float(cfg.get("rope_theta", 10000.0))
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    group = H // Hkv
    keys: List[List[np.ndarray]] = [[] for _ in range(L)]
    values: List[List[np.ndarray]] = [[] for _ in range(L)]
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    logits = []
    for pos, tok in enumerate(tokens):
        x = w["model.embed_tokens.weight"][tok].copy()
        for l in range(L):
            p = f"model.layers.{l}."
            h = _rms(x, w[p + "input_layernorm.weight"], eps)
            q = _mv(w[p + "self_attn.q_proj.weight"], h) + w[p + "self_attn.q_proj.bias"]
            k = _mv(w[p + "self_attn.k_proj.weight"], h) + w[p + "self_attn.k_proj.bias"]
            v = _mv(w[p + "self_attn.v_proj.weight"], h) + w[p + "self_attn.v_proj.bias"]
            _rotate(q, pos, hd, theta)
            _rotate(k, pos, hd, theta)
            keys[l].append(k)
            values[l].append(v)
            att = np.zeros(H * hd)
            for qh in range(H):
                kh = qh // group
                qv = q[qh * hd:(qh + 1) * hd]
                sc = [float(np.dot(qv, kr[kh * hd:(kh + 1) * hd])) / math.sqrt(hd) for kr in keys[l]]
                mx = max(sc)
                e = [math.exp(s - mx) for s in sc]
                z = sum(e)
                for t, pt in enumerate(e):
                    att[qh * hd:(qh + 1) * hd] += pt / z * values[l][t][kh * hd:(kh + 1) * hd]
            x = x + _mv(w[p + "self_attn.o_proj.weight"], att)
            h = _rms(x, w[p + "post_attention_layernorm.weight"], eps)
            g = _mv(w[p + "mlp.gate_proj.weight"], h)
            u = _mv(w[p + "mlp.up_proj.weight"], h)
            act = np.array([gi / (1.0 + math.exp(-gi)) * ui for gi, ui in zip(g, u)])
            x = x + _mv(w[p + "mlp.down_proj.weight"], act)
        logits.append(_mv(head, _rms(x, w["model.norm.weight"], eps)))
    return np.stack(logits)
