"""A plain, slow Qwen2 decoder for tests: whole sequences, no cache, one function per
part, float64 on the CPU.  It shares no code with ``axon_b200``: it reads
``config.json`` with ``json`` and the weights with the ``safetensors`` package, and is
written from the formulas of the reference implementation, which each function cites
by ``file:line`` within that project.

The reference's own model code (Rust) cannot be compiled or imported here (no Rust
toolchain is available), so this file rests on the formulas, most compactly stated in
the reference's test oracle ``dense_ref`` (src/model.rs:4575-4834) plus the q/k/v
biases of ``Qwen2::hidden`` (src/model.rs:2983-2991).
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

DT = torch.float64


def read_model(folder: str):
    """(config dict, {name: float64 tensor}) of a model folder."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(DT) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


def embed(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x = E[token], no scaling for qwen2 (src/model.rs:2657-2675)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """h_i = x_i / sqrt(mean(x^2) + eps) * g_i (src/model.rs:3888-3898; dense_ref :4618-4622)."""
    inv = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return x * inv * gain


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[o] = row_o . x (+ b[o]); matrices are [out][in] (src/model.rs:2146, 2982-2991)."""
    y = x @ w.T
    return y if b is None else y + b


def rope_half(v: torch.Tensor, positions: Sequence[int], theta: float) -> torch.Tensor:
    """NEOX / rotate-half RoPE on ``v [T, heads, hd]``: freq_i = theta^(-2i/hd) for i < hd/2,
    angle = pos * freq_i; (a, b) = (v[i], v[i + hd/2]) -> (a cos - b sin, a sin + b cos)
    (src/model.rs:638-657, 2612-2621, 3922-3929; dense_ref :4644-4659)."""
    hd = v.shape[-1]
    half = hd // 2
    freq = torch.tensor([theta ** (-2.0 * i / hd) for i in range(half)], dtype=DT)
    ang = torch.tensor(list(positions), dtype=DT)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None,
                         scale: Optional[float] = None) -> torch.Tensor:
    """q [T, H, hd], k and v [T, Hkv, hd] -> [T, H, hd].  Query head qh reads kv head
    qh // (H / Hkv); s[t] = q.k_t / sqrt(hd) over positions 0..pos (the last ``window``
    of them when given); softmax; o = sum_t w_t v_t
    (src/model.rs:3354-3356, 3392, 3009-3013; src/vmath.rs:344-352; dense_ref :4768-4790)."""
    T, H, hd = q.shape
    Hkv = k.shape[1]
    group = H // Hkv
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    out = torch.zeros_like(q)
    for h in range(H):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale  # [T, T]
        idx = torch.arange(T)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask = mask | (idx[None, :] < idx[:, None] - window + 1)
        s = s.masked_fill(mask, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        w = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = w @ v[:, kh, :]
    return out


def swiglu_ffn(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """d = Wd (g / (1 + exp(-g)) * u), g = Wg h, u = Wu h
    (src/vmath.rs:128-132; src/model.rs:3043-3055; dense_ref :4794-4804)."""
    g, u = linear(h, gate), linear(h, up)
    return linear(g / (1.0 + torch.exp(-g)) * u, down)


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, positions: Sequence[int],
                    heads: int, kv_heads: int, hd: int, theta: float) -> torch.Tensor:
    """q, k, v with biases, RoPE on q and k after the bias, attention, output projection
    without bias (src/model.rs:2981-3038)."""
    T = h.shape[0]
    p = prefix + "self_attn."
    q = linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(T, heads, hd)
    k = linear(h, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(T, kv_heads, hd)
    v = linear(h, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(T, kv_heads, hd)
    q, k = rope_half(q, positions, theta), rope_half(k, positions, theta)
    o = causal_gqa_attention(q, k, v).reshape(T, heads * hd)
    return linear(o, w[p + "o_proj.weight"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] (float64) of a whole sequence (src/model.rs:2955-3060, 2640-2645)."""
    L, D, H = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads", H)
    hd = cfg.get("head_dim") or D // H
    theta = float(cfg.get("rope_theta", 10000.0))
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    positions = list(range(len(tokens)))
    x = embed(w["model.embed_tokens.weight"], tokens)
    for l in range(L):
        p = f"model.layers.{l}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_block(h, w, p, positions, H, Hkv, hd, theta)
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    h = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head)


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """n greedy tokens after the prompt; the last index wins among equal maxima
    (src/generate.rs:222-263)."""
    ids = list(prompt)
    out = []
    for _ in range(n):
        row = forward(cfg, w, ids)[-1]
        best = int((row == row.max()).nonzero().max())
        out.append(best)
        ids.append(best)
    return out
