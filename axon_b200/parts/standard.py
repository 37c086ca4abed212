"""The parts the Qwen2 decoder is made of: RMSNorm, rotary position encoding,
grouped-query attention over the paged cache, the SwiGLU feed-forward, the pre-norm
block, the embedding and the linear head.

Formulas are the reference's (each docstring cites them); the code here only
orders kernel launches.  Sizes and constants come from ``spec.params``.
"""

from __future__ import annotations

import math
from typing import Any, Callable, Dict, Optional

import torch

from ..kernels import linear as _linear
from ..kernels import ops
from .base import FeedForward, Mixer, Part, Runtime, StepContext, fold_owed, norm_owed, register_part
from .spec import KvNeed, PartSpec, TensorDecl


@register_part
class RMSNorm(Part):
    """``h = x * rsqrt(mean(x^2) + eps) * gain`` in float32 (src/model.rs:3888-3898).

    params: ``size``, ``eps``; optional ``unit_offset`` (gain stored as ``w``, applied
    as ``1 + w``).  tensors: ``gain [size]``.
    """

    category, kind = "norm", "rmsnorm"
    graph_safe = True
    folds_owed = True

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {"gain": TensorDecl((spec.params["size"],), "gain")}

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.unit_offset = bool(spec.params.get("unit_offset", False))
        self.gain = tensors["gain"]

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None, pending=None) -> None:
        ops.rmsnorm(x, self.gain, out, self.eps, rows=rows, unit_offset=self.unit_offset, pending=pending)


@register_part
class RotaryEncoding(Part):
    """Rotary position encoding: ``freq_i = theta^(-2i/rot)`` and the angle
    ``pos * freq_i`` in float64, (cos, sin) rounded to float32 once
    (src/model.rs:638-657, 2612-2621).  Pairs ``(i, i + rot/2)`` when ``pairing`` is
    ``"half"`` (src/model.rs:3922-3929), ``(2i, 2i+1)`` when ``"adjacent"``.

    params: ``head_dim``, ``theta``, ``pairing``; optional ``rot`` (rotated elements of
    a head, default all) and ``magnitude`` (scale of cos and sin, default 1).
    """

    category, kind = "position", "rope"
    graph_safe = True

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rot = int(p.get("rot") or self.head_dim)
        self.theta = float(p["theta"])
        self.magnitude = float(p.get("magnitude", 1.0))
        pairing = p.get("pairing", "half")
        if pairing not in ("half", "adjacent"):
            raise ValueError(f"rope pairing '{pairing}' is not 'half' or 'adjacent'")
        self.adjacent = pairing == "adjacent"
        if self.rot % 2 or self.rot > self.head_dim or self.rot <= 0:
            raise ValueError(f"rope rotates an even number of elements up to the head size, not {self.rot}")
        half = self.rot // 2
        inv = [self.theta ** (-2.0 * i / self.rot) for i in range(half)]
        self.inv_freq = torch.tensor(inv, dtype=torch.float64, device=rt.device)
        self._key = ("rope", self.rot, self.theta, self.magnitude)

    def rotation(self, ctx: StepContext) -> torch.Tensor:
        """The step's (cos, sin) table ``[n, rot/2, 2]``; computed once per step and
        shared by every layer with the same parameters."""
        t = ctx.scratch.get(self._key)
        if t is None:
            t = self.rt.buffer(f"rope_table_{self.rot}_{self.theta}_{self.magnitude}",
                               (ctx.n_tokens, self.rot // 2, 2), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, t, self.magnitude)
            ctx.scratch[self._key] = t
        return t


@register_part
class Attention(Mixer):
    """Causal grouped-query attention over the paged cache.

    ``q = Wq h + bq`` (and k, v), q and k rotated after the bias, K stored rotated and V
    as is (src/model.rs:2982-3007); query head ``qh`` reads kv head ``qh // (H / Hkv)``;
    ``softmax(q.k / sqrt(head_dim))`` over positions ``0..pos`` (the last ``window`` of
    them when a window is set), all in float32; ``x += Wo o`` (src/model.rs:3354-3463,
    3031-3038).

    params: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``qkv_bias``,
    ``out_bias``, ``window`` (None = all), ``scale`` (None = 1/sqrt(head_dim)).
    nested: ``position`` (may be absent).  tensors: ``q k v o`` and the biases.
    """

    category, kind = "mixer", "attention"
    graph_safe = True
    may_defer = True
    nested = {"position": "position"}

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        p = spec.params
        d, q, kv = p["hidden_size"], p["heads"] * p["head_dim"], p["kv_heads"] * p["head_dim"]
        t = {"q": TensorDecl((q, d)), "k": TensorDecl((kv, d)), "v": TensorDecl((kv, d)),
             "o": TensorDecl((d, q))}
        if p.get("qkv_bias"):
            t.update({"q_bias": TensorDecl((q,), "bias"), "k_bias": TensorDecl((kv,), "bias"),
                      "v_bias": TensorDecl((kv,), "bias")})
        if p.get("out_bias"):
            t["o_bias"] = TensorDecl((d,), "bias")
        return t

    @classmethod
    def cache_need(cls, spec: PartSpec) -> KvNeed:
        p = spec.params
        return KvNeed(int(p["kv_heads"]), int(p["head_dim"]), p.get("window") or None)

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads, self.head_dim = int(p["heads"]), int(p["kv_heads"]), int(p["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads do not split over {self.kv_heads} kv heads")
        self.q_dim, self.kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(p.get("window") or 0)
        # one product for q, k and v: rows [Wq; Wk; Wv]
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.b_qkv = (torch.cat([tensors["q_bias"], tensors["k_bias"], tensors["v_bias"]]).contiguous()
                      if p.get("qkv_bias") else None)
        self.w_o = tensors["o"]
        self.b_o = tensors.get("o_bias") if p.get("out_bias") else None
        self.position = build(spec.parts["position"]) if "position" in spec.parts else None

    def graph_key(self, ctx: StepContext):
        """The split count of the decode-shape attention, which follows the longest context among
        the segments short enough for that shape (every segment, in a step of single tokens)."""
        if self.rt.precise:
            return ()
        from ..kernels import fast
        group = self.heads // self.kv_heads
        fits = 16 // group if group <= 16 else 0
        short = [kv for n, kv in zip(ctx.seg_q_len, ctx.seg_kv_len) if n <= fits]
        if not short:
            return ()
        return (("key_splits", fast.decode_split_count(len(short), self.kv_heads, max(short))),)

    def forward(self, h, x, ctx: StepContext, cache: ops.KvView, write_cache: bool = True, defer: bool = False):
        rt, n = self.rt, ctx.n_tokens
        qkv = rt.buffer("qkv", (n, self.q_dim + 2 * self.kv_dim), torch.float32)
        # a product split over K leaves its partial sums to the kernel that reads its output
        owed = _linear.linear(h, self.w_qkv, qkv, bias=self.b_qkv, precise=rt.precise, defer=True)
        table, rot, adjacent = None, 0, False
        if self.position is not None:
            table, rot, adjacent = self.position.rotation(ctx), self.position.rot, self.position.adjacent
        att = rt.buffer("att", (n, self.q_dim))
        # steps of single tokens: rotation, cache write and attention in one kernel
        if not _linear.attention_decode_fused(qkv, owed, table, rot, adjacent, cache, ctx, att, self.heads, self.scale,
                                              write_cache, precise=rt.precise):
            q = rt.buffer("q", (n, self.q_dim))
            ops.rope_kv_write(qkv, table, ctx.positions, ctx.token_slot, q, cache, self.heads, rot, adjacent,
                              write_kv=write_cache, pending=owed)
            _linear.attention(q, cache, ctx, att, self.heads, self.scale, precise=rt.precise)
        return _linear.linear(att, self.w_o, x, bias=self.b_o, accumulate=True, precise=rt.precise, defer=defer)


@register_part
class SwiGLU(FeedForward):
    """``x += Wd (silu(Wg h) * (Wu h))`` with ``silu(g) = g / (1 + exp(-g))``
    (src/vmath.rs:128-132, src/model.rs:3043-3055).  Gate and up rows are interleaved
    at load (row 2j gate, 2j+1 up) so that one product yields both and a fused
    epilogue sees each pair together.

    params: ``hidden_size``, ``intermediate_size``.  tensors: ``gate up down``.
    """

    category, kind = "ffn", "swiglu"
    graph_safe = True
    may_defer = True

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        d, f = spec.params["hidden_size"], spec.params["intermediate_size"]
        return {"gate": TensorDecl((f, d)), "up": TensorDecl((f, d)), "down": TensorDecl((d, f))}

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        self.hidden, self.ffn = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        self.w_gate_up = torch.stack([tensors["gate"], tensors["up"]], dim=1).reshape(2 * self.ffn, self.hidden).contiguous()
        self.w_down = tensors["down"]

    def forward(self, h, x, ctx: StepContext, defer: bool = False):
        rt, n = self.rt, h.shape[0]
        act = rt.buffer("ffn_act", (n, self.ffn))
        _linear.linear_swiglu(h, self.w_gate_up, act, rt)
        return _linear.linear(act, self.w_down, x, accumulate=True, precise=rt.precise, defer=defer)


@register_part
class PreNormBlock(Part):
    """``x += mixer(norm_mixer(x)); x += ffn(norm_ffn(x))`` with a float32 residual
    (src/model.rs:2955-3060)."""

    category, kind = "block", "prenorm"
    graph_safe = True
    passes_owed = True
    nested = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        self.norm_mixer = build(spec.parts["norm_mixer"])
        self.mixer = build(spec.parts["mixer"])
        self.norm_ffn = build(spec.parts["norm_ffn"])
        self.ffn = build(spec.parts["ffn"])

    def graph_key(self, ctx: StepContext):
        return self.norm_mixer.graph_key(ctx) + self.mixer.graph_key(ctx) + self.norm_ffn.graph_key(ctx) + self.ffn.graph_key(ctx)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any, write_cache: bool = True, pending=None):
        """``pending``: what ``x`` is still owed on entry; returns what it is owed on exit."""
        h = self.rt.buffer("block_h", tuple(x.shape))
        norm_owed(self.norm_mixer, x, h, pending)
        if self.mixer.may_defer:
            owed = self.mixer.forward(h, x, ctx, cache, write_cache, defer=True)
        else:
            owed = self.mixer.forward(h, x, ctx, cache, write_cache)
        norm_owed(self.norm_ffn, x, h, owed)
        if self.ffn.may_defer:
            return self.ffn.forward(h, x, ctx, defer=True)
        self.ffn.forward(h, x, ctx)
        return None


@register_part
class Embedding(Part):
    """``x = E[token]`` widened to float32, times ``scale`` when one is set
    (src/model.rs:2657-2675).  params: ``vocab_size``, ``hidden_size``; tensors: ``table``."""

    category, kind = "embedding", "embedding"
    graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {"table": TensorDecl((spec.params["vocab_size"], spec.params["hidden_size"]), "table")}

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        self.table = tensors["table"]
        self.scale = float(spec.params.get("scale") or 1.0)

    def forward(self, tokens: torch.Tensor, x: torch.Tensor) -> None:
        ops.embed(tokens, self.table, x, self.scale)


@register_part
class LinearHead(Part):
    """``logits = W h`` in float32, no bias (src/model.rs:2640-2645).
    params: ``vocab_size``, ``hidden_size``; tensors: ``weight``."""

    category, kind = "head", "linear_head"
    graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.params["vocab_size"], spec.params["hidden_size"]), "table")}

    def __init__(self, spec, tensors, rt, build):
        super().__init__(spec, tensors, rt, build)
        self.weight = tensors["weight"]

    def forward(self, h: torch.Tensor, logits: torch.Tensor) -> None:
        _linear.linear(h, self.weight, logits, precise=self.rt.precise)
