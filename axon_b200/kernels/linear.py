"""Which kernel runs a product or an attention call.

The 32-bit model (``precise``) always takes the plain FFMA kernels.  The bfloat16
model takes the tuned sm_100a kernels when they accept the sizes (each says what it
needs) and the plain templated kernels otherwise, so every size the configuration
allows gives a right result.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           accumulate: bool = False, precise: bool = False, defer: bool = False):
    """``out = a @ w.T (+ bias)``; ``accumulate`` adds into a float32 ``out``.

    With ``defer`` the caller promises to hand what this returns to the next reader of
    ``out``: None when ``out`` is complete, else a ``fast.PendingFold`` (the product was split
    over K and its partial sums wait in scratch; ``ops.rmsnorm`` and ``ops.rope_kv_write``
    fold them on their way, ``ops.fold_partials`` does it for any other reader)."""
    if not precise:
        from . import fast
        ran = fast.gemm(a, w, out, bias, accumulate, defer)
        if ran:
            return ran if isinstance(ran, fast.PendingFold) else None
    ops.gemm_plain(a, w, out, bias, accumulate)
    return None


def linear_swiglu(h: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, rt) -> None:
    """``act = silu(gate) * up`` of ``h @ w_gate_up.T`` with interleaved gate/up rows."""
    n = h.shape[0]
    if not rt.precise:
        from . import fast
        if fast.gemm_swiglu(h, w_gate_up, act):
            return
    gu = rt.buffer("gate_up", (n, w_gate_up.shape[0]), torch.float32)
    linear(h, w_gate_up, gu, precise=rt.precise)
    ops.swiglu(gu, act)


def attention(q: torch.Tensor, kv: ops.KvView, ctx, out: torch.Tensor, heads: int, scale: float,
              precise: bool = False) -> None:
    if not precise:
        from . import fast
        if fast.attention(q, kv, ctx, out, heads, scale):
            return
    ops.attention_plain(q, kv, ctx.positions, ctx.token_slot, out, heads, scale)


def attention_decode_fused(qkv: torch.Tensor, pending, table, rot: int, adjacent: bool, kv: ops.KvView, ctx,
                           out: torch.Tensor, heads: int, scale: float, write_kv: bool, precise: bool = False) -> bool:
    """One kernel for rotation, cache write and attention of a step of single tokens; False when
    the sizes (or the 32-bit model) need the separate kernels, in which case nothing ran."""
    if precise:
        return False
    from . import fast
    return fast.attention_decode_fused(qkv, pending, table, rot, adjacent, kv, ctx, out, heads, scale, write_kv)
